/*
 * CPU oracle for the T0-GPU GEMM hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's own CPU reference
 * arithmetic (clearnature/rust-gpu).  It exists so the CUDA path can be
 * checked against it; the product library never links, loads or calls it.
 * Only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may use it.
 *
 * Parity pin: the GEMM restatement is checked against the reference's
 * committed PyTorch golden vectors (the .bin files under benchmarks/torch_ref/) and against
 * every known-answer pattern the reference's tests hold for this path.  The
 * fused W4A16 GEMM has no counterpart test in the reference ("parity
 * unpinned" for that one op): only its dequant formula, nibble order and wire
 * format are pinned by reference tests.
 */
#ifndef T0_ORACLE_H
#define T0_ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- bf16 conversions ------------------------------------------------- */
/* src/t0/tile_ir.rs:4677 — truncation (upper 16 bits). */
uint16_t oracle_f32_to_bf16_trunc(float v);
/* examples/test_gemm_correctness.rs:15-20 — round to nearest even. */
uint16_t oracle_f32_to_bf16_rne(float v);
/* src/t0/tile_ir.rs:4681 — bits << 16. */
float oracle_bf16_to_f32(uint16_t v);

/* ---- seeded input generators (counter based: element i depends only on
 *      (seed, i), so any sub-range can be regenerated) ------------------- */
uint64_t oracle_splitmix64(uint64_t seed, uint64_t index);
/* uniform [-1,1) rounded (RNE) to bf16 bits */
void oracle_fill_uniform_bf16(uint16_t* out, uint64_t n, uint64_t seed, uint64_t first_index);
/* uniform 32-bit words (eight uniform int4 codes each) */
void oracle_fill_u32(uint32_t* out, uint64_t n, uint64_t seed, uint64_t first_index);
/* uniform (lo,hi) rounded (RNE) to bf16 bits: lo + u*(hi-lo), fp32, no fma */
void oracle_fill_range_bf16(uint16_t* out, uint64_t n, uint64_t seed, uint64_t first_index, float lo, float hi);
/* N(0,1) by Box-Muller on the same stream, rounded (RNE) to bf16 (host only) */
void oracle_fill_normal_bf16(uint16_t* out, uint64_t n, uint64_t seed);

/* ---- GEMM ------------------------------------------------------------- */
/* src/t0/tile_ir.rs:5021-5038 (same body: src/t0/test_tile_gemm_suite.rs:26-35,
 * src/t0/tile_boundary_tests.rs:27-39, examples/test_gemm_correctness.rs:28-42):
 * y[i,j] = sum_k f32(x[i,k]) * f32(wt[j,k]), fp32 multiply, fp32 sequential
 * accumulation with k ascending.  Rows [row_begin,row_end) only; y is the
 * full [m,n] array (row stride n).  threads<=0 picks all host cores. */
void oracle_gemm_nt_bf16_rows(const uint16_t* x, const uint16_t* wt, float* y,
                              uint32_t m, uint32_t k, uint32_t n,
                              uint32_t row_begin, uint32_t row_end, int threads);
void oracle_gemm_nt_bf16(const uint16_t* x, const uint16_t* wt, float* y,
                         uint32_t m, uint32_t k, uint32_t n, int threads);
/* same sum with B given as [K,N] row-major (GemmTranspose::NN, gemm_gen.rs:27) */
void oracle_gemm_nn_bf16(const uint16_t* x, const uint16_t* b, float* y,
                         uint32_t m, uint32_t k, uint32_t n, int threads);
/* float64 accumulation, to separate GPU error from the oracle's own fp32
 * rounding in borderline cases (not a parity target) */
void oracle_gemm_nt_bf16_f64(const uint16_t* x, const uint16_t* wt, double* y,
                             uint32_t m, uint32_t k, uint32_t n, int threads);
/* split-K: plane s holds the fp32 partial over k in [s*K/split,(s+1)*K/split)
 * (gemm_gen.rs:447-448); y_sum (may be NULL) is the fp32 sum of planes in
 * split order (examples/test_gemm_correctness.rs:203-207). */
void oracle_gemm_nt_bf16_splitk(const uint16_t* x, const uint16_t* wt, float* planes, float* y_sum,
                                uint32_t m, uint32_t k, uint32_t n, uint32_t split_k, int threads);
/* bf16 output variant: RNE of the fp32 accumulator */
void oracle_f32_to_bf16_rne_array(const float* in, uint16_t* out, uint64_t n);

/* ---- epilogues -------------------------------------------------------- */
/* gemm_gen.rs:40-49: mode 1 = acc + bias[col]; mode 2 = max(acc + bias[col], 0) */
void oracle_epilogue_gemm_gen(float* y, const float* bias, uint32_t m, uint32_t n, int mode);
/* tile_ir.rs:41-62,3406-3533: op codes 0 BiasAdd, 1 Scale, 2 ReLU, 3 SiLU,
 * 4 GELU (x*sigmoid(1.702x)), 5 Abs, 6 Neg, 7 Clamp, applied in order.
 * SiLU/GELU follow the instruction sequence: exp2(-x*log2e), +1, reciprocal, multiply. */
void oracle_epilogue_tile(float* y, uint32_t m, uint32_t n, const int* ops, int n_ops,
                          const float* bias, float scale, float clamp_min, float clamp_max);

/* ---- INT4 ------------------------------------------------------------- */
/* src/t0/quant_kernels.rs:5-9,74-100: reference wire format.  packed: 2 codes
 * per byte (low nibble = even element), scales f32 and zero points i32 indexed
 * by flat_element >> group_log2; out[e] = f32(code - zp) * scale. */
void oracle_dequant_int4_ref_f32(const uint8_t* packed, const float* scales, const int32_t* zps,
                                 float* out, uint32_t rows, uint32_t cols, uint32_t group_log2);
/* quant_kernels.rs:114-116,167-168: same, stored as truncated bf16 */
void oracle_dequant_int4_ref_bf16(const uint8_t* packed, const float* scales, const int32_t* zps,
                                  uint16_t* out, uint32_t rows, uint32_t cols, uint32_t group_log2);
/* B200 layout: codes packed 8 per u32 along K (packed[K/8][N], code k%8 in
 * bits 4*(k%8)), scales bf16 [K/G][N], zero points uint4 packed 8 per u32
 * along N (zeros[K/G][N/8], column n%8 in bits 4*(n%8));
 * w[k,n] = RNE_bf16( f32(q - z) * f32(s) ). */
void oracle_dequant_w4_b200(const uint32_t* packed, const uint16_t* scales, const uint32_t* zeros,
                            uint16_t* w_out, uint32_t K, uint32_t N, uint32_t group);
/* Streaming (tile-major) layout of the B200 W4A16 kernel: sizes/offsets and the repack itself. */
size_t oracle_w4_prepacked_layout(uint32_t K, uint32_t N, uint32_t group, size_t off[3]);
void oracle_w4_prepack(const uint32_t* packed, const uint16_t* scales, const uint32_t* zeros,
                       uint8_t* out, uint32_t K, uint32_t N, uint32_t group);
/* y[m,n] = sum_k f32(a[m,k]) * f32(w[k,n]) with w from oracle_dequant_w4_b200,
 * fp32 sequential accumulation, k ascending */
void oracle_w4a16_gemm(const uint16_t* a, const uint32_t* packed, const uint16_t* scales,
                       const uint32_t* zeros, float* y,
                       uint32_t M, uint32_t N, uint32_t K, uint32_t group, int threads);
/* quant_kernels.rs:242-286 wire format: header rows,cols,group (u32 LE), packed,
 * scales f32, zero points i32.  Returns 0 and fills the offsets, or -1 when the
 * blob is shorter than the header says. */
int oracle_gptq_parse(const uint8_t* raw, size_t len, uint32_t* rows, uint32_t* cols, uint32_t* group,
                      size_t* packed_off, size_t* scales_off, size_t* zps_off);
/* reference container (rows = output features N, cols = input features K) ->
 * B200 layout; scales are rounded RNE to bf16.  Returns the number of scales
 * that were not exactly representable, or -1 if a zero point is outside 0..15. */
long oracle_gptq_to_b200(const uint8_t* packed, const float* scales, const int32_t* zps,
                         uint32_t rows, uint32_t cols, uint32_t group,
                         uint32_t* packed_out, uint16_t* scales_out, uint32_t* zeros_out);

int oracle_host_threads(void);

#ifdef __cplusplus
}
#endif
#endif

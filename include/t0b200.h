/*
 * t0b200 — B200 (sm_100a) implementation of the T0-GPU GEMM hot path behind a C ABI.
 *
 * Every entry point is what a foreign-function binding in the reference
 * (clearnature/rust-gpu, crate t0-gpu) would bind for this path; the comment
 * above each one cites the Rust item it replaces (paths relative to that tree).
 *
 * Conventions
 *   - every fallible call returns int: 0 = OK, non-zero = error code below;
 *     the message is available from t0_last_error() (thread-local).  A Rust
 *     `panic!`/`assert!` in the reference becomes T0_ERR_INVALID here.
 *   - handles are opaque pointers owned by the caller until the matching free.
 *   - plain pointers and sizes only; device addresses travel as uint64_t
 *     exactly as the reference carries them in its kernarg blobs.
 *   - there is no CPU fallback: compute entry points fail with T0_ERR_CUDA when
 *     no B200-class device is present.
 */
#ifndef T0B200_H
#define T0B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ errors */
enum {
    T0_OK = 0,
    T0_ERR_INVALID = 1,      /* bad argument / a panic in the reference            */
    T0_ERR_CUDA = 2,         /* CUDA runtime or driver call failed                 */
    T0_ERR_POISONED = 3,     /* runtime poisoned by an earlier device failure      */
    T0_ERR_TIMEOUT = 4,      /* a bounded device-side wait expired                 */
    T0_ERR_BOUNDS = 5,       /* buffer too small for the requested operation       */
    T0_ERR_UNSUPPORTED = 6,  /* shape/config this build has no kernel for          */
    T0_ERR_IO = 7            /* tune-cache file problem                            */
};
/* Rust `Result<_, String>` error text of the last failing call on this thread. */
const char* t0_last_error(void);
/* Library/ABI version: major*10000 + minor*100 + patch. */
int t0_version(void);

/* ------------------------------------------------------- GemmConfig (a3) */
/* src/t0/gemm_gen.rs:23-33 GemmTranspose */
enum { T0_NT = 0, T0_NN = 1 };
/* src/t0/gemm_gen.rs:40-49 EpilogueOp */
enum { T0_EPI_STORE_F32 = 0, T0_EPI_BIAS_ADD_STORE_F32 = 1, T0_EPI_BIAS_ADD_RELU_STORE_F32 = 2 };

/* src/t0/gemm_gen.rs:55-84 GemmConfig — same fields, same meaning.  On B200:
 * tile_m/tile_n/tile_k are the CTA tile, wg_size the CTA thread count that
 * compute_grid multiplies by, use_lds/double_buffer select the multi-stage
 * shared-memory pipeline (always on), split_k 0 or 1 means None, wgp_mode
 * selects the two-CTA pair tile, lds_pad and n_col_passes are accepted and
 * ignored (no bank padding / column passes exist on this hardware). */
typedef struct t0_gemm_config {
    uint32_t tile_m, tile_n, tile_k, wg_size;
    uint8_t use_lds, double_buffer;
    uint8_t _pad0[2];
    uint32_t split_k;
    uint32_t lds_pad, n_col_passes;
    uint8_t swap_grid, wgp_mode, transpose, epilogue;
} t0_gemm_config;

/* GemmConfig::tile_16x64_k16() ... tile_64x128_2pass() (gemm_gen.rs:86-145);
 * `preset` is the Rust constructor name, e.g. "tile_128x64_k32". */
int t0_gemm_config_preset(const char* preset, t0_gemm_config* out);
/* GemmConfig::name() (gemm_gen.rs:215-235); writes a NUL-terminated string. */
int t0_gemm_config_name(const t0_gemm_config* cfg, char* buf, size_t buf_len);
/* GemmConfig::estimated_vgprs() (gemm_gen.rs:189-201), kept for callers that print it. */
uint32_t t0_gemm_config_estimated_vgprs(const t0_gemm_config* cfg);
/* GemmConfig::is_feasible() (gemm_gen.rs:203-213): 1 when this library can run the config. */
int t0_gemm_config_is_feasible(const t0_gemm_config* cfg);
/* GemmConfig::lds_total() (gemm_gen.rs:168-170): shared memory of the B200 pipeline for this config. */
uint32_t t0_gemm_config_lds_total(const t0_gemm_config* cfg);
/* sweep_configs() / standard_configs() (gemm_gen.rs:239-251,407-427): fills up
 * to `cap` entries, returns the total count. */
int t0_sweep_configs(t0_gemm_config* out, int cap);
int t0_standard_configs(t0_gemm_config* out, int cap);

/* ------------------------------------------------- selection (a6, a7, a8) */
/* auto_select(m, k, n) (gemm_gen.rs:340-342 -> cost_model.rs:660-668). Argument order (m, k, n).
 * Environment: T0_FORCE_CFG=<preset name> (a GemmConfig constructor name such as tile_128x64_k32, optionally followed by
 * ":sk<N>" for split-K) makes auto_select and cached_auto_select return that config for every shape - an A/B and
 * debugging switch of the same family as the reference's T0_* ablation variables (gpu_context.rs:327,335). */
int t0_auto_select(uint32_t m, uint32_t k, uint32_t n, t0_gemm_config* out);
/* auto_select_legacy(m, k, n) (gemm_gen.rs:351-404): the hand-tuned table, verbatim semantics. */
int t0_auto_select_legacy(uint32_t m, uint32_t k, uint32_t n, t0_gemm_config* out);
/* auto_select_backward_data / _weight (gemm_gen.rs:510-549) */
int t0_auto_select_backward_data(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0_gemm_config* out);
int t0_auto_select_backward_weight(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0_gemm_config* out);
/* cost_model::auto_schedule_gemm (cost_model.rs:464-534): ranked candidates for
 * (m, n, k) with their predicted TFLOP/s; returns the number written (<= cap). */
int t0_auto_schedule_gemm(uint32_t m, uint32_t n, uint32_t k, t0_gemm_config* out, double* pred_tflops, int cap);
/* prefill_spec_cache (prefill_spec_cache.rs:55-76,79-113,125-138) */
int t0_cached_auto_select(uint32_t m, uint32_t k, uint32_t n, t0_gemm_config* out);
int t0_cached_auto_select_backward_data(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0_gemm_config* out);
int t0_cached_auto_select_backward_weight(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0_gemm_config* out);
int t0_prewarm_cache(const uint32_t* mkn_triples, size_t n_triples);
void t0_clear_cache(void);
size_t t0_cache_size(void);

/* ------------------------------------------------------- grids (a5) */
/* compute_grid / compute_grid_split_k / compute_grid_auto (gemm_gen.rs:308-329,430-437):
 * grid in THREADS: swap_grid ? (tiles_n*wg_size, tiles_m[*sk]) : (tiles_m*wg_size, tiles_n[*sk]). */
int t0_compute_grid(const t0_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t* gx, uint32_t* gy);
int t0_compute_grid_split_k(const t0_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t split_k, uint32_t* gx, uint32_t* gy);
int t0_compute_grid_auto(const t0_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t* gx, uint32_t* gy);
/* compute_grid_backward_data / _weight (gemm_gen.rs:533-536,567-570) */
int t0_compute_grid_backward_data(const t0_gemm_config* cfg, uint32_t m, uint32_t k_orig, uint32_t* gx, uint32_t* gy);
int t0_compute_grid_backward_weight(const t0_gemm_config* cfg, uint32_t n_orig, uint32_t k_orig, uint32_t* gx, uint32_t* gy);

/* ------------------------------------------------------- kernargs (a9) */
/* build_kernargs(x, wt, y, k, n, m, cfg) -> [u8;40] (gemm_gen.rs:442-458). Argument order kept. */
int t0_build_kernargs(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                      const t0_gemm_config* cfg, uint8_t out[40]);
/* build_kernargs_with_bias(..., bias) -> [u8;48] (gemm_gen.rs:466-484) */
int t0_build_kernargs_with_bias(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                const t0_gemm_config* cfg, uint64_t bias, uint8_t out[48]);
/* build_kernargs_backward_data / _weight (gemm_gen.rs:523-530,557-564) */
int t0_build_kernargs_backward_data(uint64_t dy, uint64_t w, uint64_t dx, uint32_t m, uint32_t n_orig, uint32_t k_orig,
                                    const t0_gemm_config* cfg, uint8_t out[40]);
int t0_build_kernargs_backward_weight(uint64_t dy_t, uint64_t x_t, uint64_t dw, uint32_t m, uint32_t n_orig, uint32_t k_orig,
                                      const t0_gemm_config* cfg, uint8_t out[40]);

/* ------------------------------------------------------- TileGemm (a11, a13) */
/* src/t0/tile_ir.rs:41-62 EpilogueOp (TileIR chain) */
enum { T0_TEPI_BIAS_ADD = 0, T0_TEPI_SCALE = 1, T0_TEPI_RELU = 2, T0_TEPI_SILU = 3,
       T0_TEPI_GELU = 4, T0_TEPI_ABS = 5, T0_TEPI_NEG = 6, T0_TEPI_CLAMP = 7 };
#define T0_TILE_MAX_EPILOGUE 8
/* src/t0/tile_ir.rs:109-152 TileGemm.  waves_per_wg 0 = None; wmma_format 0 = BF16_F32
 * (the only format this library computes). */
typedef struct t0_tile_gemm {
    uint32_t tile_m, tile_n, tile_k;
    uint8_t wgp_mode, double_buffer, triple_buffer, swap_grid;
    uint32_t split_k;
    uint8_t transpose, acc_swap, persistent, n_epilogue;
    uint8_t epilogue[T0_TILE_MAX_EPILOGUE];
    uint32_t waves_per_wg;
    uint32_t wmma_format;
} t0_tile_gemm;
/* TileGemm::tile_128x64_k16() ... (tile_ir.rs:156-604); `preset` is the Rust constructor name. */
int t0_tile_gemm_preset(const char* preset, t0_tile_gemm* out);
/* TileGemm::name() (tile_ir.rs:677-701) */
int t0_tile_gemm_name(const t0_tile_gemm* spec, char* buf, size_t buf_len);
/* TileGemm::wg_size() / lds_total() (tile_ir.rs:607-651) — the reference's arithmetic, kept for grid maths */
uint32_t t0_tile_gemm_wg_size(const t0_tile_gemm* spec);
uint32_t t0_tile_gemm_lds_total(const t0_tile_gemm* spec);
/* tile_auto_select(m, k, n, transpose) (tile_ir.rs:740-870) */
int t0_tile_auto_select(uint32_t m, uint32_t k, uint32_t n, int transpose, t0_tile_gemm* out);
/* tile_ir::build_kernargs_m (tile_ir.rs:4595-4634): 44 bytes (64 in persistent mode);
 * returns the length through out_len.  Extra epilogue arguments are appended in the
 * order bias u64, scale f32, clamp_min f32, clamp_max f32 when the chain uses them
 * (tile_ir.rs:1015-1026). */
int t0_tile_build_kernargs_m(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                             const t0_tile_gemm* spec, uint8_t* out, size_t cap, size_t* out_len);
int t0_tile_build_kernargs_epilogue(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                    const t0_tile_gemm* spec, uint64_t bias, float scale, float clamp_min, float clamp_max,
                                    uint8_t* out, size_t cap, size_t* out_len);
/* tile_ir::compute_grid(&spec, m, n) -> [u32;3] (tile_ir.rs:4645-4665) */
int t0_tile_compute_grid(const t0_tile_gemm* spec, uint32_t m, uint32_t n, uint32_t grid[3]);
/* tile_ir::f32_to_bf16 (truncate) / bf16_to_f32 (tile_ir.rs:4677-4683) */
uint16_t t0_f32_to_bf16(float v);
float t0_bf16_to_f32(uint16_t v);

/* ------------------------------------------------------- runtime (a17) */
typedef struct t0_runtime t0_runtime;   /* GpuRuntime   src/ignis/gpu_context.rs:99-119 */
typedef struct t0_buffer t0_buffer;     /* GpuBuffer    src/kfd/buffer.rs:9-123        */
typedef struct t0_kernel t0_kernel;     /* GpuKernel    src/kfd/kernel.rs:8-19         */

/* GpuRuntime::new() (gpu_context.rs:151-171): one CUDA stream (the in-order AQL queue), a buffer pool, a kernel cache. */
int t0_rt_new(int device, t0_runtime** out);
void t0_rt_free(t0_runtime* rt);
/* is_poisoned / mark_poisoned (gpu_context.rs:190-198) */
int t0_rt_is_poisoned(const t0_runtime* rt);
void t0_rt_mark_poisoned(t0_runtime* rt);
/* queue.synchronize() / wait_idle() (src/kfd/aql.rs:473): drain the stream; a device-side failure poisons the runtime. */
int t0_rt_synchronize(t0_runtime* rt);
int t0_rt_wait_idle(t0_runtime* rt);
/* The wait limit of AqlQueue::wait_read_ptr (src/kfd/aql.rs:529-549: the reference gives up on a dispatch after a fixed time,
 * returns Err and the runtime is poisoned, gpu_context.rs:352-355).  Here the limit applies to every single barrier wait
 * inside a GEMM kernel (default 2 s; 0 restores the default): a wait that runs out makes the kernel unwind, release its tensor
 * memory and write a status word; the next synchronising call returns T0_ERR_TIMEOUT and poisons the runtime. */
int t0_rt_set_wait_limit_ns(t0_runtime* rt, uint64_t ns);
/* Self-test of that path (no counterpart in the reference): the NEXT GEMM launch of this runtime leaves out the first
 * operand load of its first tile, so that tile's accumulate wait runs out after the wait limit.  Nothing faults and the
 * kernel returns by itself; the call that synchronises reports T0_ERR_TIMEOUT, the runtime is poisoned, the output of
 * that launch is incomplete.  Set a short limit first (milliseconds).  For tests of the error handling only. */
int t0_rt_selftest_drop_one_load(t0_runtime* rt);
/* Scratch buffers (no counterpart in the reference, whose dispatch paths allocate per call).  Some launch paths keep a
 * per-runtime device buffer that grows on first use at each larger size: growing drains the stream, frees and allocates,
 * so the first such call stalls a pipeline and is illegal inside a stream capture.  The paths and their buffers:
 *   t0_gemm_launch / t0_gemm_batch / t0_gemm_submit with a K that is not a multiple of 8 (or N in the NN layout) or an
 *     operand that is not 16-byte aligned: padded copies of the operands, T0_SCRATCH_OPERAND_A = M * roundup(K, 8) * 2 bytes, T0_SCRATCH_OPERAND_B = N * roundup(K, 8) * 2
 *     (NT) or K * roundup(N, 8) * 2 (NN);
 *   split_k > 1 where the one-launch cluster form does not apply (pair tiles, padded operands, bf16 partial planes):
 *     T0_SCRATCH_SPLITK_PLANES = M * N * split_k * 4;
 *   t0_w4a16_gemm outside the fused shapes: T0_SCRATCH_W4_WEIGHTS = K * N * 2;
 *   every fused W4A16 call (row layout and streaming layout): T0_SCRATCH_W4_FUSED, t0_rt_w4_fused_scratch_bytes(rt) bytes,
 *     a fixed size per device, so only the first fused call of a runtime allocates;
 *   t0_matmul_f32*, t0_blas_gemm_f32: bf16 copies of the operands, T0_SCRATCH_F32_A / _B = elements * 2, and, for
 *     alpha/beta other than 1/0 or ldc != n, T0_SCRATCH_F32_C = m * n * 4;
 *   t0_gemm_host and the multi-GPU host entry: pinned staging sets and device operands made on first use per shape.
 * Everything else (aligned shapes of the bf16 GEMM, the cluster split-K, t0_w4a16_gemm_static) never allocates.
 * t0_rt_reserve_scratch grows one buffer to at least `bytes` ahead of time, so that later launches up to that size
 * neither allocate nor synchronise. */
enum {
    T0_SCRATCH_OPERAND_A = 0, T0_SCRATCH_OPERAND_B = 1, T0_SCRATCH_SPLITK_PLANES = 2, T0_SCRATCH_W4_WEIGHTS = 3,
    T0_SCRATCH_W4_FUSED = 4, T0_SCRATCH_F32_A = 5, T0_SCRATCH_F32_B = 6, T0_SCRATCH_F32_C = 7
};
int t0_rt_reserve_scratch(t0_runtime* rt, int which, size_t bytes);
size_t t0_rt_w4_fused_scratch_bytes(const t0_runtime* rt);
/* the CUDA stream handle (cudaStream_t) and device ordinal, for callers that time or order work themselves */
void* t0_rt_stream(const t0_runtime* rt);
int t0_rt_device(const t0_runtime* rt);
int t0_rt_sm_count(const t0_runtime* rt);

/* rt.alloc / alloc_zero / alloc_f32 / recycle (gpu_context.rs:508-530) with BufferPool semantics
 * (gpu_context.rs:31-92): sizes rounded to 4 KiB, recycled buffers are zeroed on hand-out. */
int t0_rt_alloc(t0_runtime* rt, size_t n_bytes, t0_buffer** out);
int t0_rt_alloc_zero(t0_runtime* rt, size_t n_bytes, t0_buffer** out);
int t0_rt_alloc_f32(t0_runtime* rt, size_t n_elems, t0_buffer** out);
void t0_rt_recycle(t0_runtime* rt, t0_buffer* buf);
size_t t0_rt_pool_cached_bytes(const t0_runtime* rt);
void t0_rt_pool_clear(t0_runtime* rt);
/* read_f32 / write_f32 / upload_f32 (gpu_context.rs:535-558) */
int t0_rt_read_f32(t0_runtime* rt, const t0_buffer* buf, size_t n, float* out);
int t0_rt_write_f32(t0_runtime* rt, t0_buffer* buf, const float* data, size_t n);
int t0_rt_upload_f32(t0_runtime* rt, const float* data, size_t n, t0_buffer** out);

/* GpuBuffer::{write, read, write_bytes, read_bytes, zero, gpu_addr, size} (src/kfd/buffer.rs:23-109), bounds-checked;
 * Drop (buffer.rs:125-146) = t0_buf_free. */
int t0_buf_write(t0_buffer* buf, const void* data, size_t len);
int t0_buf_read(const t0_buffer* buf, void* out, size_t len);
int t0_buf_write_bytes(t0_buffer* buf, size_t offset, const void* data, size_t len);
int t0_buf_read_bytes(const t0_buffer* buf, size_t offset, void* out, size_t len);
int t0_buf_zero(t0_buffer* buf);
uint64_t t0_buf_gpu_addr(const t0_buffer* buf);
size_t t0_buf_size(const t0_buffer* buf);
void t0_buf_free(t0_buffer* buf);

/* generate(&cfg) + rt.ensure_kernel_t0(name, builder, wg, lds) (gemm_gen.rs:261-297, gpu_context.rs:212-259):
 * looks up the precompiled sm_100a kernel for the config, cached by cfg.name(). */
int t0_rt_ensure_gemm_kernel(t0_runtime* rt, const t0_gemm_config* cfg, t0_kernel** out);
/* lower_gemm(&spec) + ensure_kernel_t0 (tile_ir.rs:887, gpu_context.rs:212) */
int t0_rt_ensure_tile_kernel(t0_runtime* rt, const t0_tile_gemm* spec, t0_kernel** out);
/* GpuKernel.kernarg_size (src/kfd/kernel.rs:8-19) and the cache key */
uint32_t t0_kernel_kernarg_size(const t0_kernel* k);
const char* t0_kernel_name(const t0_kernel* k);
size_t t0_rt_kernel_cache_size(const t0_runtime* rt);

/* rt.dispatch(&kernel, grid, kernargs) (gpu_context.rs:305-356): submit + wait; checks poison, asserts
 * kernargs.len() == kernel.kernarg_size, decodes the blob, validates every pointer against the live
 * allocations of this runtime, launches, waits; a device failure poisons the runtime.
 * The 40/48-byte gemm_gen blob carries no M: M = tiles_m * tile_m is taken from the grid, as the
 * reference kernel implicitly does (every row of every launched tile is written). */
int t0_rt_dispatch(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* kernargs, size_t len);
/* dispatch_async (gpu_context.rs:400-410): submit only; slot index through out_slot (may be NULL) */
int t0_rt_dispatch_async(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* kernargs, size_t len, size_t* out_slot);
/* dispatch_bench (gpu_context.rs:363-374): submit + wait without validation */
int t0_rt_dispatch_bench(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* kernargs, size_t len);
/* prefill_dispatch::DispatchQueue::{submit, flush} (src/t0/prefill_dispatch.rs:61-206): fire-and-forget submits that only
 * check the poison flag, then one wait.  The stream is the queue, so a "queue" is the runtime itself. */
int t0_rt_submit(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* kernargs, size_t len);
int t0_rt_flush(t0_runtime* rt);
/* number of kernels this runtime has launched (all kinds) since creation */
uint64_t t0_rt_launch_count(const t0_runtime* rt);
/* Tracing aid (the reference reads SHADER_CYCLES for the same purpose, src/t0/ir.rs:571): CTA 0 of every GEMM kernel
 * stamps the SM cycle counter and the nanosecond timer at entry and exit.  Returns the SM clock (MHz) the last GEMM kernel
 * actually ran at and, optionally, that CTA's lifetime in microseconds.  Waits for the stream. */
int t0_rt_last_kernel_clock(t0_runtime* rt, double* sm_mhz, double* kernel_us);
/* CUDA-event stopwatch on the runtime's stream: start records an event, stop records another, waits and returns ms */
int t0_rt_timer_start(t0_runtime* rt);
int t0_rt_timer_stop(t0_runtime* rt, float* ms);

/* ------------------------------------------------------- direct GEMM entry */
/* The launch that generate()+dispatch() amounts to, with explicit arguments instead of a kernarg blob.
 * y[M,N] (f32, or bf16 when out_bf16) = x[M,K] (bf16) * op(b): transpose T0_NT: b is [N,K]; T0_NN: b is [K,N].
 * split_k > 1 with planes != 0 writes split_k f32 planes of M*N (gemm_gen.rs:447-448); with planes == 0 the
 * partial sums are reduced on the device in split order into y.  epilogue as t0_gemm_config.epilogue.
 * A request that leaves tile_n, split_k, pair_cta and planes all 0 is scheduled by the cost model (t0_cached_auto_select):
 * tile, CTA pair or not, and possibly split-K with the device-side reduction; the result in y is complete either way. */
typedef struct t0_gemm_args {
    uint64_t x, b, y, bias;
    uint32_t m, n, k;
    uint32_t tile_n;        /* 0 = choose; else 32/64/128/256 */
    uint32_t split_k;       /* 0/1 = none */
    uint8_t transpose, epilogue, out_bf16, planes;
    uint8_t swap_grid;
    uint8_t pair_cta;       /* 0 = choose by shape, 1 = two-CTA pair kernel (256 x 256 tiles; 256 x 128 for NT with tile_n <= 128), 2 = single-CTA kernel */
    uint8_t _pad[2];
    /* TileIR epilogue chain (used when n_tile_epilogue > 0; epilogue above is then ignored) */
    uint8_t n_tile_epilogue;
    uint8_t tile_epilogue[T0_TILE_MAX_EPILOGUE];
    uint8_t _pad2[3];
    float scale, clamp_min, clamp_max;
} t0_gemm_args;
int t0_gemm_launch(t0_runtime* rt, const t0_gemm_args* args);
/* `count` launches from an array, submitted back to back from native code (the batch form of the above; the reference's
 * timing loops submit N dispatches and wait once, src/t0/tile_ir.rs:5704-5717). */
int t0_gemm_launch_batch(t0_runtime* rt, const t0_gemm_args* args, size_t count);
/* Several independent GEMMs in ONE launch (the reference's nearest item is DispatchQueue::submit / flush, src/kfd/aql.rs, which
 * batches independent dispatches behind one doorbell).  Where all the problems have one shape and one configuration and that
 * configuration is the one-launch split-K (the skinny shapes: the CTAs of a tile form a cluster), the clusters of a single
 * persistent launch walk the tiles of all the problems (up to 32 per launch): launch, prologue and drain are paid once and
 * the exchange of one tile overlaps the main loop of the next.  With tile_n and split_k given, every y is the same, bit for
 * bit, as from t0_gemm_launch with those values.  With both left at 0 the split is chosen for the group, not for one
 * problem: several skinny problems fill the GPU with fewer splits (often none, which then runs the plain kernel over all the
 * problems' tiles), so y agrees with t0_gemm_launch to rounding (another order of the fp32 sums along K), not bit for bit.
 * The problems run at the same time, so no y may overlap an operand or the y of another problem: that is checked
 * (T0_ERR_INVALID).  Other shapes (NN layout, CTA-pair tiles), or problems that differ, are launched back to back as by
 * t0_gemm_launch_batch. */
int t0_gemm_launch_grouped(t0_runtime* rt, const t0_gemm_args* args, size_t count);
/* GEMM with a gathered output (no counterpart in the reference, which is single-GPU; it is the compute step and the
 * all-gather of the sharded GEMM in one kernel).  The product goes to args->y and, in the same epilogue, to n_peers further
 * f32 [M,N] buffers (at most 7), normally slot `rank` of the other GPUs' rank-major result C_g[g][M][N/g]: the epilogue
 * issues one TMA store per destination for every 32 x 32 block, so the blocks cross NVLink while the main loop runs.
 * peer_y[i] are device addresses valid in this process: memory of a GPU with peer access enabled, or a mapping opened with
 * t0_rt_ipc_open.  Needs N % 32 == 0, 16-byte aligned destinations, f32 output, no split-K (T0_ERR_UNSUPPORTED otherwise).
 * The stores are complete when the launch is: order readers on the other GPUs after it (an event, a barrier). */
int t0_gemm_launch_gather(t0_runtime* rt, const t0_gemm_args* args, const uint64_t* peer_y, uint32_t n_peers);
/* Sharing a buffer with another process on the same machine (one process per GPU): t0_buf_ipc_export writes the 64-byte
 * handle of the buffer's allocation, t0_rt_ipc_open maps it into this process (peer access over NVLink) and returns the
 * device address of the allocation's start, t0_rt_ipc_close drains the runtime's stream and unmaps it. */
int t0_buf_ipc_export(const t0_buffer* buf, uint8_t handle[64]);
int t0_rt_ipc_open(t0_runtime* rt, const uint8_t handle[64], uint64_t* device_ptr);
int t0_rt_ipc_close(t0_runtime* rt, uint64_t device_ptr);
/* The same launches with x, b, y (and bias) as HOST addresses: operands are uploaded, the product is computed and the
 * result is downloaded, and consecutive problems overlap - problem i+1 crosses the link while problem i is computed and
 * read back (three queues, two staging sets on the device).  This is the upload / dispatch / read-back sequence of the
 * reference's host-facing GEMM calls (T0BlasLib::gemm, src/universal/math/blas.rs:18-100; dispatch_gemm_forward,
 * src/ignis/ops/bf16_matmul.rs:61-190) for an array of problems.  x is bf16 [m][k]; b is bf16 [n][k] (NT) or [k][n] (NN);
 * y is f32 (or bf16 with out_bf16) [m][n]; bias f32 [n]; `planes` must be 0.  Returns when every result is in host memory.
 * Page-locked host memory is needed for the copies to overlap. */
int t0_gemm_launch_host_batch(t0_runtime* rt, const t0_gemm_args* args, size_t count);
int t0_gemm_launch_host(t0_runtime* rt, const t0_gemm_args* args);

/* ------------------------------------------------------- cost-model records */
/* TileConfig (src/t0/cost_model.rs:130-168) and TileCost (:171-190): the cost model's own candidate record and its
 * estimate.  On B200 `waves_per_wg` counts the CTA's warps (6: producer, UMMA issuer, four epilogue warps),
 * `vgprs` / `sgprs` / `occupancy` report registers per thread, 0 and resident CTAs per SM, `lds_bytes` the dynamic
 * shared memory of the kernel instance, `score` the predicted TFLOP/s. */
typedef struct t0_tile_config {
    uint32_t tile_m, tile_n, tile_k, waves_per_wg;
    uint8_t use_lds, wgp_mode, swap_grid, _pad;
    uint32_t split_k;        /* 1 = no split */
    uint32_t lds_pad;
} t0_tile_config;
typedef struct t0_tile_cost {
    t0_tile_config config;
    uint32_t vgprs, sgprs, lds_bytes, occupancy, n_wgs;
    int feasible;
    double score;
    char bottleneck[24];
} t0_tile_cost;
/* auto_schedule_gemm(m, n, k, fmt) -> Vec<TileCost>, best first (cost_model.rs:464-534); returns how many were written */
int t0_auto_schedule_tile_costs(uint32_t m, uint32_t n, uint32_t k, t0_tile_cost* out, int cap);
/* TileConfig::name / to_gemm_config / to_tile_gemm / can_use_tile_ir (cost_model.rs:157-163,578-647).  to_gemm_config keeps
 * the tile width (no 64-column passes: that was a register-file workaround of the reference's target). */
int t0_tile_config_name(const t0_tile_config* c, char* buf, size_t buf_len);
int t0_tile_config_to_gemm_config(const t0_tile_config* c, t0_gemm_config* out);
int t0_tile_config_to_tile_gemm(const t0_tile_config* c, t0_tile_gemm* out);
int t0_tile_config_can_use_tile_ir(const t0_tile_config* c);

/* ------------------------------------------------------- warp-layout planners */
/* WarpLayout / WarpOrientation and the planners (src/t0/tile_ir.rs:8365-8545): pure host arithmetic over a tile shape,
 * kept for callers that size their own kernels with it.  The reference's asserts become T0_ERR_INVALID. */
enum { T0_WARP_ROW_DOMINANT = 0, T0_WARP_COL_DOMINANT = 1, T0_WARP_SQUARE = 2 };
typedef struct t0_warp_layout {
    uint32_t n_warps, rows_per_warp, cols_per_warp;
    uint32_t orientation;     /* T0_WARP_* */
} t0_warp_layout;
int t0_warp_layout_row_dominant(uint32_t n_warps, uint32_t tile_m, uint32_t tile_n, t0_warp_layout* out);   /* :8390-8413 */
int t0_warp_layout_col_dominant(uint32_t n_warps, uint32_t tile_m, uint32_t tile_n, t0_warp_layout* out);   /* :8418-8429 */
int t0_warp_layout_square(uint32_t n_warps, uint32_t tile_m, uint32_t tile_n, t0_warp_layout* out);         /* :8434-8451 */
uint32_t t0_warp_layout_wmma_row_blocks(const t0_warp_layout* l);      /* rows_per_warp / 16 */
uint32_t t0_warp_layout_wmma_col_tiles(const t0_warp_layout* l);       /* cols_per_warp / 16 */
uint32_t t0_warp_layout_wmma_ops_per_warp(const t0_warp_layout* l);
uint32_t t0_warp_layout_acc_vgprs_per_warp(const t0_warp_layout* l);   /* 8 per 16 x 16 output block */
uint32_t t0_warp_layout_wg_size(const t0_warp_layout* l);
int t0_warp_layout_is_compatible(const t0_warp_layout* l, uint32_t tile_m, uint32_t tile_n);
int t0_plan_flash_attention_warps(uint32_t n_warps, uint32_t m, uint32_t n, uint32_t d, t0_warp_layout* qk, t0_warp_layout* av);   /* :8487-8524 */
int t0_plan_single_dot_warps(uint32_t n_warps, uint32_t tile_m, uint32_t tile_n, t0_warp_layout* out);                              /* :8529-8540 */

/* ------------------------------------------------------- f32 framework entries */
/* Ignis matmul(x[M,K] f32, w[K,N] f32) -> y[M,N] f32 (src/ignis/ops/bf16_matmul.rs:33-59,162-207): operands rounded to
 * bf16 (nearest even, :371-372) on the device, fp32 accumulate.  Device pointers; no padding, transposing or host round
 * trips (the reference does all three on the CPU, :356-423).  Argument order (m, k, n) as the reference's helpers. */
int t0_matmul_f32(t0_runtime* rt, uint64_t x, uint64_t w, uint64_t y, uint32_t m, uint32_t k, uint32_t n);
/* matmul_with_wt_bf16 (:93-133): the weight already transposed to [N,K] and in bf16 */
int t0_matmul_f32_with_wt_bf16(t0_runtime* rt, uint64_t x, uint64_t wt_bf16, uint64_t y, uint32_t m, uint32_t k, uint32_t n);
/* gemm_backward_data (:216-262): dX[M,K] = dY[M,N] * W[K,N]^T;  gemm_backward_weight (:264-312): dW[K,N] = X[M,K]^T * dY[M,N] */
int t0_matmul_f32_backward_data(t0_runtime* rt, uint64_t dy, uint64_t w, uint64_t dx, uint32_t m, uint32_t k, uint32_t n);
int t0_matmul_f32_backward_weight(t0_runtime* rt, uint64_t x, uint64_t dy, uint64_t dw, uint32_t m, uint32_t k, uint32_t n);
/* BlasLib::gemm / gemv for DType::F32 (src/universal/math/mod.rs:24-47; CPU body math/blas.rs:18-100):
 * C[m,n] = alpha * A[m,k] * B[k,n] + beta * C, row-major with leading dimensions; y = alpha * A[m,n] * x + beta * y.
 * gemm multiplies on the bf16 tensor path (inputs rounded to bf16, fp32 accumulate: the GEMM tolerance applies, where the
 * reference's CPU body is exact f32); gemv is f32 throughout.  beta == 0 does not read C / y. */
int t0_blas_gemm_f32(t0_runtime* rt, uint32_t m, uint32_t n, uint32_t k, float alpha, uint64_t a, uint32_t lda, uint64_t b, uint32_t ldb,
                     float beta, uint64_t c, uint32_t ldc);
int t0_blas_gemv_f32(t0_runtime* rt, uint32_t m, uint32_t n, float alpha, uint64_t a, uint32_t lda, uint64_t x, uint32_t incx, float beta,
                     uint64_t y, uint32_t incy);

/* ------------------------------------------------------- autotuner (a10) */
typedef struct t0_tuner t0_tuner;   /* GemmTuner  src/t0/auto_gemm.rs:46-55 */
/* GemmTuner::new() / with_cache_dir(dir) (auto_gemm.rs:59-75).  Default directory: $T0_TUNE_DIR, else
 * ~/.t0_autotune/b200_sm100a (the reference uses ~/.t0_autotune; the sub-directory keeps other hardware's results apart). */
int t0_tuner_new(t0_tuner** out);
int t0_tuner_with_cache_dir(const char* dir, t0_tuner** out);
void t0_tuner_free(t0_tuner* t);
/* the public fields max_candidates (8) and n_iters (5) (auto_gemm.rs:52-54); 0 leaves a field unchanged */
int t0_tuner_configure(t0_tuner* t, size_t max_candidates, size_t n_iters);
size_t t0_tuner_max_candidates(const t0_tuner* t);
size_t t0_tuner_n_iters(const t0_tuner* t);
size_t t0_tuner_cache_len(const t0_tuner* t);
const char* t0_tuner_cache_dir(const t0_tuner* t);
/* GemmTuner::tune(rt, m, n, k) -> GemmConfig (auto_gemm.rs:82-216): memory cache, disk cache gemm_{M}x{N}x{K}.json,
 * else cost-model candidates -> 256^3 smoke test -> timed runs (median of n_iters) -> save.  Argument order (m, n, k). */
int t0_tuner_tune(t0_tuner* t, t0_runtime* rt, uint32_t m, uint32_t n, uint32_t k, t0_gemm_config* out);
/* GemmTuner::benchmark_tile_ir (auto_gemm.rs:352-431): times one TileGemm spec through the TileIR dispatch path */
int t0_tuner_benchmark_tile_ir(t0_tuner* t, t0_runtime* rt, const t0_tile_gemm* spec, uint32_t m, uint32_t n, uint32_t k, double* tflops);
/* GemmTuneResult of a tuned size (auto_gemm.rs:30-41): best TFLOP/s, whether it came from disk, how many candidates were timed */
int t0_tuner_result(const t0_tuner* t, uint32_t m, uint32_t n, uint32_t k, double* best_tflops, int* from_cache, int* n_measured);
/* save_cache / load_cache (auto_gemm.rs:439-501) and the JSON field reader (:603-625), exposed as the reference's tests use them */
int t0_tuner_save_cache(t0_tuner* t, uint32_t m, uint32_t n, uint32_t k, const t0_gemm_config* best, double best_tflops);
int t0_tuner_load_cache(t0_tuner* t, uint32_t m, uint32_t n, uint32_t k, t0_gemm_config* best, double* best_tflops);
int t0_parse_json_number(const char* json, const char* key, double* out);
/* invalidate / clear / report (auto_gemm.rs:504-531) */
void t0_tuner_invalidate(t0_tuner* t, uint32_t m, uint32_t n, uint32_t k);
void t0_tuner_clear(t0_tuner* t);
void t0_tuner_report(const t0_tuner* t);
/* global_tuner() (auto_gemm.rs:539) and the one-shot auto_gemm(rt, a, b, c, m, n, k) -> Result<f64> (auto_gemm.rs:555-590):
 * tune or cache hit, then dispatch with the best config; returns the tuned TFLOP/s through `tflops`.
 * c always receives the complete product in its first m*n floats: a split-K winner is launched with the
 * device-side reduction instead of leaving partial planes for the host to add. */
t0_tuner* t0_global_tuner(void);
int t0_auto_gemm(t0_runtime* rt, t0_buffer* a, t0_buffer* b, t0_buffer* c, uint32_t m, uint32_t n, uint32_t k, double* tflops);

/* ------------------------------------------------------- INT4 weights (a14, a15) */
/* build_dequant_int4_f32 / _bf16 (src/t0/quant_kernels.rs:53-171) in the reference wire format: packed = two codes per byte,
 * low nibble first (:5-9); scales f32 and zero points i32 indexed by flat_element >> group_size_log2;
 * out[e] = f32(code - zp) * scale, stored as f32 or as truncated bf16 (:167-168).  rows*cols elements. */
int t0_dequant_int4(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zero_points, uint64_t out, uint32_t rows, uint32_t cols,
                    uint32_t group_size_log2, int out_bf16);
/* The same two kernels as dispatchable objects with the reference's 40-byte kernarg blob
 * [packed, scales, zero_points, output: u64 x 4, rows, cols: u32 x 2] (quant_kernels.rs:45-47). */
int t0_rt_ensure_dequant_kernel(t0_runtime* rt, uint32_t group_size_log2, int out_bf16, t0_kernel** out);
/* B200 weight layout: codes packed eight per u32 along K (packed[K/8][N], code k%8 in bits 4*(k%8)), bf16 scales [K/G][N],
 * uint4 zero points packed eight per u32 along N (zeros[K/G][ceil(N/8)], column n%8 in bits 4*(n%8)).
 * w[k,n] = RNE_bf16(f32(q - z) * f32(s)) written as bf16 [K][N]. */
int t0_w4_dequant(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out_bf16, uint32_t K, uint32_t N, uint32_t group);
/* Fused W4A16 GEMM (no counterpart kernel in the reference; nearest items GptqWeight and the dequant kernels above):
 * y[M,N] f32 = a[M,K] bf16 * w[K,N], w dequantised in the main loop as above, fp32 accumulation.
 * Three paths, chosen by shape:
 *   M <= 16 (N % 32 == 0, K % 128 == 0, group % 128 == 0): one fused kernel on this row layout.  The row layout puts the 16 KiB
 *     a CTA needs per step in sixteen pieces 4N bytes apart, so this entry is the slower of the two M <= 16 entries;
 *     the fast one is t0_w4a16_gemm_prepacked below, on weights rewritten once by t0_w4_prepack;
 *   16 < M <= 128 (N % 32 == 0, K % 64 == 0, group % 64 == 0, 16-byte aligned pointers): one fused tcgen05 kernel, weights
 *     dequantised into the shared-memory operand inside the main loop, split along K across a thread-block cluster;
 *   anything else: dequantise once into runtime scratch (allocated on first use, K*N*2 bytes), then the bf16 GEMM. */
int t0_w4a16_gemm(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N,
                  uint32_t K, uint32_t group);
/* The same call with its arguments in a record, and `count` of them submitted back to back from native code
 * (decode loops call one projection after another; cf. prefill_dispatch.rs:61-206). */
typedef struct t0_w4a16_args {
    uint64_t a, packed, scales, zeros, y;
    uint32_t m, n, k, group;
} t0_w4a16_args;
int t0_w4a16_gemm_batch(t0_runtime* rt, const t0_w4a16_args* args, size_t count);
/* `count` INDEPENDENT problems (no y is the a or the y of another: checked, T0_ERR_INVALID).  Where they share one shape with
 * 16 < M <= 128 that the fused tcgen05 kernel takes, up to 32 of them run in ONE launch whose CTAs walk the column tiles of all
 * the problems: K is then not split, so launch, prologue and the exchange between the parts of K are paid once per launch
 * instead of once per GEMM (the projections of a decode or small-batch prefill step that read the same input).  The fp32
 * sums run along K in one piece, so y agrees with t0_w4a16_gemm to rounding, not bit for bit.  Anything else is submitted
 * back to back as by t0_w4a16_gemm_batch. */
int t0_w4a16_gemm_grouped(t0_runtime* rt, const t0_w4a16_args* args, size_t count);
/* Streaming weight layout for the fused kernel (no counterpart in the reference).  The row layout above puts the 16 KiB
 * a CTA needs per step in sixteen 1 KiB pieces 4N bytes apart, which HBM serves at about a quarter of its copy bandwidth,
 * and leaves the codes in an order no MMA fragment has.  t0_w4_prepack rewrites the three arrays once (weight-load time)
 * into one buffer of t0_w4_prepacked_bytes(K, N, group) bytes:
 *   tiles[N/256][K/128][4096] u32: one contiguous 16 KiB tile per (256-column band, 128-deep k step) in mma.sync fragment
 *     order: word ((w*2 + j)*32 + lane)*4 + e holds, for column tile w (16 columns), k step s = 4j + e (16 k) and lane
 *     (g = lane/4, t = lane%4), in nibbles c and c+4 (c = 0..3) the codes (k, k+1) of column 16w + g + 8(c&1) at
 *     k = 16s + 2t + 8(c>>1);
 *   then scales[N/256][K/group][256] bf16, then zero points [N/256][K/group][32] u32 (columns past N are zero).
 * t0_w4a16_gemm_prepacked computes the same product as t0_w4a16_gemm from that buffer (M <= 16, K % 128 == 0,
 * group % 128 == 0, N % 8 == 0, any K*N; a 16-byte aligned, the buffer 128-byte aligned); other shapes return
 * T0_ERR_UNSUPPORTED.  The fp32 sums are added in a fixed order that depends only on the shapes in the call, so a call
 * repeats bit for bit; the order differs from the row-layout entry's, so the two agree to rounding, not bit for bit.
 * The batch form reads t0_w4a16_args.packed as the prepacked buffer and ignores .scales / .zeros.  It runs up to 32
 * problems per launch, all of them at the same time on one persistent grid: the problems of one call must be independent
 * (no y of one may be the a or the y of another); order dependent projections with separate calls. */
size_t t0_w4_prepacked_bytes(uint32_t K, uint32_t N, uint32_t group);
int t0_w4_prepack(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out, uint32_t K, uint32_t N, uint32_t group);
int t0_w4a16_gemm_prepacked(t0_runtime* rt, uint64_t a, uint64_t prepacked, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group);
int t0_w4a16_gemm_prepacked_batch(t0_runtime* rt, const t0_w4a16_args* args, size_t count);
/* Tile-major weight layout for 16 < M <= 128 (no counterpart in the reference).  In the row layout the 8 KB of packed words
 * a CTA needs per 64-deep chunk are eight 1 KB pieces 4N bytes apart, which HBM serves at about a third of its copy
 * bandwidth; that, not the arithmetic, then bounds the fused tcgen05 kernel.  t0_w4_to_tiled rewrites the three arrays
 * once (weight-load time) into one buffer of t0_w4_tiled_bytes(K, N, group) bytes in which every 256-column tile is a matrix
 * of its own:  words [T][K/8][256] u32, then scales [T][K/group][256] bf16, then zero points [T][K/group][32] u32,
 * T = ceil(N / 256), columns past N zero; within a word code k (k = 0..7) sits in nibble (k >> 1) + 4 (k & 1), the order in
 * which the kernels' pairwise extraction yields consecutive k.  K % 64 == 0, group % 64 == 0, group | K; any N.
 * t0_w4a16_gemm_tiled computes the same product as t0_w4a16_gemm from that buffer (M <= 128; y f32 [M,N]);
 * t0_w4a16_gemm_tiled_grouped takes INDEPENDENT problems (checked) whose .packed is the tile-major buffer (.scales / .zeros are
 * ignored) and runs consecutive problems of one shape up to 32 per launch: K is then not split, and the dequantised weights
 * are the tensor-memory operand of the UMMAs (they never pass through shared memory). */
size_t t0_w4_tiled_bytes(uint32_t K, uint32_t N, uint32_t group);
int t0_w4_to_tiled(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out, uint32_t K, uint32_t N, uint32_t group);
int t0_w4a16_gemm_tiled(t0_runtime* rt, uint64_t a, uint64_t tiled, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group);
int t0_w4a16_gemm_tiled_grouped(t0_runtime* rt, const t0_w4a16_args* args, size_t count);
/* The fused W4A16 GEMM for callers that may not allocate device memory (no counterpart in the reference, which has no
 * fused INT4 GEMM).  Same arguments and result as t0_w4a16_gemm, bit for bit, but the scratch the kernel needs lives in a
 * fixed array inside the library (t0_w4a16_gemm_static_scratch_bytes() bytes per device), so the call never allocates or
 * frees.  Limits: M <= 16, K % 128 == 0, group % 128 == 0, N % 32 == 0, N <= 1048576, at most 160 SMs; anything else
 * returns T0_ERR_UNSUPPORTED (there is no two-step fallback here).  The first call on a device looks up the array's
 * address: make it before starting a stream capture.  All calls on one device share the array: calls that overlap in
 * time (different runtimes or streams) race; calls on one runtime are ordered by its stream.  The array holds arrival
 * counters that a completed call leaves at zero; a call that ended in T0_ERR_TIMEOUT may not, so every runtime clears them
 * (a stream-ordered memset, no allocation) before its first static call: after such a failure make a new runtime, and do
 * not go on using this entry from other runtimes of the same device that were created before the failure. */
int t0_w4a16_gemm_static(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N,
                         uint32_t K, uint32_t group);
size_t t0_w4a16_gemm_static_scratch_bytes(void);
/* Int4WmmaConfig (quant_kernels.rs:316-336): the INT4 tile record {tile_m, tile_n, tile_k} with its two constructors,
 * k16() = 16 x 16 x 16 and k32() = 16 x 16 x 32.  The reference only describes its integer WMMA tile with it and no kernel
 * reads it; it is kept so that code that builds or prints one still compiles against this library. */
typedef struct t0_int4_wmma_config {
    uint32_t tile_m, tile_n, tile_k;
} t0_int4_wmma_config;
int t0_int4_wmma_config_k16(t0_int4_wmma_config* out);
int t0_int4_wmma_config_k32(t0_int4_wmma_config* out);
/* GptqWeight::from_bytes (quant_kernels.rs:242-286): header rows, cols, group_size (u32 LE), packed codes, f32 scales,
 * i32 zero points.  Fills the three section offsets; the asserts of the reference are error codes here. */
int t0_gptq_parse(const uint8_t* raw, size_t len, uint32_t* rows, uint32_t* cols, uint32_t* group_size, size_t* packed_off,
                  size_t* scales_off, size_t* zero_points_off);
/* GptqWeight::gpu_buffer_size (quant_kernels.rs:289-293) */
size_t t0_gptq_gpu_buffer_size(uint32_t rows, uint32_t cols, uint32_t group_size);
/* Host-side repack of a GptqWeight (rows = output features N, cols = input features K) into the B200 layout above.
 * Scales are rounded (RNE) to bf16; returns how many were not exactly representable, or -1 on error. */
long t0_gptq_to_b200(const uint8_t* packed, const float* scales, const int32_t* zero_points, uint32_t rows, uint32_t cols,
                     uint32_t group_size, uint32_t* packed_out, uint16_t* scales_out, uint32_t* zeros_out);

/* ------------------------------------------------------- multi-GPU sharding */
/* The reference is single-GPU (its MultiGpuManager bounces through host memory, src/universal/runtime/multi_gpu.rs:64-159);
 * this section has no Rust counterpart to bind.  A large GEMM shards by N-column blocks: GPU r computes
 * C[:, r*N/g:(r+1)*N/g] from the replicated A and its rows [r*N/g, (r+1)*N/g) of WT[N,K].  No exchange in the computation. */
typedef struct t0_mg t0_mg;
/* the partition rule, for callers that run one process per GPU */
int t0_shard_columns(uint32_t n, uint32_t n_gpus, uint32_t rank, uint32_t* first_col, uint32_t* n_cols);
/* one process driving n_gpus devices: one runtime (stream, pool) per device */
int t0_mg_new(int n_gpus, t0_mg** out);
void t0_mg_free(t0_mg* mg);
int t0_mg_size(const t0_mg* mg);
t0_runtime* t0_mg_runtime(t0_mg* mg, int rank);
int t0_mg_synchronize(t0_mg* mg);
/* launches rank r's block on GPU r for every r, without waiting: x[r] = A on GPU r ([M,K] bf16), b_slice[r] = its N/g rows of
 * WT, y_slice[r] = where its [M, N/g] f32 block goes (slot r of the gather buffer when a gathered C is wanted). */
int t0_mg_gemm_sharded(t0_mg* mg, const uint64_t* x, const uint64_t* b_slice, const uint64_t* y_slice, uint32_t m, uint32_t n, uint32_t k,
                       uint32_t tile_n, int pair_cta);
/* The sharded GEMM and the all-gather of C in one kernel per GPU: GPU r computes its [M, N/g] block and its epilogue stores
 * every 32 x 32 block into slot r of ALL the buffers c_gathered[0..g) (its own and, over NVLink, the other GPUs'), so when
 * the g launches are complete (t0_mg_synchronize) every GPU holds all of C in the rank-major layout C_g[g][M][N/g].  No
 * second pass, no NCCL; needs peer access between the GPUs and (N/g) % 32 == 0. */
int t0_mg_gemm_sharded_gathered(t0_mg* mg, const uint64_t* x, const uint64_t* b_slice, const uint64_t* c_gathered, uint32_t m, uint32_t n,
                                uint32_t k);
/* The same product with HOST operands (the upload / dispatch / read-back sequence of the reference's host-facing calls,
 * src/universal/math/blas.rs:18-100, spread over the GPUs): x_host = A[M,K] bf16, wt_host = WT[N,K] bf16, y_host = C[M,N] f32
 * row-major.  A is replicated on the devices but crosses the host link once: GPU r uploads rows [r M/g, (r+1) M/g) and
 * the GPUs complete their copies from each other over NVLink (plain peer copies); each uploads its N/g rows of WT, multiplies,
 * and writes its column block into y_host.  Returns when y_host is complete.  Page-locked host memory lets the GPUs' copies
 * run concurrently.  The device buffers belong to the handle and are reused by later calls. */
int t0_mg_gemm_sharded_host(t0_mg* mg, const void* x_host, const void* wt_host, void* y_host, uint32_t m, uint32_t n, uint32_t k);
/* optional: every GPU ends up with all of C in the rank-major layout C_g[g][M][N/g]; c_gathered[r] is that buffer on GPU r,
 * whose slot r the GEMM already filled.  One in-place ncclAllGather over NVLink (NCCL is loaded at run time). */
int t0_mg_all_gather_c(t0_mg* mg, const uint64_t* c_gathered, uint32_t m, uint32_t n);

/* ------------------------------------------------------- seeded inputs */
/* Device-side generators for benchmark-sized inputs: element i of the stream (seed) gets the same bits as the
 * host generator of the test oracle, so any sub-range can be checked on the CPU without a full download. */
int t0_fill_uniform_bf16(t0_runtime* rt, uint64_t dst, uint64_t n, uint64_t seed, uint64_t first_index);
int t0_fill_u32(t0_runtime* rt, uint64_t dst, uint64_t n, uint64_t seed, uint64_t first_index);
int t0_fill_range_bf16(t0_runtime* rt, uint64_t dst, uint64_t n, uint64_t seed, uint64_t first_index, float lo, float hi);

#ifdef __cplusplus
}
#endif
#endif /* T0B200_H */

/*
 * CPU oracle for the T0-GPU GEMM hot path.  TEST INFRASTRUCTURE ONLY — see
 * oracle.h.  Every function cites the reference file:line it restates
 * (paths are relative to the clearnature/rust-gpu tree).
 *
 * The GEMM loops are blocked over output columns so that the compiler can
 * vectorise ACROSS columns; each output element still receives exactly the
 * reference's arithmetic: fp32 product, fp32 running sum, k ascending.  (A
 * product of two bf16 values is exact in fp32, so a fused multiply-add would
 * give the same bits; the build still disables contraction.)
 */
#define _GNU_SOURCE
#include "oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdatomic.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#if defined(__x86_64__) && defined(__GNUC__)
#define ORACLE_CLONES __attribute__((target_clones("avx512f", "avx2", "default")))
#else
#define ORACLE_CLONES
#endif

/* ---------------------------------------------------------------- bf16 -- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* src/t0/tile_ir.rs:4677 */
uint16_t oracle_f32_to_bf16_trunc(float v) { return (uint16_t)(f2u(v) >> 16); }

/* examples/test_gemm_correctness.rs:15-20 */
uint16_t oracle_f32_to_bf16_rne(float v) {
    uint32_t bits = f2u(v);
    uint32_t round = ((bits >> 16) & 1u) + 0x7FFFu;
    return (uint16_t)((bits + round) >> 16);
}

/* src/t0/tile_ir.rs:4681 */
float oracle_bf16_to_f32(uint16_t v) { return u2f((uint32_t)v << 16); }

void oracle_f32_to_bf16_rne_array(const float* in, uint16_t* out, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = oracle_f32_to_bf16_rne(in[i]);
}

int oracle_host_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

/* ---------------------------------------------------------- generators -- */

uint64_t oracle_splitmix64(uint64_t seed, uint64_t index) {
    uint64_t z = seed + (index + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline float unit24(uint64_t r) { return (float)(uint32_t)(r >> 40) * (1.0f / 16777216.0f); }

void oracle_fill_uniform_bf16(uint16_t* out, uint64_t n, uint64_t seed, uint64_t first_index) {
    for (uint64_t i = 0; i < n; ++i) {
        float u = unit24(oracle_splitmix64(seed, first_index + i));
        out[i] = oracle_f32_to_bf16_rne(2.0f * u - 1.0f);
    }
}

void oracle_fill_u32(uint32_t* out, uint64_t n, uint64_t seed, uint64_t first_index) {
    for (uint64_t i = 0; i < n; ++i) out[i] = (uint32_t)(oracle_splitmix64(seed, first_index + i) >> 32);
}

void oracle_fill_range_bf16(uint16_t* out, uint64_t n, uint64_t seed, uint64_t first_index, float lo, float hi) {
    float span = hi - lo;
    for (uint64_t i = 0; i < n; ++i) {
        float u = unit24(oracle_splitmix64(seed, first_index + i));
        float p = u * span;
        out[i] = oracle_f32_to_bf16_rne(lo + p);
    }
}

void oracle_fill_normal_bf16(uint16_t* out, uint64_t n, uint64_t seed) {
    for (uint64_t i = 0; i < n; i += 2) {
        double u1 = ((double)(oracle_splitmix64(seed, i) >> 11) + 1.0) * (1.0 / 9007199254740993.0);
        double u2 = (double)(oracle_splitmix64(seed, i + 1) >> 11) * (1.0 / 9007199254740992.0);
        double r = sqrt(-2.0 * log(u1));
        out[i] = oracle_f32_to_bf16_rne((float)(r * cos(6.283185307179586 * u2)));
        if (i + 1 < n) out[i + 1] = oracle_f32_to_bf16_rne((float)(r * sin(6.283185307179586 * u2)));
    }
}

/* ---------------------------------------------------------------- GEMM -- */

#define JB 32   /* output columns per block   */
#define IB 64   /* output rows per work item  */

typedef struct {
    const uint16_t* x;     /* [m,k] */
    const uint16_t* b;     /* NT: wt[n,k]; NN: b[k,n] */
    float* y;              /* f32 out (or NULL) */
    double* y64;           /* f64 out (or NULL) */
    uint32_t m, k, n;
    uint32_t row_begin, row_end;
    uint32_t k_begin, k_end;   /* contraction range (split-K planes) */
    int nn;                    /* 1: b is [k,n] */
    atomic_uint next;
    uint32_t n_items, items_j;
} gemm_job;

/* one (row chunk, column block): sums[j] += a * bt[kk][j], kk ascending */
ORACLE_CLONES
static void block_f32(const uint16_t* x, uint32_t ldx, const float* bt, uint32_t kk_len,
                      uint32_t rows, float* y, uint32_t ldy, uint32_t jn) {
    for (uint32_t i = 0; i < rows; ++i) {
        float sums[JB];
        for (int j = 0; j < JB; ++j) sums[j] = 0.0f;
        const uint16_t* xr = x + (size_t)i * ldx;
        for (uint32_t kk = 0; kk < kk_len; ++kk) {
            float a = u2f((uint32_t)xr[kk] << 16);
            const float* br = bt + (size_t)kk * JB;
            for (int j = 0; j < JB; ++j) sums[j] += a * br[j];
        }
        for (uint32_t j = 0; j < jn; ++j) y[(size_t)i * ldy + j] = sums[j];
    }
}

ORACLE_CLONES
static void block_f64(const uint16_t* x, uint32_t ldx, const float* bt, uint32_t kk_len,
                      uint32_t rows, double* y, uint32_t ldy, uint32_t jn) {
    for (uint32_t i = 0; i < rows; ++i) {
        double sums[JB];
        for (int j = 0; j < JB; ++j) sums[j] = 0.0;
        const uint16_t* xr = x + (size_t)i * ldx;
        for (uint32_t kk = 0; kk < kk_len; ++kk) {
            double a = (double)u2f((uint32_t)xr[kk] << 16);
            const float* br = bt + (size_t)kk * JB;
            for (int j = 0; j < JB; ++j) sums[j] += a * (double)br[j];
        }
        for (uint32_t j = 0; j < jn; ++j) y[(size_t)i * ldy + j] = sums[j];
    }
}

static void* gemm_worker(void* arg) {
    gemm_job* job = (gemm_job*)arg;
    uint32_t klen = job->k_end - job->k_begin;
    float* bt = (float*)malloc((size_t)(klen ? klen : 1) * JB * sizeof(float));
    if (!bt) return NULL;
    uint32_t cached_j = UINT32_MAX;
    for (;;) {
        uint32_t item = atomic_fetch_add(&job->next, 1);
        if (item >= job->n_items) break;
        uint32_t jb = item % job->items_j;
        uint32_t ib = item / job->items_j;
        uint32_t j0 = jb * JB;
        uint32_t jn = job->n - j0 < JB ? job->n - j0 : JB;
        uint32_t i0 = job->row_begin + ib * IB;
        uint32_t rows = job->row_end - i0 < IB ? job->row_end - i0 : IB;
        if (cached_j != jb) {
            for (uint32_t kk = 0; kk < klen; ++kk) {
                float* br = bt + (size_t)kk * JB;
                for (uint32_t j = 0; j < JB; ++j) {
                    uint16_t v = 0;
                    if (j < jn) {
                        v = job->nn ? job->b[(size_t)(job->k_begin + kk) * job->n + j0 + j]
                                    : job->b[(size_t)(j0 + j) * job->k + job->k_begin + kk];
                    }
                    br[j] = u2f((uint32_t)v << 16);
                }
            }
            cached_j = jb;
        }
        const uint16_t* xs = job->x + (size_t)i0 * job->k + job->k_begin;
        if (job->y64) block_f64(xs, job->k, bt, klen, rows, job->y64 + (size_t)i0 * job->n + j0, job->n, jn);
        else          block_f32(xs, job->k, bt, klen, rows, job->y + (size_t)i0 * job->n + j0, job->n, jn);
    }
    free(bt);
    return NULL;
}

static void run_gemm(gemm_job* job, int threads) {
    if (job->row_end <= job->row_begin || job->n == 0) return;
    uint32_t items_i = (job->row_end - job->row_begin + IB - 1) / IB;
    job->items_j = (job->n + JB - 1) / JB;
    /* work item = (row chunk, column block); the transposed column block is
     * rebuilt per item, which costs about 1/IB of the item's multiply-adds */
    job->n_items = items_i * job->items_j;
    atomic_init(&job->next, 0);
    if (threads <= 0) threads = oracle_host_threads();
    if ((uint32_t)threads > job->n_items) threads = (int)job->n_items;
    if (threads <= 1) { gemm_worker(job); return; }
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        if (pthread_create(&th[t], NULL, gemm_worker, job) == 0) ++started; else break;
    }
    if (started == 0) gemm_worker(job);
    for (int t = 0; t < started; ++t) pthread_join(th[t], NULL);
    free(th);
}

/* src/t0/tile_ir.rs:5021-5038 */
void oracle_gemm_nt_bf16_rows(const uint16_t* x, const uint16_t* wt, float* y,
                              uint32_t m, uint32_t k, uint32_t n,
                              uint32_t row_begin, uint32_t row_end, int threads) {
    gemm_job job; memset(&job, 0, sizeof job);
    job.x = x; job.b = wt; job.y = y; job.m = m; job.k = k; job.n = n;
    job.row_begin = row_begin; job.row_end = row_end < m ? row_end : m;
    job.k_begin = 0; job.k_end = k; job.nn = 0;
    run_gemm(&job, threads);
}

void oracle_gemm_nt_bf16(const uint16_t* x, const uint16_t* wt, float* y,
                         uint32_t m, uint32_t k, uint32_t n, int threads) {
    oracle_gemm_nt_bf16_rows(x, wt, y, m, k, n, 0, m, threads);
}

/* GemmTranspose::NN, src/t0/gemm_gen.rs:27: same sum, B stored [K,N] */
void oracle_gemm_nn_bf16(const uint16_t* x, const uint16_t* b, float* y,
                         uint32_t m, uint32_t k, uint32_t n, int threads) {
    gemm_job job; memset(&job, 0, sizeof job);
    job.x = x; job.b = b; job.y = y; job.m = m; job.k = k; job.n = n;
    job.row_begin = 0; job.row_end = m; job.k_begin = 0; job.k_end = k; job.nn = 1;
    run_gemm(&job, threads);
}

void oracle_gemm_nt_bf16_f64(const uint16_t* x, const uint16_t* wt, double* y,
                             uint32_t m, uint32_t k, uint32_t n, int threads) {
    gemm_job job; memset(&job, 0, sizeof job);
    job.x = x; job.b = wt; job.y64 = y; job.m = m; job.k = k; job.n = n;
    job.row_begin = 0; job.row_end = m; job.k_begin = 0; job.k_end = k; job.nn = 0;
    run_gemm(&job, threads);
}

/* src/t0/gemm_gen.rs:447-448 (one fp32 plane per split at Y + id*M*N*4);
 * examples/test_gemm_correctness.rs:203-207 (host sums planes in split order) */
void oracle_gemm_nt_bf16_splitk(const uint16_t* x, const uint16_t* wt, float* planes, float* y_sum,
                                uint32_t m, uint32_t k, uint32_t n, uint32_t split_k, int threads) {
    uint32_t chunk = k / split_k;
    size_t mn = (size_t)m * n;
    for (uint32_t s = 0; s < split_k; ++s) {
        gemm_job job; memset(&job, 0, sizeof job);
        job.x = x; job.b = wt; job.y = planes + (size_t)s * mn; job.m = m; job.k = k; job.n = n;
        job.row_begin = 0; job.row_end = m;
        job.k_begin = s * chunk; job.k_end = (s + 1 == split_k) ? k : (s + 1) * chunk; job.nn = 0;
        run_gemm(&job, threads);
    }
    if (y_sum) {
        for (size_t i = 0; i < mn; ++i) y_sum[i] = 0.0f;
        for (uint32_t s = 0; s < split_k; ++s)
            for (size_t i = 0; i < mn; ++i) y_sum[i] += planes[(size_t)s * mn + i];
    }
}

/* ----------------------------------------------------------- epilogues -- */

/* src/t0/gemm_gen.rs:40-49 */
void oracle_epilogue_gemm_gen(float* y, const float* bias, uint32_t m, uint32_t n, int mode) {
    if (mode == 0) return;
    for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < n; ++j) {
            float v = y[(size_t)i * n + j] + bias[j];
            if (mode == 2) v = v > 0.0f ? v : 0.0f;
            y[(size_t)i * n + j] = v;
        }
}

/* src/t0/tile_ir.rs:3406-3533 */
static float sigmoid_seq(float x) {
    /* negate, scale by log2(e), exp2, add one, reciprocal (tile_ir.rs:3448-3477) */
    float scaled = (-x) * 1.44269504088896340736f;
    float e = exp2f(scaled);
    return 1.0f / (e + 1.0f);
}

void oracle_epilogue_tile(float* y, uint32_t m, uint32_t n, const int* ops, int n_ops,
                          const float* bias, float scale, float clamp_min, float clamp_max) {
    for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < n; ++j) {
            float v = y[(size_t)i * n + j];
            for (int o = 0; o < n_ops; ++o) {
                switch (ops[o]) {
                    case 0: if (bias) v = v + bias[j]; break;
                    case 1: v = v * scale; break;
                    case 2: v = fmaxf(v, 0.0f); break;
                    case 3: v = v * sigmoid_seq(v); break;
                    case 4: v = v * sigmoid_seq(v * 1.702f); break;
                    case 5: v = u2f(f2u(v) & 0x7FFFFFFFu); break;
                    case 6: v = u2f(f2u(v) ^ 0x80000000u); break;
                    case 7: v = fminf(fmaxf(v, clamp_min), clamp_max); break;
                    default: break;
                }
            }
            y[(size_t)i * n + j] = v;
        }
}

/* ---------------------------------------------------------------- INT4 -- */

/* src/t0/quant_kernels.rs:74-100 (documented format :5-20) */
void oracle_dequant_int4_ref_f32(const uint8_t* packed, const float* scales, const int32_t* zps,
                                 float* out, uint32_t rows, uint32_t cols, uint32_t group_log2) {
    uint64_t total = (uint64_t)rows * cols;
    for (uint64_t e = 0; e < total; ++e) {
        uint8_t byte = packed[e >> 1];
        int32_t q = (e & 1) ? ((byte >> 4) & 0x0F) : (byte & 0x0F);
        uint64_t g = e >> group_log2;
        int32_t s = q - zps[g];
        out[e] = (float)s * scales[g];
    }
}

/* src/t0/quant_kernels.rs:127-171 (truncating store :167-168) */
void oracle_dequant_int4_ref_bf16(const uint8_t* packed, const float* scales, const int32_t* zps,
                                  uint16_t* out, uint32_t rows, uint32_t cols, uint32_t group_log2) {
    uint64_t total = (uint64_t)rows * cols;
    for (uint64_t e = 0; e < total; ++e) {
        uint8_t byte = packed[e >> 1];
        int32_t q = (e & 1) ? ((byte >> 4) & 0x0F) : (byte & 0x0F);
        uint64_t g = e >> group_log2;
        int32_t s = q - zps[g];
        out[e] = oracle_f32_to_bf16_trunc((float)s * scales[g]);
    }
}

/* The reference's formula (quant_kernels.rs:95-100) in the B200 layout, with
 * its low-nibble-first rule (:5-9) extended to eight codes per word. */
void oracle_dequant_w4_b200(const uint32_t* packed, const uint16_t* scales, const uint32_t* zeros,
                            uint16_t* w_out, uint32_t K, uint32_t N, uint32_t group) {
    uint32_t nz = (N + 7) / 8;
    for (uint32_t k = 0; k < K; ++k) {
        uint32_t g = k / group;
        for (uint32_t n = 0; n < N; ++n) {
            int32_t q = (int32_t)((packed[(size_t)(k >> 3) * N + n] >> (4 * (k & 7))) & 0xF);
            int32_t z = (int32_t)((zeros[(size_t)g * nz + (n >> 3)] >> (4 * (n & 7))) & 0xF);
            float s = oracle_bf16_to_f32(scales[(size_t)g * N + n]);
            w_out[(size_t)k * N + n] = oracle_f32_to_bf16_rne((float)(q - z) * s);
        }
    }
}

void oracle_w4a16_gemm(const uint16_t* a, const uint32_t* packed, const uint16_t* scales,
                       const uint32_t* zeros, float* y,
                       uint32_t M, uint32_t N, uint32_t K, uint32_t group, int threads) {
    uint16_t* w = (uint16_t*)malloc((size_t)K * N * sizeof(uint16_t));
    if (!w) return;
    oracle_dequant_w4_b200(packed, scales, zeros, w, K, N, group);
    oracle_gemm_nn_bf16(a, w, y, M, K, N, threads);
    free(w);
}

/* The streaming layout of the B200 W4A16 kernel (this build's own format; no reference counterpart).
 * One buffer: tiles[band][kstep][4096] u32, then scales_t[band][K/G][256] bf16, then
 * zeros_t[band][K/G][32] u32; band = 256 columns (zero-padded past N), kstep = 128 k.  A tile is in
 * mma.sync fragment order: word index ((w*2 + j)*32 + lane)*4 + e holds, for column tile w (16 columns),
 * k step s = 4j + e (16 k) and lane (g = lane/4, t = lane%4), in nibbles c and c+4 (c = 0..3) the codes
 * (k, k+1) of column 16w + g + 8(c&1) at k = 16s + 2t + 8(c>>1).  Offsets of the three parts are
 * returned through off[3]; the result is the size. */
size_t oracle_w4_prepacked_layout(uint32_t K, uint32_t N, uint32_t group, size_t off[3]) {
    size_t bands = (N + 255) / 256, ksteps = K / 128, groups = K / group;
    off[0] = 0;
    off[1] = bands * ksteps * 16 * 256 * 4;
    off[2] = off[1] + bands * groups * 256 * 2;
    return off[2] + bands * groups * 32 * 4;
}

static uint32_t w4_code(const uint32_t* packed, uint32_t N, uint32_t k, uint32_t n) {
    return (packed[(size_t)(k >> 3) * N + n] >> (4 * (k & 7))) & 0xFu;
}

void oracle_w4_prepack(const uint32_t* packed, const uint16_t* scales, const uint32_t* zeros,
                       uint8_t* out, uint32_t K, uint32_t N, uint32_t group) {
    size_t off[3];
    size_t total = oracle_w4_prepacked_layout(K, N, group, off);
    uint32_t bands = (N + 255) / 256, ksteps = K / 128, groups = K / group, nz = (N + 7) / 8;
    memset(out, 0, total);
    uint32_t* tiles = (uint32_t*)(out + off[0]);
    uint16_t* st = (uint16_t*)(out + off[1]);
    uint32_t* zt = (uint32_t*)(out + off[2]);
    for (uint32_t b = 0; b < bands; ++b) {
        for (uint32_t ks = 0; ks < ksteps; ++ks) {
            uint32_t* tile = tiles + ((size_t)b * ksteps + ks) * 4096;
            for (uint32_t w = 0; w < 16; ++w)
                for (uint32_t s = 0; s < 8; ++s)
                    for (uint32_t lane = 0; lane < 32; ++lane) {
                        uint32_t g = lane >> 2, t = lane & 3, v = 0;
                        for (uint32_t c = 0; c < 4; ++c) {
                            uint32_t n = b * 256 + w * 16 + g + 8 * (c & 1);
                            uint32_t k = ks * 128 + s * 16 + 2 * t + 8 * (c >> 1);
                            if (n >= N) continue;
                            v |= w4_code(packed, N, k, n) << (4 * c);
                            v |= w4_code(packed, N, k + 1, n) << (4 * (c + 4));
                        }
                        tile[((w * 2 + (s >> 2)) * 32 + lane) * 4 + (s & 3)] = v;
                    }
        }
        for (uint32_t c = 0; c < 256; ++c) {
            uint32_t n = b * 256 + c;
            if (n >= N) continue;
            for (uint32_t g = 0; g < groups; ++g) {
                st[((size_t)b * groups + g) * 256 + c] = scales[(size_t)g * N + n];
                uint32_t z = (zeros[(size_t)g * nz + (n >> 3)] >> (4 * (n & 7))) & 0xFu;
                zt[((size_t)b * groups + g) * 32 + (c >> 3)] |= z << (4 * (c & 7));
            }
        }
    }
}

static uint32_t rd_u32le(const uint8_t* p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

/* src/t0/quant_kernels.rs:242-286 */
int oracle_gptq_parse(const uint8_t* raw, size_t len, uint32_t* rows, uint32_t* cols, uint32_t* group,
                      size_t* packed_off, size_t* scales_off, size_t* zps_off) {
    if (len < 12) return -1;
    *rows = rd_u32le(raw); *cols = rd_u32le(raw + 4); *group = rd_u32le(raw + 8);
    if (*group == 0) return -1;
    uint32_t n_groups = *cols / *group;
    size_t n_params = (size_t)n_groups * *rows;
    size_t packed_len = (size_t)*rows * *cols / 2;
    if (len < 12 + packed_len + n_params * 8) return -1;
    *packed_off = 12; *scales_off = 12 + packed_len; *zps_off = 12 + packed_len + n_params * 4;
    return 0;
}

long oracle_gptq_to_b200(const uint8_t* packed, const float* scales, const int32_t* zps,
                         uint32_t rows, uint32_t cols, uint32_t group,
                         uint32_t* packed_out, uint16_t* scales_out, uint32_t* zeros_out) {
    uint32_t N = rows, K = cols, n_groups = cols / group, nz = (N + 7) / 8;
    long inexact = 0;
    memset(packed_out, 0, (size_t)(K / 8) * N * 4);
    memset(zeros_out, 0, (size_t)n_groups * nz * 4);
    for (uint32_t n = 0; n < N; ++n) {
        for (uint32_t k = 0; k < K; ++k) {
            uint64_t e = (uint64_t)n * K + k;
            uint8_t byte = packed[e >> 1];
            uint32_t q = (e & 1) ? ((byte >> 4) & 0xF) : (byte & 0xF);
            packed_out[(size_t)(k >> 3) * N + n] |= q << (4 * (k & 7));
        }
        for (uint32_t g = 0; g < n_groups; ++g) {
            int32_t z = zps[(size_t)n * n_groups + g];
            if (z < 0 || z > 15) return -1;
            zeros_out[(size_t)g * nz + (n >> 3)] |= (uint32_t)z << (4 * (n & 7));
            float s = scales[(size_t)n * n_groups + g];
            uint16_t sb = oracle_f32_to_bf16_rne(s);
            if (oracle_bf16_to_f32(sb) != s) ++inexact;
            scales_out[(size_t)g * N + n] = sb;
        }
    }
    return inexact;
}

// INT4 weights: K3 (stand-alone dequantisation) and K2 (fused W4A16 GEMM, dequant in the main loop).
//
// Reference: src/t0/quant_kernels.rs — `build_dequant_int4_f32/bf16` (:53-171) compute
// out[e] = f32(code(e) - zp[e >> g]) * scale[e >> g] with two codes per byte, low nibble first (:5-9);
// `GptqWeight` (:188-294) is the container and wire format.  The reference has no fused INT4 GEMM; the
// fused kernel here computes  y[m,n] = sum_k a[m,k] * w[k,n],  w = RNE_bf16((q - z) * s),  fp32 accumulate,
// on the B200 weight layout: codes packed eight per u32 along K (packed[K/8][N]), bf16 scales [K/G][N],
// uint4 zero points packed eight per u32 along N (zeros[K/G][N/8]).
//
// K2 is HBM-bound for M <= 16 (the int4 weights are ~97% of the bytes), so it is organised around the
// weight stream:
//   * 148 persistent CTAs of 16 warps; the flattened space (32-column slab) x (512-deep k step) is cut
//     into equal contiguous ranges, one per CTA (a slab may straddle two CTAs);
//   * per k step every lane issues ONE 16-byte load (4 columns x 8 codes) so a warp reads four full
//     128-byte rows; loads for the next steps are already in flight (register queue);
//   * codes become bf16 with one logic op (0x4300 | q is the bf16 128+q), minus (128+z), times s: two
//     bf16x2 ops per pair, bit-identical to the oracle's fp32 formula because (q-z)*s is exact in fp32;
//   * mma.sync m16n8k16 (bf16 in, fp32 out) does the dot products: the activations are the 16-row
//     operand, read from shared memory where they sit pre-permuted to match the code order in a word;
//   * the 16 warps' k slices are summed through shared memory in a fixed order; a slab finished by one
//     CTA is stored directly, a straddling slab goes through a small scratch area and the CTA that
//     arrives last adds the pieces in k order (no CTA ever waits for another).
#include "runtime_internal.h"

#include <cuda_bf16.h>

using namespace t0;

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kSlabCols = 32;
constexpr int kUnitK = kWarps * 32;      // k depth of one step of the CTA: 32 per warp
constexpr int kDepth = 4;                // steps kept in flight per lane
constexpr int kPieceFloats = 16 * kSlabCols;
constexpr size_t kCounterRegion = 64 * 1024;   // arrival counters: up to 16384 slabs (N <= 524288)

struct W4Params {
    const uint16_t* a;
    const uint32_t* packed;
    const uint16_t* scales;
    const uint32_t* zeros;
    float* y;
    float* partials;     // [grid][2][16*32]
    int* counters;       // [n_slabs], zero between calls
    uint32_t M, N, K, group;
    uint32_t nz;         // u32 words per row of `zeros`
    uint32_t n_slabs, ksteps, total_units;
    uint32_t a_stride;   // bytes between activation rows in shared memory
    uint32_t rows;       // activation rows staged: 8 or 16
};

struct UnitRegs {
    uint4 w;     // 4 columns x 8 codes
    uint2 s;     // 4 bf16 scales
    uint32_t z;  // 4 zero points in the low 16 bits
};

__device__ __forceinline__ uint32_t owner_of(uint32_t unit, uint32_t grid, uint32_t total) {
    return (uint32_t)((((uint64_t)unit + 1) * grid - 1) / total);
}
__device__ __forceinline__ uint32_t range_begin(uint32_t cta, uint32_t grid, uint32_t total) {
    return (uint32_t)((uint64_t)cta * total / grid);
}

__device__ __forceinline__ UnitRegs load_unit(const W4Params& p, uint32_t unit, uint32_t warp, uint32_t g, uint32_t t) {
    UnitRegs r;
    r.w = make_uint4(0, 0, 0, 0);
    r.s = make_uint2(0, 0);
    r.z = 0;
    const uint32_t slab = unit / p.ksteps, ks = unit - slab * p.ksteps;
    const uint32_t kbase = ks * kUnitK + warp * 32;
    const uint32_t col = slab * kSlabCols + 4 * g;
    if (kbase < p.K && col < p.N) {
        const uint32_t kg = (kbase >> 3) + t;
        r.w = __ldcs((const uint4*)(p.packed + (size_t)kg * p.N + col));
        const uint32_t grp = kbase / p.group;
        r.s = __ldg((const uint2*)(p.scales + (size_t)grp * p.N + col));
        r.z = __ldg(p.zeros + (size_t)grp * p.nz + (col >> 3)) >> ((col & 4) * 4);
    }
    return r;
}

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hsub2(*(__nv_bfloat162*)&a, *(__nv_bfloat162*)&b);
    return *(uint32_t*)&r;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2(*(__nv_bfloat162*)&a, *(__nv_bfloat162*)&b);
    return *(uint32_t*)&r;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kThreads, 1) w4a16_gemm_kernel(const W4Params p) {
    extern __shared__ uint8_t smem[];
    uint8_t* a_smem = smem;                                            // [rows][a_stride]
    float* red = (float*)(smem + (size_t)p.rows * p.a_stride);        // [kWarps][16][33]
    __shared__ int s_last;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t u0 = range_begin(blockIdx.x, gridDim.x, p.total_units);
    const uint32_t u1 = range_begin(blockIdx.x + 1, gridDim.x, p.total_units);

    // weights first: they are the long pole
    UnitRegs q[kDepth];
#pragma unroll
    for (int d = 0; d < kDepth; ++d)
        if (u0 + d < u1) q[d] = load_unit(p, u0 + d, warp, g, t);

    // stage the activations: within every group of eight k the order becomes 0,4,1,5,2,6,3,7 so that the
    // pair (code i, code i+4) a single mask pulls out of a word lines up with consecutive bf16 in a row
    const uint32_t k8 = p.K >> 3;
    for (uint32_t i = tid; i < p.rows * k8; i += kThreads) {
        const uint32_t r = i / k8, c = i - r * k8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < p.M) v = __ldg((const uint4*)(p.a + (size_t)r * p.K + (size_t)c * 8));
        uint4 o;
        o.x = __byte_perm(v.x, v.z, 0x5410);   // k0, k4
        o.y = __byte_perm(v.x, v.z, 0x7632);   // k1, k5
        o.z = __byte_perm(v.y, v.w, 0x5410);   // k2, k6
        o.w = __byte_perm(v.y, v.w, 0x7632);   // k3, k7
        *(uint4*)(a_smem + (size_t)r * p.a_stride + (size_t)c * 16) = o;
    }
    __syncthreads();

    float acc[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[c][j] = 0.0f;

    for (uint32_t u = u0; u < u1; ++u) {
        // take the oldest entry of the queue, refill it with the step kDepth ahead
        const UnitRegs cur = q[0];
#pragma unroll
        for (int d = 0; d < kDepth - 1; ++d) q[d] = q[d + 1];
        if (u + kDepth < u1) q[kDepth - 1] = load_unit(p, u + kDepth, warp, g, t);

        const uint32_t slab = u / p.ksteps, ks = u - slab * p.ksteps;
        const uint32_t kbase = ks * kUnitK + warp * 32;
        if (kbase < p.K) {
            const uint8_t* arow = a_smem + (size_t)g * p.a_stride + (size_t)(kbase + 8 * t) * 2;
            const uint4 alo = *(const uint4*)arow;
            uint4 ahi = make_uint4(0, 0, 0, 0);
            if (p.rows > 8) ahi = *(const uint4*)(arow + 8 * (size_t)p.a_stride);
            const uint32_t words[4] = {cur.w.x, cur.w.y, cur.w.z, cur.w.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t z = (cur.z >> (4 * c)) & 0xFu;
                const uint32_t zz = 0x43004300u | z | (z << 16);                         // bf16x2 (128+z, 128+z)
                const uint32_t sbits = (c & 1) ? ((c & 2 ? cur.s.y : cur.s.x) >> 16) : ((c & 2 ? cur.s.y : cur.s.x) & 0xFFFFu);
                const uint32_t ss = sbits | (sbits << 16);
                uint32_t wv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t v = ((words[c] >> (4 * i)) & 0x000F000Fu) | 0x43004300u;   // bf16x2 (128+q_i, 128+q_{i+4})
                    wv[i] = bf16x2_mul(bf16x2_sub(v, zz), ss);
                }
                mma_bf16_16816(acc[c], alo.x, ahi.x, alo.y, ahi.y, wv[0], wv[1]);
                mma_bf16_16816(acc[c], alo.z, ahi.z, alo.w, ahi.w, wv[2], wv[3]);
            }
        }

        const bool slab_ends = (ks + 1 == p.ksteps) || (u + 1 == u1);
        if (slab_ends) {
            // fixed-order sum of the 16 warps' k slices
            float* mine = red + (size_t)warp * 16 * 33;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                mine[g * 33 + 4 * (2 * t) + c] = acc[c][0];
                mine[g * 33 + 4 * (2 * t + 1) + c] = acc[c][1];
                mine[(g + 8) * 33 + 4 * (2 * t) + c] = acc[c][2];
                mine[(g + 8) * 33 + 4 * (2 * t + 1) + c] = acc[c][3];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[c][j] = 0.0f;
            }
            __syncthreads();
            const uint32_t row = tid >> 5, col = tid & 31;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) sum += red[(size_t)w * 16 * 33 + row * 33 + col];

            const uint32_t first_unit = slab * p.ksteps, last_unit = first_unit + p.ksteps;   // [first, last)
            const uint32_t ncol = slab * kSlabCols + col;
            const bool whole = first_unit >= u0 && last_unit <= u1;
            if (whole) {
                if (row < p.M && ncol < p.N) p.y[(size_t)row * p.N + ncol] = sum;
            } else {
                const uint32_t c_first = owner_of(first_unit, gridDim.x, p.total_units);
                const uint32_t c_last = owner_of(last_unit - 1, gridDim.x, p.total_units);
                const uint32_t slot = (first_unit <= u0) ? 0u : 1u;   // the piece of the slab holding this CTA's first unit is slot 0
                p.partials[((size_t)blockIdx.x * 2 + slot) * kPieceFloats + tid] = sum;
                __threadfence();
                __syncthreads();
                if (tid == 0) s_last = (atomicAdd(&p.counters[slab], 1) == (int)(c_last - c_first)) ? 1 : 0;
                __syncthreads();
                if (s_last) {
                    __threadfence();
                    float total = 0.0f;
                    for (uint32_t c = c_first; c <= c_last; ++c) {
                        const uint32_t cs = (first_unit <= range_begin(c, gridDim.x, p.total_units)) ? 0u : 1u;
                        total += __ldcg(p.partials + ((size_t)c * 2 + cs) * kPieceFloats + tid);
                    }
                    if (row < p.M && ncol < p.N) p.y[(size_t)row * p.N + ncol] = total;
                    if (tid == 0) p.counters[slab] = 0;   // ready for the next call
                }
            }
            __syncthreads();
        }
    }
}

// ------------------------------------------------------------------ K3: stand-alone dequantisation

// Reference wire format (quant_kernels.rs:53-171): one thread per 32 consecutive elements.
__global__ void dequant_int4_ref_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                        const int32_t* __restrict__ zps, void* __restrict__ out, uint64_t total,
                                        uint32_t group_log2, uint32_t out_bf16) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x * 32;
    for (uint64_t e0 = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 32; e0 < total; e0 += stride) {
        const bool fast = e0 + 32 <= total && (((uintptr_t)packed & 15) == 0);
        uint32_t words[4];
        if (fast) {
            const uint4 v = __ldcs((const uint4*)(packed + (e0 >> 1)));
            words[0] = v.x; words[1] = v.y; words[2] = v.z; words[3] = v.w;
        }
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
            const uint64_t e = e0 + i;
            if (e >= total) break;
            uint32_t code;
            if (fast) code = (words[i >> 3] >> (4 * (i & 7))) & 0xFu;          // byte e/2, low nibble for even e
            else { const uint8_t b = packed[e >> 1]; code = (e & 1) ? (b >> 4) : (b & 0xFu); }
            const uint64_t grp = e >> group_log2;
            const float v = __fmul_rn((float)((int32_t)code - __ldg(zps + grp)), __ldg(scales + grp));
            if (out_bf16) ((uint16_t*)out)[e] = (uint16_t)(__float_as_uint(v) >> 16);   // truncating store (quant_kernels.rs:167-168)
            else ((float*)out)[e] = v;
        }
    }
}

// B200 layout -> bf16 [K][N]: one thread per (k group of 8, 4 columns); writes 8 rows of 8 bytes.
__global__ void dequant_w4_b200_kernel(const uint32_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                                       const uint32_t* __restrict__ zeros, uint16_t* __restrict__ out, uint32_t K, uint32_t N,
                                       uint32_t group, uint32_t nz) {
    const uint32_t n4 = (N + 3) / 4;
    const uint64_t total = (uint64_t)(K / 8) * n4;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t kg = (uint32_t)(i / n4), col = (uint32_t)(i % n4) * 4;
        const uint32_t grp = (kg * 8) / group;
        for (uint32_t c = 0; c < 4 && col + c < N; ++c) {
            const uint32_t n = col + c;
            const uint32_t word = packed[(size_t)kg * N + n];
            const int32_t z = (int32_t)((zeros[(size_t)grp * nz + (n >> 3)] >> (4 * (n & 7))) & 0xFu);
            const float s = __uint_as_float((uint32_t)scales[(size_t)grp * N + n] << 16);
#pragma unroll
            for (uint32_t kk = 0; kk < 8; ++kk) {
                const int32_t qv = (int32_t)((word >> (4 * kk)) & 0xFu);
                const float v = __fmul_rn((float)(qv - z), s);
                const uint32_t bits = __float_as_uint(v);
                out[(size_t)(kg * 8 + kk) * N + n] = (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
            }
        }
    }
}

uint32_t grid_for(uint64_t n, uint32_t block) {
    uint64_t gsz = (n + block - 1) / block;
    const uint64_t cap = 148ull * 16;
    return (uint32_t)(gsz < 1 ? 1 : (gsz > cap ? cap : gsz));
}

int launch_w4_dequant(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out, uint32_t K, uint32_t N,
                      uint32_t group) {
    if (K == 0 || N == 0) return T0_OK;
    if (K % 8) return fail(T0_ERR_INVALID, "K=%u must be a multiple of 8 (eight codes per word)", K);
    if (group == 0 || group % 8) return fail(T0_ERR_INVALID, "group size %u must be a positive multiple of 8", group);
    const uint64_t total = (uint64_t)(K / 8) * ((N + 3) / 4);
    dequant_w4_b200_kernel<<<grid_for(total, 256), 256, 0, rt->stream>>>((const uint32_t*)packed, (const uint16_t*)scales,
                                                                        (const uint32_t*)zeros, (uint16_t*)out, K, N, group, (N + 7) / 8);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "dequant launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

}  // namespace

extern "C" {

int t0_w4_dequant(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out_bf16, uint32_t K, uint32_t N, uint32_t group) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!packed || !scales || !zeros || !out_bf16) return fail(T0_ERR_INVALID, "null device pointer");
    DeviceGuard guard(rt->device);
    return launch_w4_dequant(rt, packed, scales, zeros, out_bf16, K, N, group);
}

int t0_dequant_int4(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zero_points, uint64_t out, uint32_t rows, uint32_t cols,
                    uint32_t group_size_log2, int out_bf16) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    const uint64_t total = (uint64_t)rows * cols;
    if (total == 0) return T0_OK;
    if (!packed || !scales || !zero_points || !out) return fail(T0_ERR_INVALID, "null device pointer");
    if (group_size_log2 > 31) return fail(T0_ERR_INVALID, "group_size_log2=%u out of range", group_size_log2);
    DeviceGuard guard(rt->device);
    dequant_int4_ref_kernel<<<grid_for((total + 31) / 32, 256), 256, 0, rt->stream>>>(
        (const uint8_t*)packed, (const float*)scales, (const int32_t*)zero_points, (void*)out, total, group_size_log2, out_bf16 ? 1u : 0u);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "dequant launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

int t0_w4a16_gemm(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N,
                  uint32_t K, uint32_t group) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (M == 0 || N == 0) return T0_OK;
    if (!a || !packed || !scales || !zeros || !y) return fail(T0_ERR_INVALID, "null device pointer");
    if (K == 0 || K % 8) return fail(T0_ERR_INVALID, "K=%u must be a positive multiple of 8 (eight codes per word)", K);
    if (group == 0 || group % 8 || K % group) return fail(T0_ERR_INVALID, "group size %u must divide K=%u and be a multiple of 8", group, K);
    DeviceGuard guard(rt->device);

    const uint32_t rows = M <= 8 ? 8 : 16;
    const uint32_t a_stride = K * 2 + 64;   // +64 B: the eight rows a quarter-warp reads land in distinct banks
    const size_t smem = (size_t)rows * a_stride + (size_t)kWarps * 16 * 33 * sizeof(float);
    const bool fused = M <= 16 && (N % 8 == 0) && (K % 32 == 0) && (group % 32 == 0) && smem <= 200 * 1024 &&
                       ceil_div(N, kSlabCols) * sizeof(int) <= kCounterRegion &&
                       ((a | packed | scales) & 15) == 0 && (zeros & 3) == 0 && (y & 3) == 0;
    if (!fused) {
        // general shapes: dequantise once into scratch, then the tcgen05 GEMM on B[K,N]
        rc = ensure_scratch(rt, rt->scratch_w, (size_t)K * N * 2);
        if (rc != T0_OK) return rc;
        rc = launch_w4_dequant(rt, packed, scales, zeros, (uint64_t)(uintptr_t)rt->scratch_w.ptr, K, N, group);
        if (rc != T0_OK) return rc;
        t0_gemm_args ga;
        memset(&ga, 0, sizeof ga);
        ga.x = a; ga.b = (uint64_t)(uintptr_t)rt->scratch_w.ptr; ga.y = y;
        ga.m = M; ga.n = N; ga.k = K; ga.transpose = T0_NN; ga.swap_grid = 1;
        return t0_gemm_launch(rt, &ga);
    }

    const uint32_t n_slabs = ceil_div(N, kSlabCols), ksteps = ceil_div(K, kUnitK);
    const uint64_t total = (uint64_t)n_slabs * ksteps;
    if (total > 0x7FFFFFFFull) return fail(T0_ERR_UNSUPPORTED, "problem too large");
    const uint32_t grid = (uint32_t)std::min<uint64_t>(total, (uint64_t)rt->sm_count);
    // scratch: one arrival counter per slab (zero between calls) in a fixed 64 KiB region, then two straddling
    // pieces per CTA
    const size_t piece_bytes = (size_t)grid * 2 * kPieceFloats * sizeof(float);
    const size_t need = kCounterRegion + piece_bytes;
    if (need > rt->scratch_w4.size) {
        rc = ensure_scratch(rt, rt->scratch_w4, need);
        if (rc != T0_OK) return rc;
        T0_CUDA(cudaMemsetAsync(rt->scratch_w4.ptr, 0, kCounterRegion, rt->stream));
    }
    W4Params p;
    memset(&p, 0, sizeof p);
    p.a = (const uint16_t*)a; p.packed = (const uint32_t*)packed; p.scales = (const uint16_t*)scales; p.zeros = (const uint32_t*)zeros;
    p.y = (float*)y;
    p.counters = (int*)rt->scratch_w4.ptr;
    p.partials = (float*)((uint8_t*)rt->scratch_w4.ptr + kCounterRegion);
    p.M = M; p.N = N; p.K = K; p.group = group; p.nz = (N + 7) / 8;
    p.n_slabs = n_slabs; p.ksteps = ksteps; p.total_units = (uint32_t)total;
    p.a_stride = a_stride; p.rows = rows;

    static bool attr_set[64] = {};
    if (rt->device < 64 && !attr_set[rt->device]) {
        T0_CUDA(cudaFuncSetAttribute(w4a16_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[rt->device] = true;
    }
    w4a16_gemm_kernel<<<grid, kThreads, smem, rt->stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "W4A16 kernel launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

// ------------------------------------------------------------------ GptqWeight container (host side)

int t0_gptq_parse(const uint8_t* raw, size_t len, uint32_t* rows, uint32_t* cols, uint32_t* group_size, size_t* packed_off,
                  size_t* scales_off, size_t* zero_points_off) {
    // quant_kernels.rs:251-286 (`from_bytes` asserts become error codes)
    if (!raw || !rows || !cols || !group_size || !packed_off || !scales_off || !zero_points_off) return fail(T0_ERR_INVALID, "null argument");
    if (len < 12) return fail(T0_ERR_INVALID, "GPTQ data too short (need at least 12 bytes header)");
    auto rd = [&](size_t o) { return (uint32_t)raw[o] | ((uint32_t)raw[o + 1] << 8) | ((uint32_t)raw[o + 2] << 16) | ((uint32_t)raw[o + 3] << 24); };
    *rows = rd(0); *cols = rd(4); *group_size = rd(8);
    if (*group_size == 0) return fail(T0_ERR_INVALID, "GPTQ group size is zero");
    const size_t n_params = (size_t)(*cols / *group_size) * *rows;
    const size_t packed_len = (size_t)*rows * *cols / 2;
    const size_t expected = 12 + packed_len + n_params * 8;
    if (len < expected) return fail(T0_ERR_BOUNDS, "GPTQ data truncated: need %zu bytes, got %zu", expected, len);
    *packed_off = 12; *scales_off = 12 + packed_len; *zero_points_off = 12 + packed_len + n_params * 4;
    return T0_OK;
}

size_t t0_gptq_gpu_buffer_size(uint32_t rows, uint32_t cols, uint32_t group_size) {
    // quant_kernels.rs:289-293
    if (group_size == 0) return 0;
    const size_t n_params = (size_t)(cols / group_size) * rows;
    return (size_t)rows * cols / 2 + n_params * 8;
}

long t0_gptq_to_b200(const uint8_t* packed, const float* scales, const int32_t* zero_points, uint32_t rows, uint32_t cols,
                     uint32_t group_size, uint32_t* packed_out, uint16_t* scales_out, uint32_t* zeros_out) {
    if (!packed || !scales || !zero_points || !packed_out || !scales_out || !zeros_out) { fail(T0_ERR_INVALID, "null argument"); return -1; }
    if (group_size == 0 || cols % group_size || cols % 8) { fail(T0_ERR_INVALID, "cols=%u must be a multiple of 8 and of the group size %u", cols, group_size); return -1; }
    const uint32_t N = rows, K = cols, n_groups = cols / group_size, nz = (N + 7) / 8;
    memset(packed_out, 0, (size_t)(K / 8) * N * 4);
    memset(zeros_out, 0, (size_t)n_groups * nz * 4);
    long inexact = 0;
    for (uint32_t n = 0; n < N; ++n) {
        for (uint32_t k = 0; k < K; ++k) {
            const uint64_t e = (uint64_t)n * K + k;
            const uint8_t b = packed[e >> 1];
            const uint32_t code = (e & 1) ? (b >> 4) : (b & 0xFu);
            packed_out[(size_t)(k >> 3) * N + n] |= code << (4 * (k & 7));
        }
        for (uint32_t gi = 0; gi < n_groups; ++gi) {
            const int32_t z = zero_points[(size_t)n * n_groups + gi];
            if (z < 0 || z > 15) { fail(T0_ERR_UNSUPPORTED, "zero point %d of row %u group %u does not fit four bits", z, n, gi); return -1; }
            zeros_out[(size_t)gi * nz + (n >> 3)] |= (uint32_t)z << (4 * (n & 7));
            uint32_t bits;
            const float s = scales[(size_t)n * n_groups + gi];
            memcpy(&bits, &s, 4);
            const uint16_t sb = (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
            if (((uint32_t)sb << 16) != bits) ++inexact;
            scales_out[(size_t)gi * N + n] = sb;
        }
    }
    return inexact;
}

}  // extern "C"

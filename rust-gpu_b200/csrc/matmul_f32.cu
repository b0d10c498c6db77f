// The framework-facing f32 entries over the bf16 GEMM: Ignis `matmul` and its backward helpers, and the
// `BlasLib::gemm` / `gemv` facade.
//
// Reference: src/ignis/ops/bf16_matmul.rs — `matmul(x[M,K] f32, w[K,N] f32) -> y[M,N] f32` (:33-59) runs
// `dispatch_gemm_forward` (:162-207): read x and w back to the host, round to bf16 (nearest even, :371-372), transpose w,
// pad everything to tile multiples, upload, GEMM, un-pad with a copy kernel (:318-348).  `gemm_backward_data` (:216-262)
// is dX = dY * W^T, `gemm_backward_weight` (:264-312) is dW = X^T * dY, `matmul_with_wt_bf16` (:93-133) takes the weight
// already transposed and in bf16.  src/universal/math/mod.rs:24-47 is the BLAS trait, math/blas.rs:18-100 its CPU body.
//
// Here the conversions are one pass on the device (f32 -> bf16, optionally transposing), the GEMM reads the operands
// where they lie (NN layout for w, so no transpose of the weight at all; ragged edges are handled by TMA zero fill and
// masked stores), and nothing is padded, copied back or round-tripped through the host.
#include "runtime_internal.h"
#include "kernels.h"

using namespace t0;

namespace {

__device__ __forceinline__ uint16_t bf16_rne_bits(float v) {
    // bf16_matmul.rs:371-372: (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
    const uint32_t bits = __float_as_uint(v);
    return (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}

// dst[r][c] = bf16(src[r * ld_src + c]), dense rows x cols
__global__ void cvt_f32_bf16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, uint32_t rows, uint32_t cols, uint32_t ld_src) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t gtid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if ((cols % 8 == 0) && (ld_src % 4 == 0) && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
        // eight elements per thread: two 16-byte streaming loads (the f32 source is read once), one 16-byte store
        const uint32_t units_per_row = cols / 8;
        const uint64_t units = (uint64_t)rows * units_per_row;
        for (uint64_t u = gtid; u < units; u += stride) {
            const uint32_t r = (uint32_t)(u / units_per_row), c = (uint32_t)(u - (uint64_t)r * units_per_row) * 8;
            const float4* s4 = (const float4*)(src + (size_t)r * ld_src + c);
            const float4 lo = __ldcs(s4), hi = __ldcs(s4 + 1);
            uint4 o;
            o.x = (uint32_t)bf16_rne_bits(lo.x) | ((uint32_t)bf16_rne_bits(lo.y) << 16);
            o.y = (uint32_t)bf16_rne_bits(lo.z) | ((uint32_t)bf16_rne_bits(lo.w) << 16);
            o.z = (uint32_t)bf16_rne_bits(hi.x) | ((uint32_t)bf16_rne_bits(hi.y) << 16);
            o.w = (uint32_t)bf16_rne_bits(hi.z) | ((uint32_t)bf16_rne_bits(hi.w) << 16);
            *(uint4*)(dst + (size_t)r * cols + c) = o;
        }
        return;
    }
    const uint64_t total = (uint64_t)rows * cols;
    for (uint64_t i = gtid; i < total; i += stride) {
        const uint32_t r = (uint32_t)(i / cols), c = (uint32_t)(i - (uint64_t)r * cols);
        dst[i] = bf16_rne_bits(src[(size_t)r * ld_src + c]);
    }
}

// dst[c][r] = bf16(src[r][c]): 32 x 32 tiles through shared memory so both sides are coalesced
__global__ void cvt_f32_bf16_transpose_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, uint32_t rows, uint32_t cols) {
    __shared__ float tile[32][33];
    const uint32_t tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
    for (uint32_t t = blockIdx.x; t < tiles_c * tiles_r; t += gridDim.x) {
        const uint32_t tr = t / tiles_c, tc = t - tr * tiles_c;
        for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
            const uint32_t r = tr * 32 + i, c = tc * 32 + threadIdx.x;
            tile[i][threadIdx.x] = (r < rows && c < cols) ? src[(size_t)r * cols + c] : 0.0f;
        }
        __syncthreads();
        for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
            const uint32_t c = tc * 32 + i, r = tr * 32 + threadIdx.x;
            if (c < cols && r < rows) dst[(size_t)c * rows + r] = bf16_rne_bits(tile[threadIdx.x][i]);
        }
        __syncthreads();
    }
}

// c[i][j] = alpha * t[i][j] + beta * c[i][j]   (blas.rs:56: alpha * sum + beta * c)
__global__ void axpby_kernel(const float* __restrict__ t, float* __restrict__ c, uint32_t m, uint32_t n, uint32_t ldc, float alpha, float beta) {
    const uint64_t total = (uint64_t)m * n;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t r = (uint32_t)(i / n), j = (uint32_t)(i - (uint64_t)r * n);
        float* dst = c + (size_t)r * ldc + j;
        // beta == 0 must not read c (BLAS convention; the reference multiplies, which propagates NaN from garbage)
        *dst = beta == 0.0f ? alpha * t[i] : alpha * t[i] + beta * *dst;
    }
}

// y[i] = alpha * sum_j a[i*lda + j] * x[j*incx] + beta * y[i*incy]: one warp per row, f32 throughout (blas.rs:77-100)
__global__ void gemv_f32_kernel(const float* __restrict__ a, const float* __restrict__ x, float* __restrict__ y, uint32_t m, uint32_t n,
                                uint32_t lda, uint32_t incx, uint32_t incy, float alpha, float beta) {
    const uint32_t warps_per_block = blockDim.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < m; row += gridDim.x * warps_per_block) {
        float sum = 0.0f;
        for (uint32_t j = lane; j < n; j += 32) sum = fmaf(a[(size_t)row * lda + j], x[(size_t)j * incx], sum);
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
        if (lane == 0) {
            float* dst = y + (size_t)row * incy;
            *dst = beta == 0.0f ? alpha * sum : alpha * sum + beta * *dst;
        }
    }
}

uint32_t blocks_for(uint64_t n, uint32_t per_block, uint32_t sms) {
    const uint64_t want = (n + per_block - 1) / per_block;
    return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(want, (uint64_t)sms * 8));
}

int convert(t0_runtime* rt, Scratch& s, uint64_t src, uint32_t rows, uint32_t cols, uint32_t ld_src, bool transpose, uint64_t* out) {
    const size_t bytes = std::max<size_t>((size_t)rows * cols * 2, 16);
    int rc = ensure_scratch(rt, s, bytes);
    if (rc != T0_OK) return rc;
    if ((uint64_t)rows * cols) {
        if (!transpose) {
            cvt_f32_bf16_kernel<<<blocks_for((uint64_t)rows * cols, 2048, rt->sm_count), 256, 0, rt->stream>>>((const float*)src, (uint16_t*)s.ptr, rows, cols, ld_src);
        } else {
            const uint64_t tiles = (uint64_t)((rows + 31) / 32) * ((cols + 31) / 32);
            cvt_f32_bf16_transpose_kernel<<<blocks_for(tiles, 1, rt->sm_count), dim3(32, 8), 0, rt->stream>>>((const float*)src, (uint16_t*)s.ptr, rows, cols);
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(T0_ERR_CUDA, "f32 -> bf16 conversion launch failed: %s", cudaGetErrorString(e));
        rt->launches.fetch_add(1);
    }
    *out = (uint64_t)(uintptr_t)s.ptr;
    return T0_OK;
}

int gemm_bf16(t0_runtime* rt, uint64_t a, uint64_t b, uint64_t y, uint32_t m, uint32_t n, uint32_t k, int transpose) {
    t0_gemm_args ga;
    memset(&ga, 0, sizeof ga);
    ga.x = a; ga.b = b; ga.y = y;
    ga.m = m; ga.n = n; ga.k = k;
    ga.transpose = (uint8_t)transpose; ga.swap_grid = 1;
    return t0_gemm_launch(rt, &ga);
}

int check_ptrs(t0_runtime* rt, std::initializer_list<uint64_t> ptrs) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    for (uint64_t p : ptrs)
        if (!p) return fail(T0_ERR_INVALID, "null device pointer");
    return T0_OK;
}

}  // namespace

extern "C" {

int t0_matmul_f32(t0_runtime* rt, uint64_t x, uint64_t w, uint64_t y, uint32_t m, uint32_t k, uint32_t n) {
    int rc = check_ptrs(rt, {x, w, y});
    if (rc != T0_OK) return rc;
    if (m == 0 || n == 0) return T0_OK;
    DeviceGuard guard(rt->device);
    uint64_t xa = 0, wb = 0;
    rc = convert(rt, rt->scratch_cvt_a, x, m, k, k, false, &xa);
    if (rc == T0_OK) rc = convert(rt, rt->scratch_cvt_b, w, k, n, n, false, &wb);
    if (rc != T0_OK) return rc;
    return gemm_bf16(rt, xa, wb, y, m, n, k, T0_NN);                 // y = x * w, w read as B[K,N]
}

int t0_matmul_f32_with_wt_bf16(t0_runtime* rt, uint64_t x, uint64_t wt_bf16, uint64_t y, uint32_t m, uint32_t k, uint32_t n) {
    int rc = check_ptrs(rt, {x, wt_bf16, y});
    if (rc != T0_OK) return rc;
    if (m == 0 || n == 0) return T0_OK;
    DeviceGuard guard(rt->device);
    uint64_t xa = 0;
    rc = convert(rt, rt->scratch_cvt_a, x, m, k, k, false, &xa);
    if (rc != T0_OK) return rc;
    return gemm_bf16(rt, xa, wt_bf16, y, m, n, k, T0_NT);
}

int t0_matmul_f32_backward_data(t0_runtime* rt, uint64_t dy, uint64_t w, uint64_t dx, uint32_t m, uint32_t k, uint32_t n) {
    int rc = check_ptrs(rt, {dy, w, dx});
    if (rc != T0_OK) return rc;
    if (m == 0 || k == 0) return T0_OK;
    DeviceGuard guard(rt->device);
    uint64_t a = 0, b = 0;
    rc = convert(rt, rt->scratch_cvt_a, dy, m, n, n, false, &a);
    if (rc == T0_OK) rc = convert(rt, rt->scratch_cvt_b, w, k, n, n, false, &b);
    if (rc != T0_OK) return rc;
    return gemm_bf16(rt, a, b, dx, m, k, n, T0_NT);                  // dX[M,K] = dY[M,N] * W[K,N]^T: contraction over N
}

int t0_matmul_f32_backward_weight(t0_runtime* rt, uint64_t x, uint64_t dy, uint64_t dw, uint32_t m, uint32_t k, uint32_t n) {
    int rc = check_ptrs(rt, {x, dy, dw});
    if (rc != T0_OK) return rc;
    if (k == 0 || n == 0) return T0_OK;
    DeviceGuard guard(rt->device);
    uint64_t a = 0, b = 0;
    rc = convert(rt, rt->scratch_cvt_a, x, m, k, k, true, &a);       // X^T [K, M]
    if (rc == T0_OK) rc = convert(rt, rt->scratch_cvt_b, dy, m, n, n, false, &b);
    if (rc != T0_OK) return rc;
    return gemm_bf16(rt, a, b, dw, k, n, m, T0_NN);                  // dW[K,N] = X^T[K,M] * dY[M,N]: contraction over M
}

int t0_blas_gemm_f32(t0_runtime* rt, uint32_t m, uint32_t n, uint32_t k, float alpha, uint64_t a, uint32_t lda, uint64_t b, uint32_t ldb,
                     float beta, uint64_t c, uint32_t ldc) {
    int rc = check_ptrs(rt, {a, b, c});
    if (rc != T0_OK) return rc;
    if (m == 0 || n == 0) return T0_OK;
    if (lda < k || ldb < n || ldc < n) return fail(T0_ERR_INVALID, "leading dimensions (%u, %u, %u) smaller than the rows they stride (%u, %u, %u)", lda, ldb, ldc, k, n, n);
    DeviceGuard guard(rt->device);
    uint64_t xa = 0, xb = 0;
    rc = convert(rt, rt->scratch_cvt_a, a, m, k, lda, false, &xa);
    if (rc == T0_OK) rc = convert(rt, rt->scratch_cvt_b, b, k, n, ldb, false, &xb);
    if (rc != T0_OK) return rc;
    const bool direct = alpha == 1.0f && beta == 0.0f && ldc == n;
    uint64_t t = c;
    if (!direct) {
        rc = ensure_scratch(rt, rt->scratch_cvt_c, (size_t)m * n * 4);
        if (rc != T0_OK) return rc;
        t = (uint64_t)(uintptr_t)rt->scratch_cvt_c.ptr;
    }
    rc = gemm_bf16(rt, xa, xb, t, m, n, k, T0_NN);
    if (rc != T0_OK || direct) return rc;
    axpby_kernel<<<blocks_for((uint64_t)m * n, 1024, rt->sm_count), 256, 0, rt->stream>>>((const float*)t, (float*)c, m, n, ldc, alpha, beta);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "axpby launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

int t0_blas_gemv_f32(t0_runtime* rt, uint32_t m, uint32_t n, float alpha, uint64_t a, uint32_t lda, uint64_t x, uint32_t incx, float beta,
                     uint64_t y, uint32_t incy) {
    int rc = check_ptrs(rt, {a, x, y});
    if (rc != T0_OK) return rc;
    if (m == 0) return T0_OK;
    if (lda < n || incx == 0 || incy == 0) return fail(T0_ERR_INVALID, "lda=%u < n=%u or a zero increment", lda, n);
    DeviceGuard guard(rt->device);
    gemv_f32_kernel<<<blocks_for(m, 8, rt->sm_count), 256, 0, rt->stream>>>((const float*)a, (const float*)x, (float*)y, m, n, lda, incx, incy, alpha, beta);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "gemv launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

}  // extern "C"

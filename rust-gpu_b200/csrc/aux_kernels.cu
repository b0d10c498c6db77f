// Small bandwidth-bound helpers around the GEMM:
//   K4  split-K reduction: y = sum of the fp32 partial planes in split order, then the epilogue — the
//       device-side form of the host loop in examples/test_gemm_correctness.rs:203-207 and
//       examples/hello_gemm_gen.rs:125-136 of the reference;
//   staging copy for operands whose row stride or base address TMA cannot address;
//   counter-based input generators (bit-identical to the test oracle's host generators).
#include "kernels.h"

#include <cuda_bf16.h>

namespace t0 {

namespace {

struct EpiParams {
    const float* bias;
    uint32_t epilogue, n_ops;
    float scale, clamp_min, clamp_max;
    uint8_t ops[T0_TILE_MAX_EPILOGUE];
};

__device__ __forceinline__ float sigmoid_seq(float x) {
    const float e = exp2f((-x) * 1.44269504088896340736f);
    return __frcp_rn(e + 1.0f);
}

__device__ __forceinline__ float apply_epilogue(float v, uint32_t col, const EpiParams& e) {
    if (e.n_ops) {
        for (uint32_t o = 0; o < e.n_ops; ++o) {
            switch (e.ops[o]) {
                case T0_TEPI_BIAS_ADD: if (e.bias) v = v + __ldg(e.bias + col); break;
                case T0_TEPI_SCALE: v = v * e.scale; break;
                case T0_TEPI_RELU: v = fmaxf(v, 0.0f); break;
                case T0_TEPI_SILU: v = v * sigmoid_seq(v); break;
                case T0_TEPI_GELU: v = v * sigmoid_seq(v * 1.702f); break;
                case T0_TEPI_ABS: v = fabsf(v); break;
                case T0_TEPI_NEG: v = -v; break;
                case T0_TEPI_CLAMP: v = fminf(fmaxf(v, e.clamp_min), e.clamp_max); break;
                default: break;
            }
        }
    } else if (e.epilogue != T0_EPI_STORE_F32) {
        if (e.bias) v = v + __ldg(e.bias + col);
        if (e.epilogue == T0_EPI_BIAS_ADD_RELU_STORE_F32) v = fmaxf(v, 0.0f);
    }
    return v;
}

// One thread per output element; planes are read with stride m*n.  Consecutive threads read
// consecutive addresses in every plane, so each plane streams at full width.
__global__ void splitk_reduce_kernel(const float* __restrict__ planes, void* __restrict__ y, uint64_t mn, uint32_t n,
                                     uint32_t split_k, uint32_t out_bf16, EpiParams e) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += stride) {
        float acc = 0.0f;
        for (uint32_t s = 0; s < split_k; ++s) acc += planes[(uint64_t)s * mn + i];
        acc = apply_epilogue(acc, (uint32_t)(i % n), e);
        if (out_bf16) ((__nv_bfloat16*)y)[i] = __float2bfloat16_rn(acc);
        else ((float*)y)[i] = acc;
    }
}

__global__ void pad_copy_u16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, uint32_t rows, uint32_t cols,
                                    uint32_t dst_cols) {
    const uint64_t total = (uint64_t)rows * dst_cols;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t r = (uint32_t)(i / dst_cols), c = (uint32_t)(i % dst_cols);
        dst[i] = c < cols ? src[(uint64_t)r * cols + c] : (uint16_t)0;
    }
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t seed, uint64_t index) {
    uint64_t z = seed + (index + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ uint16_t f32_to_bf16_rne_bits(float v) {
    const uint32_t bits = __float_as_uint(v);
    const uint32_t round = ((bits >> 16) & 1u) + 0x7FFFu;
    return (uint16_t)((bits + round) >> 16);
}

__device__ __forceinline__ float unit24(uint64_t r) { return __fmul_rn((float)(uint32_t)(r >> 40), 1.0f / 16777216.0f); }

__global__ void fill_uniform_bf16_kernel(uint16_t* dst, uint64_t n, uint64_t seed, uint64_t first) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float u = unit24(splitmix64(seed, first + i));
        dst[i] = f32_to_bf16_rne_bits(__fsub_rn(__fmul_rn(2.0f, u), 1.0f));
    }
}

__global__ void fill_u32_kernel(uint32_t* dst, uint64_t n, uint64_t seed, uint64_t first) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = (uint32_t)(splitmix64(seed, first + i) >> 32);
}

__global__ void fill_range_bf16_kernel(uint16_t* dst, uint64_t n, uint64_t seed, uint64_t first, float lo, float span) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float u = unit24(splitmix64(seed, first + i));
        dst[i] = f32_to_bf16_rne_bits(__fadd_rn(lo, __fmul_rn(u, span)));
    }
}

uint32_t grid_for(uint64_t n, uint32_t block) {
    uint64_t g = (n + block - 1) / block;
    const uint64_t cap = 148ull * 16;
    return (uint32_t)(g < 1 ? 1 : (g > cap ? cap : g));
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
    return T0_OK;
}

}  // namespace

int launch_splitk_reduce(const float* planes, void* y, const float* bias, uint32_t m, uint32_t n, uint32_t split_k,
                         bool out_bf16, uint8_t epilogue, uint8_t n_ops, const uint8_t* ops, float scale, float clamp_min,
                         float clamp_max, cudaStream_t stream) {
    const uint64_t mn = (uint64_t)m * n;
    if (mn == 0) return T0_OK;
    EpiParams e;
    memset(&e, 0, sizeof e);
    e.bias = bias; e.epilogue = epilogue; e.n_ops = n_ops; e.scale = scale; e.clamp_min = clamp_min; e.clamp_max = clamp_max;
    if (ops) memcpy(e.ops, ops, n_ops < T0_TILE_MAX_EPILOGUE ? n_ops : T0_TILE_MAX_EPILOGUE);
    splitk_reduce_kernel<<<grid_for(mn, 256), 256, 0, stream>>>(planes, y, mn, n, split_k, out_bf16 ? 1u : 0u, e);
    return check_launch("split-K reduce");
}

int launch_pad_copy_u16(const void* src, void* dst, uint32_t rows, uint32_t cols, uint32_t dst_cols, cudaStream_t stream) {
    const uint64_t total = (uint64_t)rows * dst_cols;
    if (total == 0) return T0_OK;
    pad_copy_u16_kernel<<<grid_for(total, 256), 256, 0, stream>>>((const uint16_t*)src, (uint16_t*)dst, rows, cols, dst_cols);
    return check_launch("staging copy");
}

int launch_fill_uniform_bf16(void* dst, uint64_t n, uint64_t seed, uint64_t first, cudaStream_t stream) {
    if (n == 0) return T0_OK;
    fill_uniform_bf16_kernel<<<grid_for(n, 256), 256, 0, stream>>>((uint16_t*)dst, n, seed, first);
    return check_launch("fill_uniform_bf16");
}

int launch_fill_u32(void* dst, uint64_t n, uint64_t seed, uint64_t first, cudaStream_t stream) {
    if (n == 0) return T0_OK;
    fill_u32_kernel<<<grid_for(n, 256), 256, 0, stream>>>((uint32_t*)dst, n, seed, first);
    return check_launch("fill_u32");
}

int launch_fill_range_bf16(void* dst, uint64_t n, uint64_t seed, uint64_t first, float lo, float hi, cudaStream_t stream) {
    if (n == 0) return T0_OK;
    fill_range_bf16_kernel<<<grid_for(n, 256), 256, 0, stream>>>((uint16_t*)dst, n, seed, first, lo, hi - lo);
    return check_launch("fill_range_bf16");
}

}  // namespace t0

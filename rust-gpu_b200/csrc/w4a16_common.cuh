// Constants and device helpers shared by the fused W4A16 kernels (row-layout kernels in w4a16.cu, streaming-layout kernel
// in w4a16_stream.cu): the band / step geometry, the work split, the bf16x2 dequantisation primitives.
#pragma once

#include <cuda_bf16.h>

#include "runtime_internal.h"
#include "gemm_common.cuh"

namespace t0 {
namespace w4 {

constexpr int kWarps = 16;               // consumer warps; one more warp feeds them through TMA
constexpr int kThreads = (kWarps + 1) * 32;
constexpr int kSlabCols = 32;            // columns one warp owns
constexpr int kBandSlabs = 8;            // slabs side by side in a CTA: 256 columns = 1 KiB of every packed row
constexpr int kBandCols = kSlabCols * kBandSlabs;
constexpr int kSlices = kWarps / kBandSlabs;   // k slices of 64 per step
constexpr int kUnitK = kSlices * 64;     // k depth of one step of the CTA: 128
constexpr int kStages = 8;               // steps in flight per CTA (TMA ring)
constexpr int kARecord = 288;            // bytes per 8-k activation record (256 + 32: conflict-free quad reads)
constexpr int kWeightBytes = (kUnitK / 8) * kBandCols * 4;   // 16 packed rows x 1 KiB
constexpr int kScaleBytes = kBandCols * 2;
constexpr int kZeroBytes = (kBandCols / 8) * 4;
constexpr int kStageBytes = kWeightBytes + kScaleBytes + kZeroBytes + 128;   // 17152, keeps every stage 128-byte aligned
constexpr int kRedBytes = kWarps * 16 * 33 * 4;
constexpr int kPieceFloats = 16 * kBandCols;
constexpr int kMaxAUnits = 12;           // steps of activations staged at a time (54 KiB)
constexpr size_t kMaxSmem = 128 + (size_t)kStages * kStageBytes + kRedBytes + 256 + (size_t)kMaxAUnits * (kUnitK / 8) * kARecord;
constexpr size_t kCounterRegion = 16 * 1024;   // arrival counters: up to 4096 bands (N <= 1048576)

struct W4Params {
    const uint16_t* a;
    float* y;
    float* partials;     // [grid][2][16*256]
    int* counters;       // [n_bands], zero between calls
    int* status;         // error word of the runtime (bounded waits)
    uint32_t M, N, K;
    uint32_t units_per_group;   // group / 128: steps that share one row of scales and zero points
    uint32_t n_bands, ksteps, total_units;
    uint32_t a_units;    // steps of activations the shared-memory area holds (max steps of one CTA)
    const uint8_t* tiles;      // streaming layout only: [band][kstep][16][256] u32
    const uint8_t* scales_t;   //   [band][K/G][256] bf16
    const uint8_t* zeros_t;    //   [band][K/G][32] u32
    uint32_t groups;           //   K / G
    unsigned long long* stamps;   // optional trace: 4 nanosecond stamps per CTA (entry, staged, loop done, exit)
};

__device__ __forceinline__ uint32_t owner_of(uint32_t unit, uint32_t grid, uint32_t total) {
    return (uint32_t)((((uint64_t)unit + 1) * grid - 1) / total);
}
__device__ __forceinline__ uint32_t range_begin(uint32_t cta, uint32_t grid, uint32_t total) {
    return (uint32_t)((uint64_t)cta * total / grid);
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

// (x & mask) | magic in one LOP3; mask and magic must sit in registers (the instruction takes one immediate at most)
__device__ __forceinline__ uint32_t and_or(uint32_t x, uint32_t mask, uint32_t magic) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(x), "r"(mask), "r"(magic));
    return r;
}

// Trace buffer of the T0_W4_TRACE debugging aid: freed on every path out of the entry point that made it.
struct StampBuffer {
    unsigned long long* d = nullptr;
    size_t words = 0;
    int make(uint32_t grid) {
        words = (size_t)grid * 8;
        T0_CUDA(cudaMalloc(&d, words * sizeof(unsigned long long)));
        T0_CUDA(cudaMemset(d, 0, words * sizeof(unsigned long long)));
        return T0_OK;
    }
    ~StampBuffer() { if (d) cudaFree(d); }
};

}  // namespace w4
}  // namespace t0

// Internal launch interface between the runtime (runtime.cu) and the sm_100a kernels.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "common.h"

namespace t0 {

// Error word written by a kernel whose bounded wait expired: role in the top byte.
enum : int { kStatusOk = 0, kStatusProducerTimeout = 0x01000000, kStatusMmaTimeout = 0x02000000, kStatusEpilogueTimeout = 0x03000000 };

struct GemmLaunch {
    const void* x;        // bf16 [M,K]
    const void* b;        // bf16 [N,K] (NT) or [K,N] (NN)
    void* y;              // f32 [M,N] (or planes) / bf16 [M,N]
    const float* bias;    // f32 [N] or null
    uint32_t m, n, k;
    uint32_t ldx, ldb;    // row strides in elements (0 = dense)
    uint32_t tile_n;      // 32/64/128/256
    uint32_t split_k;     // >= 1
    uint64_t plane_stride;  // elements between split planes
    bool nn, out_bf16, swap_grid;
    uint8_t epilogue;     // T0_EPI_*
    uint8_t n_ops;        // TileIR chain (overrides epilogue when > 0)
    uint8_t ops[T0_TILE_MAX_EPILOGUE];
    float scale, clamp_min, clamp_max;
    int* status;          // device error word
    unsigned long long* probe;   // optional device buffer of two words (cycles, ns) written by CTA 0
    uint32_t n_sms;
    uint64_t wait_limit_ns;      // 0 = the default limit (ptx::kWaitLimitNs)
    bool drop_load;              // self-test: CTA 0's producer leaves out its first load, so a bounded wait must run out
    // Gathered output (multi-GPU): the product is also stored to n_peer_y other f32 [M,N] buffers, normally other GPUs'
    // memory mapped into this process.  Needs the TMA-store epilogue for every chunk: f32 output, N % 32 == 0, 16-byte aligned
    // bases, no split-K.  peer_map_slot = device memory for kMaxPeerY tensor maps (128-byte aligned) that stays untouched
    // until the launch has finished.
    void* peer_y[7];
    uint32_t n_peer_y;
    void* peer_map_slot;
    bool peer_maps_staged;       // the slot already holds the maps of exactly these destinations and this shape
};
constexpr uint32_t kMaxPeerY = 7;

// Launches the tcgen05 GEMM. Requirements (checked): x and b 16-byte aligned, row strides and
// K / split_k multiples of 8 elements, K % split_k == 0.  Returns a T0_* code.
int launch_gemm_sm100(const GemmLaunch& g, cudaStream_t stream);

// The CTA-pair form (cta_group::2; 256 x 256 tiles, or 256 x 128 when tile_n <= 128); NT, and NN with 256-wide tiles.
int launch_gemm_sm100_pair(const GemmLaunch& g, cudaStream_t stream);
uint32_t gemm_pair_smem_bytes(uint32_t pair_n);

// Split-K inside one launch: the split_k CTAs of an output tile form a cluster and add their partial sums through
// distributed shared memory (same sum, in split order, as planes + reduction).  NT layout, split_k 2 / 4 / 8, tile_n 64 / 128.
bool gemm_splitk_cluster_supported(const GemmLaunch& g);
int launch_gemm_sm100_splitk(const GemmLaunch& g, cudaStream_t stream);
// Several problems of ONE shape and configuration (only x, b and y differ) in one launch of the same kernel: the clusters walk
// the tiles of all the problems, so launch, prologue and drain are paid once and the exchange of one tile overlaps the main
// loop of the next.  The problems run concurrently: no y may be an input of another.  At most kMaxGroupedGemms per launch.
constexpr uint32_t kMaxGroupedGemms = 32;
int launch_gemm_sm100_splitk_grouped(const GemmLaunch* gs, uint32_t count, cudaStream_t stream);
// The same for shapes that need no split-K once several problems fill the GPU: the single-CTA kernel, NT, tile width 64 / 128.
int launch_gemm_sm100_grouped(const GemmLaunch* gs, uint32_t count, cudaStream_t stream);

// y[i] = sum_s planes[s][i] in split order, then the epilogue; K4.
int launch_splitk_reduce(const float* planes, void* y, const float* bias, uint32_t m, uint32_t n, uint32_t split_k,
                         bool out_bf16, uint8_t epilogue, uint8_t n_ops, const uint8_t* ops, float scale, float clamp_min,
                         float clamp_max, cudaStream_t stream);

// dst[r][0..dst_cols) = src[r][0..cols) zero-extended, 16-bit elements (staging copy for shapes TMA cannot address).
int launch_pad_copy_u16(const void* src, void* dst, uint32_t rows, uint32_t cols, uint32_t dst_cols, cudaStream_t stream);

int launch_fill_uniform_bf16(void* dst, uint64_t n, uint64_t seed, uint64_t first, cudaStream_t stream);
int launch_fill_u32(void* dst, uint64_t n, uint64_t seed, uint64_t first, cudaStream_t stream);
int launch_fill_range_bf16(void* dst, uint64_t n, uint64_t seed, uint64_t first, float lo, float hi, cudaStream_t stream);

// Shared-memory footprint of the GEMM pipeline for a tile width.
uint32_t gemm_stage_count(uint32_t tile_n);
uint32_t gemm_smem_bytes(uint32_t tile_n);

// Scratch of the fused W4A16 kernels: the arrival-counter region, and counters plus two pieces per CTA for a grid of `ctas`.
size_t w4a16_counter_region_bytes();
size_t w4a16_fixed_scratch_bytes(uint32_t ctas);

}  // namespace t0

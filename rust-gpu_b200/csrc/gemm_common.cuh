// Pieces shared by the single-CTA and the CTA-pair GEMM kernels: launch parameters, the persistent
// tile schedule, the epilogue/store of one accumulator chunk, and the TMA tensor-map builders.
#pragma once

#include <cuda_bf16.h>
#include <cstdlib>
#include <mutex>

#include "kernels.h"
#include "ptx_sm100.cuh"

namespace t0 {
namespace gemm {

constexpr uint32_t BM = 128;            // accumulator rows per CTA (one UMMA M=128 half or whole)
constexpr uint32_t BK = 64;             // one 128-byte swizzle atom of bf16
constexpr uint32_t kAStageBytes = BM * BK * 2;

struct KParams {
    void* y;
    const float* bias;
    int* status;
    unsigned long long* probe;   // optional: {SM cycles, nanoseconds} of CTA 0, for the in-kernel clock estimate
    unsigned long long* trace;   // optional (T0_GEMM_TRACE=1): eight nanosecond stamps of CTA 0's roles, see trace_stamp
    uint64_t plane_stride;
    uint64_t wait_limit_ns;      // limit of every single barrier wait in this launch
    uint32_t M, N, K;
    uint32_t tiles_m, tiles_n, split_k;
    uint32_t kb_per_split;
    uint32_t swap_grid, raster_group;
    uint32_t sk_stages, sk_alias; // split-K cluster kernel: ring depth; 1 = the accumulator is parked over the ring (one tile per cluster)
    uint32_t tail_start;         // pair kernel: work items from here on are half-width tiles (two per output tile); = total when unused
    uint32_t out_bf16, epilogue, n_ops;
    uint32_t tma_store;          // full f32 chunks leave through the output tensor map
    uint32_t drop_load;          // self-test of the failure path: the producer of CTA 0 leaves out its first operand load
    uint32_t n_problems;         // split-K cluster kernel, grouped launch: problems of one shape in this launch (0 or 1 = a single problem)
    uint32_t n_peers;            // gathered output: every TMA-stored chunk also goes to this many other buffers (other GPUs' memory)
    const CUtensorMap* peer_maps; // their output tensor maps, in global memory (written by the host before the launch)
    float scale, clamp_min, clamp_max;
    uint8_t ops[T0_TILE_MAX_EPILOGUE];
};

// Grouped launch (several problems of one shape in one launch): the problems' tensor maps and outputs ride in the kernel
// parameters; the kernels that are not grouped take the empty record.
struct NoGroup { uint32_t unused; };

struct WorkItem { uint32_t m_blk, n_blk, split; };

__device__ __forceinline__ WorkItem decode_work(uint32_t w, const KParams& p) {
    WorkItem it;
    it.split = w % p.split_k;
    const uint32_t t = w / p.split_k;
    const uint32_t tiles_fast = p.swap_grid ? p.tiles_n : p.tiles_m;
    const uint32_t tiles_slow = p.swap_grid ? p.tiles_m : p.tiles_n;
    const uint32_t group_size = p.raster_group * tiles_fast;
    const uint32_t g = t / group_size;
    const uint32_t first = g * p.raster_group;
    const uint32_t gsz = min(p.raster_group, tiles_slow - first);
    const uint32_t r = t - g * group_size;
    const uint32_t slow = first + r % gsz;
    const uint32_t fast = r / gsz;
    it.m_blk = p.swap_grid ? slow : fast;
    it.n_blk = p.swap_grid ? fast : slow;
    return it;
}

__device__ __forceinline__ float sigmoid_seq(float x) {
    // tile_ir.rs:3448-3477: negate, scale by log2(e), exp2, add one, reciprocal
    const float e = exp2f((-x) * 1.44269504088896340736f);
    return __frcp_rn(e + 1.0f);
}

__device__ __forceinline__ float apply_chain(float v, float bias, const KParams& p) {
    for (uint32_t o = 0; o < p.n_ops; ++o) {
        switch (p.ops[o]) {
            case T0_TEPI_BIAS_ADD: v = v + bias; break;
            case T0_TEPI_SCALE: v = v * p.scale; break;
            case T0_TEPI_RELU: v = fmaxf(v, 0.0f); break;
            case T0_TEPI_SILU: v = v * sigmoid_seq(v); break;
            case T0_TEPI_GELU: v = v * sigmoid_seq(v * 1.702f); break;
            case T0_TEPI_ABS: v = fabsf(v); break;
            case T0_TEPI_NEG: v = -v; break;
            case T0_TEPI_CLAMP: v = fminf(fmaxf(v, p.clamp_min), p.clamp_max); break;
            default: break;
        }
    }
    return v;
}


// Debugging aid, compiled in only with -DT0_GEMM_TRACE (the stamps cost the pair kernel 40 registers): CTA 0 records when
// its roles pass a few points of the kernel; with T0_GEMM_TRACE=1 in the environment t0_rt_last_kernel_clock prints them.
__device__ __forceinline__ void trace_stamp(const KParams& p, int i) {
#ifdef T0_GEMM_TRACE
    if (p.trace && blockIdx.x == 0) p.trace[i] = ptx::globaltimer_ns();
#endif
}

// CTA 0 stamps the SM cycle counter and the global nanosecond timer at entry and exit; the host turns
// the two deltas into the SM clock the kernel actually ran at (power management moves it).
struct ClockProbe {
    long long c0 = 0;
    unsigned long long t0 = 0;
    __device__ __forceinline__ void begin(const KParams& p) {
        if (p.probe && blockIdx.x == 0 && threadIdx.x == 0) { c0 = clock64(); t0 = ptx::globaltimer_ns(); }
    }
    __device__ __forceinline__ void end(const KParams& p) {
        if (p.probe && blockIdx.x == 0 && threadIdx.x == 0) {
            p.probe[0] = (unsigned long long)(clock64() - c0);
            p.probe[1] = ptx::globaltimer_ns() - t0;
        }
    }
};

constexpr uint32_t kEpiStageBytes = 4096;   // per epilogue warp: one 32 x 32 f32 chunk on its way to global memory

// One 32-row x 32-column chunk of the accumulator (this lane holds row `row_base + lane`): epilogue, then the store.
// A lane holds 32 consecutive columns of ONE row, so storing straight from registers makes every warp instruction touch
// 32 different 128-byte lines (16 bytes of each): 256 line accesses per chunk, which made the epilogue of a 128 x 256 tile
// cost about 5 us.  Full chunks therefore go through `stage` (this warp's 4 KiB of shared memory, 16-byte slots XOR-swizzled
// so that neither the row-wise write nor the line-wise read has bank conflicts) and leave as whole lines: a warp instruction
// stores four complete 128-byte row segments.  Ragged chunks (N edge, unaligned y or N) keep the element-wise path.
// With `map_y` (an f32 output the TMA unit can address: 16-byte aligned base and row pitch) the staged block leaves as ONE
// tiled TMA store instead of eight loads from the block and eight line-wise stores: the block's XOR pattern is the 128-byte
// swizzle of the tensor map, rows beyond M are clipped by the copy.  `stage` is the warp's pair of blocks (1024-byte aligned,
// kEpiStageBytes each).  `n_stores` is the warp's running count of committed TMA stores, carried across chunks AND tiles: store
// i leaves from block i & 1, and before block i & 1 is rewritten the warp waits until every committed store but the latest
// (which left from the other block) has read its source.  Counting only committed stores keeps that true when a tile has
// an odd number of full chunks, a single chunk, or rows the copy would clip entirely.  The caller waits for its stores
// (ptx::bulk_wait_group_all by lane 0) before shared memory goes away.
__device__ __forceinline__ void store_chunk(const KParams& p, const uint32_t (&r)[32], uint32_t row_base, uint32_t lane, uint32_t col0,
                                            uint32_t split, bool vec32, bool vec16, uint8_t* stage, uint32_t& n_stores, const CUtensorMap* map_y = nullptr,
                                            void* y_base = nullptr) {
    void* const y_out = y_base ? y_base : p.y;       // a grouped launch names the problem's output
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (p.n_ops) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float bj = (p.bias && col0 + j < p.N) ? __ldg(p.bias + col0 + j) : 0.0f;
            v[j] = apply_chain(v[j], bj, p);
        }
    } else if (p.epilogue != T0_EPI_STORE_F32) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float bj = (p.bias && col0 + j < p.N) ? __ldg(p.bias + col0 + j) : 0.0f;
            v[j] += bj;
            if (p.epilogue == T0_EPI_BIAS_ADD_RELU_STORE_F32) v[j] = fmaxf(v[j], 0.0f);
        }
    }
    const size_t plane = (size_t)split * p.plane_stride;
    const bool full = col0 + 32 <= p.N;          // warp-uniform
    if (!p.out_bf16 && vec32 && full) {
        // [32 rows][8 slots of 16 bytes], slot index XOR (row & 7); explicit shared-space accesses (the pointer went
        // through an integer for alignment, so the compiler would otherwise use generic loads and stores)
        if (map_y && row_base >= p.M) return;                 // warp-uniform: a box that starts below the last row has nothing to write
        const uint32_t sb = ptx::smem_u32(stage) + (map_y ? (n_stores & 1u) * kEpiStageBytes : 0u);
        if (map_y) {
            if (lane == 0) ptx::bulk_wait_group_read_but_one();   // the latest committed store left from the other block
            __syncwarp();
        }
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(sb + (lane * 8 + (j ^ (lane & 7))) * 16), "f"(v[4 * j]), "f"(v[4 * j + 1]),
                         "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                         : "memory");
        if (map_y) {
            ptx::fence_proxy_async_smem();                    // the copy reads the block through the async proxy
            __syncwarp();
            if (lane == 0) {
                ptx::tma_store_3d(map_y, sb, (int32_t)col0, (int32_t)row_base, (int32_t)split);
                // gathered output: the same block to the other GPUs' buffers (plain TMA stores to peer memory over NVLink),
                // in the same bulk group, so the block is reused only after all of them have read it
                for (uint32_t i = 0; i < p.n_peers; ++i) {
                    // the maps were written to global memory by a copy before this launch: before the first use, order this
                    // thread's tensor-map reads after that write (the slot is rewritten when the destinations change)
                    if (n_stores == 0) ptx::fence_proxy_tensormap_acquire(p.peer_maps + i);
                    ptx::tma_store_3d(p.peer_maps + i, sb, (int32_t)col0, (int32_t)row_base, (int32_t)split);
                }
                ptx::bulk_commit_group();
            }
            ++n_stores;
            return;
        }
        __syncwarp();
        const uint32_t slot = lane & 7;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t rr = i * 4 + (lane >> 3), row = row_base + rr;
            float4 q;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(q.x), "=f"(q.y), "=f"(q.z), "=f"(q.w) : "r"(sb + (rr * 8 + (slot ^ (rr & 7))) * 16) : "memory");
            if (row < p.M) *(float4*)((float*)y_out + plane + (size_t)row * p.N + col0 + 4 * slot) = q;
        }
        __syncwarp();
        return;
    }
    if (p.out_bf16 && vec16 && full) {
        uint4* s4 = (uint4*)stage;               // [32 rows][4 slots of 16 bytes], slot index XOR ((row >> 1) & 3)
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            uint4 q;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
            q.x = *(uint32_t*)&h0; q.y = *(uint32_t*)&h1; q.z = *(uint32_t*)&h2; q.w = *(uint32_t*)&h3;
            s4[lane * 4 + (j ^ ((lane >> 1) & 3))] = q;
        }
        __syncwarp();
        const uint32_t slot = lane & 3;
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t rr = i * 8 + (lane >> 2), row = row_base + rr;
            const uint4 q = s4[rr * 4 + (slot ^ ((rr >> 1) & 3))];
            if (row < p.M) *(uint4*)((__nv_bfloat16*)y_out + plane + (size_t)row * p.N + col0 + 8 * slot) = q;
        }
        __syncwarp();
        return;
    }
    const uint32_t row = row_base + lane;
    if (row >= p.M) return;
    const size_t off = plane + (size_t)row * p.N + col0;
    if (!p.out_bf16) {
        float* dst = (float*)y_out + off;
        for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) dst[j] = v[j];
    } else {
        __nv_bfloat16* dst = (__nv_bfloat16*)y_out + off;
        for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
    }
}

// ------------------------------------------------------------------ launch (host)

// Launch with programmatic stream serialisation so the prologue of this grid overlaps the tail of the
// previous one (T0_NO_PDL=1 in the environment turns it off).
template <typename Kernel, typename... Args>
inline cudaError_t launch_pdl(Kernel kern, uint32_t grid, uint32_t block, uint32_t smem, cudaStream_t stream, const Args&... args) {
    static const bool use_pdl = getenv("T0_NO_PDL") == nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

// ------------------------------------------------------------------ tensor maps (host)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// 3-D view [split][rows][k_per_split] of a row-major [rows][ld] bf16 matrix (K contiguous, ld >= K).
inline int make_map_kmajor(CUtensorMap* map, const void* base, uint32_t rows, uint32_t ld, uint32_t k_per_split, uint32_t split,
                    uint32_t box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {k_per_split, rows, split};
    // with a single split the third dimension has extent 1; its stride only has to be a legal value
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, split > 1 ? (cuuint64_t)k_per_split * 2 : (cuuint64_t)ld * 2 * rows};
    cuuint32_t box[3] = {BK, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled (K-major, rows=%u ld=%u) failed: %d", rows, ld, (int)r);
    return T0_OK;
}

// Plain 2-D row-major view [rows][cols] of 16- or 32-bit elements, no swizzle, box = box_cols x box_rows.
inline int make_map_2d_plain(CUtensorMap* map, const void* base, uint32_t elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_cols,
                             uint32_t box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * elem_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled (plain 2-D, %llu x %llu) failed: %d", (unsigned long long)rows, (unsigned long long)cols, (int)r);
    return T0_OK;
}

// Plain (unswizzled) 3-D view [d2][d1][d0] with byte strides for d1 and d2, box d0 x d1 x 1 (u32 or u16 elements).
inline int make_map_3d_plain(CUtensorMap* map, const void* base, uint32_t elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                             uint64_t stride2_bytes, uint32_t box0, uint32_t box1) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {box0, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled (plain 3-D, %llu x %llu x %llu) failed: %d", (unsigned long long)d2, (unsigned long long)d1, (unsigned long long)d0, (int)r);
    return T0_OK;
}

// 3-D view [planes][M][N] of the f32 output (or of split-K planes `plane_stride` elements apart), box 32 x 32, 128-byte
// swizzle: what the epilogue's TMA store writes through.  Needs a 16-byte aligned base and N % 4 == 0.
inline int make_map_out_f32(CUtensorMap* map, const void* base, uint32_t M, uint32_t N, uint32_t planes, uint64_t plane_stride) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {N, M, planes > 1 ? planes : 1};
    cuuint64_t strides[2] = {(cuuint64_t)N * 4, planes > 1 ? (cuuint64_t)plane_stride * 4 : (cuuint64_t)M * N * 4};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled (f32 output %u x %u) failed: %d", M, N, (int)r);
    return T0_OK;
}

// Gathered output: one output tensor map per extra destination, copied to `g.peer_map_slot` on the launch stream (a small
// pageable-source copy, staged by the driver before the call returns), unless the caller says the slot already holds them.
inline int stage_peer_maps(const GemmLaunch& g, KParams& p, uint32_t split, cudaStream_t stream) {
    p.n_peers = 0;
    p.peer_maps = nullptr;
    if (g.n_peer_y == 0) return T0_OK;
    if (g.n_peer_y > 7 || !g.peer_map_slot) return fail(T0_ERR_INVALID, "gathered output: %u destinations (at most 7) or no slot for their tensor maps", g.n_peer_y);
    if (!p.tma_store || split != 1 || g.n % 32 != 0)
        return fail(T0_ERR_UNSUPPORTED, "a gathered output needs the TMA-store epilogue on every chunk: f32 output, N %% 32 == 0 (N=%u), 16-byte aligned buffers, no split-K", g.n);
    if (!g.peer_maps_staged) {
        CUtensorMap maps[7];
        for (uint32_t i = 0; i < g.n_peer_y; ++i) {
            if (!g.peer_y[i] || ((uintptr_t)g.peer_y[i] & 15)) return fail(T0_ERR_INVALID, "gathered output: destination %u is null or not 16-byte aligned", i);
            int rc = make_map_out_f32(&maps[i], g.peer_y[i], g.m, g.n, 1, 0);
            if (rc != T0_OK) return rc;
        }
        cudaError_t e = cudaMemcpyAsync(g.peer_map_slot, maps, g.n_peer_y * sizeof(CUtensorMap), cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return fail(T0_ERR_CUDA, "gathered output: copying the tensor maps failed: %s", cudaGetErrorString(e));
    }
    p.peer_maps = (const CUtensorMap*)g.peer_map_slot;
    p.n_peers = g.n_peer_y;
    return T0_OK;
}

// 3-D view [split][k_per_split][N] of a row-major [K][ld] bf16 matrix (N contiguous, ld >= N).
inline int make_map_nmajor(CUtensorMap* map, const void* base, uint32_t N, uint32_t ld, uint32_t k_per_split, uint32_t split) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {N, k_per_split, split};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)k_per_split * ld * 2};   // always a multiple of 16
    cuuint32_t box[3] = {64, BK, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(T0_ERR_CUDA, "cuTensorMapEncodeTiled (N-major, N=%u) failed: %d", N, (int)r);
    return T0_OK;
}


}  // namespace gemm
}  // namespace t0

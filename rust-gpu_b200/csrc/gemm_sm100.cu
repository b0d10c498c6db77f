// K1 — dense bf16 GEMM for sm_100a: y[M,N] = x[M,K] * op(b), fp32 accumulation in tensor memory.
//
// Replaces the reference's generated RDNA kernels (src/t0/gemm_gen.rs:668-1438 generate_lds_db and
// src/t0/tile_ir.rs:887-2459 lower_gemm).  Same contract: bf16 operands, NT (b = WT[N,K]) or NN
// (b = B[K,N]) layout, f32 output, optional split-K planes at y + id*M*N (gemm_gen.rs:447-448),
// ragged M/N/K handled by zero fill and predicated stores (tile_ir.rs:1142-1203,3699-3717), fused
// epilogues (gemm_gen.rs:40-49, tile_ir.rs:3406-3533).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: 128B-swizzled tiles of A (128 x 64) and B (BN x 64) into a ring of stages
//   warp 1      UMMA issuer: four tcgen05.mma (128 x BN x 16) per stage, accumulator in tensor memory;
//               owns the tensor-memory allocation (two accumulator buffers of BN columns)
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator, apply the epilogue, store to global,
//               while the issuer already fills the other accumulator buffer
// All inter-role hand-offs are mbarriers; every wait is bounded and a wait that expires writes an
// error word the host turns into an error (no trap, no unbounded spin).
#include "kernels.h"
#include "ptx_sm100.cuh"
#include <type_traits>
#include "gemm_common.cuh"


namespace t0 {

namespace {

using namespace gemm;
constexpr uint32_t kThreads = 192;

__host__ __device__ constexpr uint32_t stages_for(uint32_t bn) { return bn == 256 ? 4 : bn == 128 ? 6 : 8; }

// Grouped launch: operand and output maps and the output addresses of up to kMaxGroupedGemms problems of one shape (12.5 KB
// of kernel parameters).
struct GroupOperands3 {
    CUtensorMap maps[3 * kMaxGroupedGemms];     // A, B, Y of problem i at 3i, 3i + 1, 3i + 2
    void* y[kMaxGroupedGemms];
};

template <uint32_t BN, bool B_MN, bool kGrouped = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_y, const KParams p,
                         const __grid_constant__ std::conditional_t<kGrouped, GroupOperands3, NoGroup> group) {
    constexpr uint32_t kStages = stages_for(BN);
    constexpr uint32_t kBStageBytes = BN * BK * 2;
    constexpr uint32_t kStageBytes = kAStageBytes + kBStageBytes;
    constexpr uint32_t kTmemCols = 2 * BN;   // two accumulator buffers; 64..512, a power of two
    constexpr uint32_t kIdesc = ptx::make_idesc_bf16_f32(BM, BN, B_MN ? 1u : 0u);

    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles need 1024-byte alignment
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + kStages * kAStageBytes;
    uint8_t* epi_stage = smem + kStages * kStageBytes;          // 4 warps x 2 blocks of kEpiStageBytes; 1024-byte aligned
    uint64_t* bars = (uint64_t*)(epi_stage + 8 * kEpiStageBytes);
    uint64_t* full_bar = bars;                       // [kStages] TMA bytes landed
    uint64_t* empty_bar = bars + kStages;            // [kStages] UMMAs finished reading the stage
    uint64_t* tmem_full_bar = bars + 2 * kStages;    // [2] accumulator complete
    uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;  // [2] accumulator drained by the epilogue
    uint32_t* tmem_holder = (uint32_t*)(bars + 2 * kStages + 4);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t work_per_problem = p.tiles_m * p.tiles_n * p.split_k;
    uint32_t total_work = work_per_problem;                 // a grouped launch walks the tiles of all its problems, problem-major
    if constexpr (kGrouped) total_work = work_per_problem * p.n_problems;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&tmem_full_bar[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&tmem_empty_bar[b]), 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::tma_prefetch_desc(&map_a);
        ptx::tma_prefetch_desc(&map_b);
        if (p.tma_store) ptx::tma_prefetch_desc(&map_y);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_holder), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    // everything above touched only shared and tensor memory; global memory comes after the previous grid is done
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    ClockProbe probe;
    probe.begin(p);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
                uint32_t prob = 0, item = w;
                if constexpr (kGrouped) { prob = w / work_per_problem; item = w - prob * work_per_problem; }
                const WorkItem wi = decode_work(item, p);
                const CUtensorMap* ma = &map_a;
                const CUtensorMap* mb = &map_b;
                if constexpr (kGrouped) { ma = &group.maps[3 * prob]; mb = &group.maps[3 * prob + 1]; }
                for (uint32_t kb = 0; kb < p.kb_per_split; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.wait_limit_ns)) {
                        atomicCAS(p.status, 0, kStatusProducerTimeout | (int)(w & 0xFFFFFF));
                        ok = false;
                        break;
                    }
                    const uint32_t fb = ptx::smem_u32(&full_bar[stage]);
                    // self-test of the failure path: this stage is never filled, so the issuer's bounded wait must run out
                    if (p.drop_load && blockIdx.x == 0 && w == 0 && kb == 0) { if (++stage == kStages) { stage = 0; phase ^= 1; } continue; }
                    ptx::mbar_arrive_expect_tx(fb, kStageBytes);
                    ptx::tma_load_3d(ptx::smem_u32(a_tiles + stage * kAStageBytes), ma, fb,
                                     (int32_t)(kb * BK), (int32_t)(wi.m_blk * BM), (int32_t)wi.split);
                    if constexpr (!B_MN) {
                        ptx::tma_load_3d(ptx::smem_u32(b_tiles + stage * kBStageBytes), mb, fb,
                                         (int32_t)(kb * BK), (int32_t)(wi.n_blk * BN), (int32_t)wi.split);
                    } else {
                        // B[K,N]: one 64(k) x 64(n) box per 64 columns; each box is an [k][128 B] block
#pragma unroll
                        for (uint32_t j = 0; j < BN / 64; ++j)
                            ptx::tma_load_3d(ptx::smem_u32(b_tiles + stage * kBStageBytes + j * (BK * 128)), mb, fb,
                                             (int32_t)(wi.n_blk * BN + j * 64), (int32_t)(kb * BK), (int32_t)wi.split);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < total_work; w += gridDim.x, ++iter) {
                const uint32_t buf = iter & 1, acc_phase = (iter >> 1) & 1;
                if (!ptx::mbar_wait(ptx::smem_u32(&tmem_empty_bar[buf]), acc_phase ^ 1, abort_flag, p.wait_limit_ns)) {
                    atomicCAS(p.status, 0, kStatusMmaTimeout | (int)(w & 0xFFFFFF));
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (uint32_t kb = 0; kb < p.kb_per_split; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag, p.wait_limit_ns)) {
                        atomicCAS(p.status, 0, kStatusMmaTimeout | 0x800000 | (int)(w & 0x7FFFFF));
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = ptx::smem_u32(a_tiles + stage * kAStageBytes);
                    const uint32_t b_addr = ptx::smem_u32(b_tiles + stage * kBStageBytes);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < BK / 16; ++k4) {
                        // K-major, 128B swizzle: 8-row groups 1024 B apart; a 16-element K step is 32 B
                        const uint64_t da = ptx::make_smem_desc(a_addr + k4 * 32, 16, 1024);
                        // N-major B: 64-column atoms 8 KiB apart, 8-row k groups 1024 B apart; a K step is two groups
                        const uint64_t db = B_MN ? ptx::make_smem_desc(b_addr + k4 * 2048, BK * 128, 1024)
                                                 : ptx::make_smem_desc(b_addr + k4 * 32, 16, 1024);
                        ptx::umma_bf16_ss(tmem_d, da, db, kIdesc, (kb | k4) != 0 ? 1u : 0u);
                    }
                    ptx::umma_commit(ptx::smem_u32(&empty_bar[stage]));
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (ok) ptx::umma_commit(ptx::smem_u32(&tmem_full_bar[buf]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const uint32_t quarter = warp & 3;   // tensor-memory lanes 32*quarter .. +31 belong to this warp
        uint32_t iter = 0, n_stores = 0;     // n_stores: this warp's committed TMA stores, see store_chunk
        for (uint32_t w = blockIdx.x; w < total_work; w += gridDim.x, ++iter) {
            uint32_t prob = 0, item = w;
            if constexpr (kGrouped) { prob = w / work_per_problem; item = w - prob * work_per_problem; }
            const WorkItem wi = decode_work(item, p);
            void* y_out = p.y;
            const CUtensorMap* my = &map_y;
            if constexpr (kGrouped) { y_out = group.y[prob]; my = &group.maps[3 * prob + 2]; }
            const bool vec32 = (p.N % 4 == 0) && (((uintptr_t)y_out & 15) == 0);
            const bool vec16 = (p.N % 8 == 0) && (((uintptr_t)y_out & 15) == 0);
            const uint32_t buf = iter & 1, acc_phase = (iter >> 1) & 1;
            if (!ptx::mbar_wait(ptx::smem_u32(&tmem_full_bar[buf]), acc_phase, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | (int)(w & 0xFFFFFF));
                break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t row_base = wi.m_blk * BM + quarter * 32;
#pragma unroll 1
            for (uint32_t c = 0; c < BN / 32; ++c) {
                const uint32_t col0 = wi.n_blk * BN + c * 32;
                if (col0 >= p.N) break;   // warp-uniform
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + ((quarter * 32) << 16) + buf * BN + c * 32, r);
                ptx::tmem_ld_wait();
                store_chunk(p, r, row_base, lane, col0, wi.split, vec32, vec16, epi_stage + quarter * 2 * kEpiStageBytes, n_stores,
                            p.tma_store ? my : nullptr, y_out);
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tmem_empty_bar[buf]));
        }
        if (p.tma_store && lane == 0) ptx::bulk_wait_group_all();   // this warp's stores are complete before shared memory goes away
    }

    // ---------------------------------------------------------------- common exit
    __syncwarp();
    probe.end(p);
    if (*abort_flag) {
        // give copies and UMMAs already in flight time to land before shared and tensor memory go away
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------ host side

template <uint32_t BN, bool B_MN, bool kGrouped = false>
int launch_instance(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& my, const KParams& p, uint32_t grid, cudaStream_t stream,
                    const std::conditional_t<kGrouped, GroupOperands3, NoGroup>& group = {}) {
    auto kern = gemm_bf16_tcgen05_kernel<BN, B_MN, kGrouped>;
    const uint32_t smem = gemm_smem_bytes(BN);
    static bool attr_set[64] = {};   // per instantiation, per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(T0_ERR_CUDA, "cudaFuncSetAttribute(smem=%u): %s", smem, cudaGetErrorString(e));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    cudaError_t e = launch_pdl(kern, grid, kThreads, smem, stream, ma, mb, my, p, group);
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "GEMM kernel launch failed: %s", cudaGetErrorString(e));
    return T0_OK;
}

}  // namespace

uint32_t gemm_stage_count(uint32_t tile_n) { return stages_for(snap_tile_n(tile_n)); }

uint32_t gemm_smem_bytes(uint32_t tile_n) {
    const uint32_t bn = snap_tile_n(tile_n);
    // tiles + barriers/holder (256 B) + the epilogue warps' staging chunks + slack for the 1024-byte alignment of the dynamic segment
    return stages_for(bn) * (kAStageBytes + bn * BK * 2) + 256 + 8 * kEpiStageBytes + 1024;
}

int launch_gemm_sm100(const GemmLaunch& g, cudaStream_t stream) {
    if (g.m == 0 || g.n == 0) return T0_OK;
    if (g.k == 0) return fail(T0_ERR_INVALID, "K must be positive");
    const uint32_t split = g.split_k ? g.split_k : 1;
    if (g.k % split) return fail(T0_ERR_UNSUPPORTED, "K=%u not divisible by split_k=%u", g.k, split);
    const uint32_t kps = g.k / split;
    const uint32_t ldx = g.ldx ? g.ldx : g.k;
    const uint32_t ldb = g.ldb ? g.ldb : (g.nn ? g.n : g.k);
    if ((ldx % 8) || (ldb % 8) || (split > 1 && (kps % 8)))
        return fail(T0_ERR_UNSUPPORTED, "row strides (%u, %u) and, with split-K, K per split (%u) must be multiples of 8 for the TMA path", ldx, ldb, kps);
    if (((uintptr_t)g.x & 15) || ((uintptr_t)g.b & 15)) return fail(T0_ERR_UNSUPPORTED, "operand pointers must be 16-byte aligned");
    const uint32_t bn = snap_tile_n(g.tile_n);
    if (g.nn && bn < 64) return fail(T0_ERR_UNSUPPORTED, "NN layout needs tile_n >= 64");

    KParams p;
    memset(&p, 0, sizeof p);
    p.wait_limit_ns = g.wait_limit_ns ? g.wait_limit_ns : ptx::kWaitLimitNs; p.drop_load = g.drop_load ? 1 : 0;
    p.y = g.y; p.bias = g.bias; p.status = g.status; p.probe = g.probe; p.trace = nullptr; p.plane_stride = g.plane_stride;
    p.M = g.m; p.N = g.n; p.K = g.k;
    p.tiles_m = ceil_div(g.m, BM); p.tiles_n = ceil_div(g.n, bn); p.split_k = split;
    p.kb_per_split = ceil_div(kps, BK);
    p.swap_grid = g.swap_grid ? 1 : 0; p.raster_group = 8;
    p.out_bf16 = g.out_bf16 ? 1 : 0; p.epilogue = g.epilogue; p.n_ops = g.n_ops;
    p.scale = g.scale; p.clamp_min = g.clamp_min; p.clamp_max = g.clamp_max;
    memcpy(p.ops, g.ops, sizeof p.ops);

    CUtensorMap ma, mb;
    int rc = make_map_kmajor(&ma, g.x, g.m, ldx, kps, split, BM);
    if (rc != T0_OK) return rc;
    rc = g.nn ? make_map_nmajor(&mb, g.b, g.n, ldb, kps, split) : make_map_kmajor(&mb, g.b, g.n, ldb, kps, split, bn);
    if (rc != T0_OK) return rc;

    const uint64_t total = (uint64_t)p.tiles_m * p.tiles_n * split;
    if (total > 0x7FFFFFFFull) return fail(T0_ERR_UNSUPPORTED, "too many tiles");
    const uint32_t grid = (uint32_t)std::min<uint64_t>(total, g.n_sms ? g.n_sms : 148);
    // f32 output the TMA unit can address (16-byte aligned base, row pitch and plane pitch): full chunks leave as TMA stores
    static const bool no_tma_store = getenv("T0_NO_TMA_STORE") != nullptr;
    CUtensorMap my = ma;   // a valid map either way; only read when p.tma_store is set
    if (!no_tma_store && !g.out_bf16 && g.n % 4 == 0 && ((uintptr_t)g.y & 15) == 0 && (split == 1 || g.plane_stride % 4 == 0)) {
        rc = make_map_out_f32(&my, g.y, g.m, g.n, split, g.plane_stride);
        if (rc != T0_OK) return rc;
        p.tma_store = 1;
    }
    rc = stage_peer_maps(g, p, split, stream);
    if (rc != T0_OK) return rc;

    if (g.nn) {
        switch (bn) {
            case 64: return launch_instance<64, true>(ma, mb, my, p, grid, stream);
            case 128: return launch_instance<128, true>(ma, mb, my, p, grid, stream);
            default: return launch_instance<256, true>(ma, mb, my, p, grid, stream);
        }
    }
    switch (bn) {
        case 32: return launch_instance<32, false>(ma, mb, my, p, grid, stream);
        case 64: return launch_instance<64, false>(ma, mb, my, p, grid, stream);
        case 128: return launch_instance<128, false>(ma, mb, my, p, grid, stream);
        default: return launch_instance<256, false>(ma, mb, my, p, grid, stream);
    }
}

// Several problems of one shape, no split-K, NT layout, 64- or 128-wide tiles, in one launch: the persistent CTAs walk the
// tiles of all the problems (see kernels.h).  Every problem must qualify for the TMA path (16-byte aligned operands, K % 8).
int launch_gemm_sm100_grouped(const GemmLaunch* gs, uint32_t count, cudaStream_t stream) {
    if (!gs || count == 0) return T0_OK;
    if (count > kMaxGroupedGemms) return fail(T0_ERR_INVALID, "at most %u problems per grouped launch (got %u)", kMaxGroupedGemms, count);
    const GemmLaunch& g0 = gs[0];
    if (g0.m == 0 || g0.n == 0) return T0_OK;
    const uint32_t bn = snap_tile_n(g0.tile_n);
    if (g0.nn || (g0.split_k > 1) || (bn != 64 && bn != 128) || g0.k == 0 || g0.k % 8 || g0.n_peer_y)
        return fail(T0_ERR_UNSUPPORTED, "grouped launch: NT layout, no split-K, tile width 64 or 128, K a positive multiple of 8");
    const uint32_t ldx = g0.ldx ? g0.ldx : g0.k, ldb = g0.ldb ? g0.ldb : g0.k;
    if ((ldx % 8) || (ldb % 8)) return fail(T0_ERR_UNSUPPORTED, "grouped launch: row strides must be multiples of 8");
    KParams p;
    memset(&p, 0, sizeof p);
    p.wait_limit_ns = g0.wait_limit_ns ? g0.wait_limit_ns : ptx::kWaitLimitNs;
    p.y = g0.y; p.bias = g0.bias; p.status = g0.status; p.probe = g0.probe;
    p.M = g0.m; p.N = g0.n; p.K = g0.k;
    p.tiles_m = ceil_div(g0.m, BM); p.tiles_n = ceil_div(g0.n, bn); p.split_k = 1;
    p.kb_per_split = ceil_div(g0.k, BK);
    p.swap_grid = g0.swap_grid ? 1 : 0; p.raster_group = 8;
    p.out_bf16 = g0.out_bf16 ? 1 : 0; p.epilogue = g0.epilogue; p.n_ops = g0.n_ops;
    p.scale = g0.scale; p.clamp_min = g0.clamp_min; p.clamp_max = g0.clamp_max;
    memcpy(p.ops, g0.ops, sizeof p.ops);
    p.n_problems = count;
    static const bool no_tma_store = getenv("T0_NO_TMA_STORE") != nullptr;
    bool tma_store = !no_tma_store && !g0.out_bf16 && g0.n % 4 == 0;
    for (uint32_t i = 0; i < count; ++i) tma_store = tma_store && (((uintptr_t)gs[i].y & 15) == 0);
    p.tma_store = tma_store ? 1 : 0;
    static GroupOperands3 group;         // 12.5 KB: kept off the stack, filled under the lock, copied by the launch
    static std::mutex group_mu;
    std::lock_guard<std::mutex> lock(group_mu);
    for (uint32_t i = 0; i < count; ++i) {
        const GemmLaunch& g = gs[i];
        if (g.m != g0.m || g.n != g0.n || g.k != g0.k || g.ldx != g0.ldx || g.ldb != g0.ldb || g.tile_n != g0.tile_n || g.split_k != g0.split_k ||
            g.nn != g0.nn || g.out_bf16 != g0.out_bf16 || g.swap_grid != g0.swap_grid || g.epilogue != g0.epilogue || g.n_ops != g0.n_ops ||
            memcmp(g.ops, g0.ops, sizeof g.ops) != 0 || g.scale != g0.scale || g.clamp_min != g0.clamp_min || g.clamp_max != g0.clamp_max ||
            g.bias != g0.bias)
            return fail(T0_ERR_INVALID, "grouped launch: problem %u differs from problem 0 in shape or configuration", i);
        if (!g.x || !g.b || !g.y) return fail(T0_ERR_INVALID, "grouped launch: null pointer in problem %u", i);
        if (((uintptr_t)g.x & 15) || ((uintptr_t)g.b & 15)) return fail(T0_ERR_UNSUPPORTED, "grouped launch: operands of problem %u are not 16-byte aligned", i);
        int rc = make_map_kmajor(&group.maps[3 * i], g.x, g.m, ldx, g.k, 1, BM);
        if (rc == T0_OK) rc = make_map_kmajor(&group.maps[3 * i + 1], g.b, g.n, ldb, g.k, 1, bn);
        if (rc != T0_OK) return rc;
        group.maps[3 * i + 2] = group.maps[3 * i];          // a valid map either way; only read when p.tma_store is set
        if (tma_store) {
            rc = make_map_out_f32(&group.maps[3 * i + 2], g.y, g.m, g.n, 1, 0);
            if (rc != T0_OK) return rc;
        }
        group.y[i] = g.y;
    }
    const uint64_t total = (uint64_t)p.tiles_m * p.tiles_n * count;
    if (total > 0x7FFFFFFFull) return fail(T0_ERR_UNSUPPORTED, "too many tiles");
    const uint32_t grid = (uint32_t)std::min<uint64_t>(total, g0.n_sms ? g0.n_sms : 148);
    return bn == 128 ? launch_instance<128, false, true>(group.maps[0], group.maps[1], group.maps[2], p, grid, stream, group)
                     : launch_instance<64, false, true>(group.maps[0], group.maps[1], group.maps[2], p, grid, stream, group);
}

}  // namespace t0

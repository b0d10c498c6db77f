// K1 (CTA-pair form) — the same bf16 GEMM as gemm_sm100.cu with two CTAs of a cluster sharing one
// 256 x 256 output tile through tcgen05 cta_group::2.  This is what the reference's `wgp_mode`
// (one workgroup spanning two compute units, src/t0/gemm_gen.rs:78-79) maps to on B200.
//
// Why: with one CTA per 128 x 256 tile every SM pulls 48 KiB from L2 per k-block; in a pair each CTA
// loads its 128 rows of A and only its 128 of the 256 rows of B (32 KiB per k-block for the same
// math), the tensor cores read the other half of B from the partner's shared memory.  A third less
// L2->SM traffic and a deeper ring (6 stages) for the same shared-memory budget.
//
// Roles per CTA are those of the single-CTA kernel.  Differences:
//   * both CTAs' TMA loads credit the EVEN CTA's `full` barrier (it expects the bytes of both);
//   * only the even CTA issues UMMAs; it commits to the `empty`/`tmem_full` barriers of both CTAs
//     (two plain commits, one per CTA);
//   * the odd CTA's epilogue warps arrive on the even CTA's `tmem_empty` barrier;
//   * a cluster barrier brackets the kernel so no CTA leaves while its partner can still touch it.
// No TMA load here is a cluster-wide broadcast: every CTA fetches its own tiles.
#include "gemm_common.cuh"

namespace t0 {

namespace {

using namespace gemm;
constexpr uint32_t kThreads = 192;   // producer, UMMA issuer, four epilogue warps
constexpr uint32_t kPairM = 256;         // output rows per pair

__host__ __device__ constexpr uint32_t pair_stages(uint32_t pair_n) { return pair_n == 256 ? 6 : 8; }

// kPairN = output columns per pair (256, or 128 when 256-wide tiles would quantise badly over the SMs)
// B_MN = B is given as B[K,N] (N contiguous): each CTA then loads its half of the columns as 64(k) x 64(n) boxes and the
// UMMA reads B through an MN-major descriptor, exactly as the single-CTA kernel does; `map_b_half` is unused (the boxes
// are 64 columns wide whatever the tile).
template <uint32_t kPairN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                              const __grid_constant__ CUtensorMap map_b_half, const __grid_constant__ CUtensorMap map_y, const KParams p) {
    constexpr uint32_t kBHalfRows = kPairN / 2;                    // rows of B each CTA loads
    constexpr uint32_t kBStageBytes = kBHalfRows * BK * 2;
    constexpr uint32_t kStageBytes = kAStageBytes + kBStageBytes;  // per CTA
    constexpr uint32_t kStages = pair_stages(kPairN);
    constexpr uint32_t kTmemCols = 2 * kPairN;                     // two accumulator buffers
    constexpr uint32_t kIdesc = ptx::make_idesc_bf16_f32(kPairM, kPairN, B_MN ? 1u : 0u);
    // Tail of the tile list: when the last wave would leave more than half of the pairs idle, its tiles are cut into two
    // half-width tiles (work items >= p.tail_start; item tail_start + 2i + h is half h of tile tail_start + i), so the wave
    // costs a half-width tile instead of a full one.  B then comes through a tensor map with a box half as tall.
    constexpr uint32_t kHalfN = kPairN / 2;
    constexpr uint32_t kIdescHalf = ptx::make_idesc_bf16_f32(kPairM, kHalfN, B_MN ? 1u : 0u);
    constexpr uint32_t kBHalfStageBytes = (kHalfN / 2) * BK * 2;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + kStages * kAStageBytes;
    uint8_t* epi_stage = smem + kStages * kStageBytes;          // 4 warps x 2 blocks of kEpiStageBytes; 1024-byte aligned
    uint64_t* bars = (uint64_t*)(epi_stage + 8 * kEpiStageBytes);
    uint64_t* full_bar = bars;                          // used in the even CTA only
    uint64_t* empty_bar = bars + kStages;
    uint64_t* tmem_full_bar = bars + 2 * kStages;
    uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;  // used in the even CTA only
    uint32_t* tmem_holder = (uint32_t*)(bars + 2 * kStages + 4);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = ptx::cluster_ctarank();   // 0 = even CTA (issues the UMMAs), 1 = odd
    const uint32_t pair_id = blockIdx.x >> 1;
    const uint32_t n_pairs = gridDim.x >> 1;
    const uint32_t n_tiles = p.tiles_m * p.tiles_n * p.split_k;
    const uint32_t tail_start = min(p.tail_start, n_tiles);
    const uint32_t total_work = tail_start + 2 * (n_tiles - tail_start);

    if (threadIdx.x == 0) {
        trace_stamp(p, 0);
        for (uint32_t s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&tmem_full_bar[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&tmem_empty_bar[b]), 8);   // four epilogue warps in each CTA
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::tma_prefetch_desc(&map_a);
        ptx::tma_prefetch_desc(&map_b);
        if (p.tma_store) ptx::tma_prefetch_desc(&map_y);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_holder), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();          // both CTAs' barriers exist before anyone signals across the pair
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    // everything above touched only shared and tensor memory; global memory comes after the previous grid is done
    if (threadIdx.x == 0) trace_stamp(p, 2);
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    if (threadIdx.x == 0) trace_stamp(p, 1);
    ClockProbe probe;
    probe.begin(p);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t w = pair_id; ok && w < total_work; w += n_pairs) {
                const bool tail = w >= tail_start;
                const uint32_t half = tail ? ((w - tail_start) & 1u) : 0u;
                const WorkItem wi = decode_work(tail ? tail_start + ((w - tail_start) >> 1) : w, p);
                for (uint32_t kb = 0; kb < p.kb_per_split; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.wait_limit_ns)) {
                        atomicCAS(p.status, 0, kStatusProducerTimeout | (int)(w & 0xFFFFFF));
                        ok = false;
                        break;
                    }
                    const uint32_t fb_local = ptx::smem_u32(&full_bar[stage]);
                    // self-test of the failure path: neither CTA of pair 0 fills this stage, so the issuer's bounded wait must run out
                    if (p.drop_load && pair_id == 0 && w == 0 && kb == 0) { if (++stage == kStages) { stage = 0; phase ^= 1; } continue; }
                    if (cta_rank == 0) ptx::mbar_arrive_expect_tx(fb_local, 2 * (kAStageBytes + (tail ? kBHalfStageBytes : kBStageBytes)));   // bytes of both CTAs
                    const uint32_t fb = ptx::mapa(fb_local, 0);   // the even CTA's barrier, from either CTA
                    ptx::tma_load_3d_pair(ptx::smem_u32(a_tiles + stage * kAStageBytes), &map_a, fb,
                                          (int32_t)(kb * BK), (int32_t)(wi.m_blk * kPairM + cta_rank * BM), (int32_t)wi.split);
                    if constexpr (B_MN) {
                        // this CTA's columns of B[K,N]: one 64(k) x 64(n) box (a [k][128 B] block) per 64 columns
                        const uint32_t cols = tail ? kHalfN / 2 : kBHalfRows;
                        const uint32_t n0 = wi.n_blk * kPairN + (tail ? half * kHalfN : 0) + cta_rank * cols;
                        for (uint32_t j = 0; j < cols / 64; ++j)
                            ptx::tma_load_3d_pair(ptx::smem_u32(b_tiles + stage * kBStageBytes + j * (BK * 128)), &map_b, fb,
                                                  (int32_t)(n0 + j * 64), (int32_t)(kb * BK), (int32_t)wi.split);
                    } else if (!tail) {
                        ptx::tma_load_3d_pair(ptx::smem_u32(b_tiles + stage * kBStageBytes), &map_b, fb,
                                              (int32_t)(kb * BK), (int32_t)(wi.n_blk * kPairN + cta_rank * kBHalfRows), (int32_t)wi.split);
                    } else {
                        ptx::tma_load_3d_pair(ptx::smem_u32(b_tiles + stage * kBStageBytes), &map_b_half, fb,
                                              (int32_t)(kb * BK), (int32_t)(wi.n_blk * kPairN + half * kHalfN + cta_rank * (kHalfN / 2)), (int32_t)wi.split);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer (even CTA only)
        if (lane == 0 && cta_rank == 0) {
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t w = pair_id; ok && w < total_work; w += n_pairs, ++iter) {
                const uint32_t buf = iter & 1, acc_phase = (iter >> 1) & 1;
                if (!ptx::mbar_wait(ptx::smem_u32(&tmem_empty_bar[buf]), acc_phase ^ 1, abort_flag, p.wait_limit_ns)) {
                    atomicCAS(p.status, 0, kStatusMmaTimeout | (int)(w & 0xFFFFFF));
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + buf * kPairN;
                const uint32_t idesc = w >= tail_start ? kIdescHalf : kIdesc;
                for (uint32_t kb = 0; kb < p.kb_per_split; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag, p.wait_limit_ns)) {
                        atomicCAS(p.status, 0, kStatusMmaTimeout | 0x800000 | (int)(w & 0x7FFFFF));
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    if (kb == 0 && w == pair_id) trace_stamp(p, 3);
                    const uint32_t a_addr = ptx::smem_u32(a_tiles + stage * kAStageBytes);
                    const uint32_t b_addr = ptx::smem_u32(b_tiles + stage * kBStageBytes);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < BK / 16; ++k4) {
                        const uint64_t da = ptx::make_smem_desc(a_addr + k4 * 32, 16, 1024);
                        // N-major B: 64-column atoms 8 KiB apart, 8-row k groups 1024 B apart; a K step is two groups
                        const uint64_t db = B_MN ? ptx::make_smem_desc(b_addr + k4 * 2048, BK * 128, 1024)
                                                 : ptx::make_smem_desc(b_addr + k4 * 32, 16, 1024);
                        ptx::umma_bf16_ss_pair(tmem_d, da, db, idesc, (kb | k4) != 0 ? 1u : 0u);
                    }
                    // the stage is free in both CTAs once these UMMAs have read it
                    const uint32_t eb = ptx::smem_u32(&empty_bar[stage]);
                    ptx::umma_commit_pair(eb);
                    ptx::umma_commit_pair(ptx::mapa(eb, 1));
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (ok) {
                    const uint32_t tb = ptx::smem_u32(&tmem_full_bar[buf]);
                    ptx::umma_commit_pair(tb);
                    ptx::umma_commit_pair(ptx::mapa(tb, 1));
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const uint32_t quarter = warp & 3;          // tensor-memory lanes 32*quarter .. +31 are the ones this warp may read
        const bool vec32 = (p.N % 4 == 0) && (((uintptr_t)p.y & 15) == 0);
        const bool vec16 = (p.N % 8 == 0) && (((uintptr_t)p.y & 15) == 0);
        uint32_t iter = 0, n_stores = 0;     // n_stores: this warp's committed TMA stores, see store_chunk
        for (uint32_t w = pair_id; w < total_work; w += n_pairs, ++iter) {
            const bool tail = w >= tail_start;
            const uint32_t half = tail ? ((w - tail_start) & 1u) : 0u;
            const WorkItem wi = decode_work(tail ? tail_start + ((w - tail_start) >> 1) : w, p);
            const uint32_t n_chunks = tail ? kHalfN / 32 : kPairN / 32;
            const uint32_t buf = iter & 1, acc_phase = (iter >> 1) & 1;
            if (!ptx::mbar_wait(ptx::smem_u32(&tmem_full_bar[buf]), acc_phase, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | (int)(w & 0xFFFFFF));
                break;
            }
            ptx::tc_fence_after_sync();
            if (iter == 0 && threadIdx.x == 64) trace_stamp(p, 4);
            const uint32_t row_base = wi.m_blk * kPairM + cta_rank * BM + quarter * 32;
#pragma unroll 1
            for (uint32_t c = 0; c < n_chunks; ++c) {
                const uint32_t col0 = wi.n_blk * kPairN + half * kHalfN + c * 32;
                if (col0 >= p.N) break;
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + ((quarter * 32) << 16) + buf * kPairN + c * 32, r);
                ptx::tmem_ld_wait();
                store_chunk(p, r, row_base, lane, col0, wi.split, vec32, vec16, epi_stage + quarter * 2 * kEpiStageBytes, n_stores, p.tma_store ? &map_y : nullptr);
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                const uint32_t te = ptx::smem_u32(&tmem_empty_bar[buf]);
                if (cta_rank == 0) ptx::mbar_arrive(te);
                else ptx::mbar_arrive_cluster(ptx::mapa(te, 0));
            }
        }
        if (p.tma_store && lane == 0) ptx::bulk_wait_group_all();   // this warp's stores are complete before shared memory goes away
        if (threadIdx.x == 64) trace_stamp(p, 5);
    }

    // ---------------------------------------------------------------- common exit
    __syncwarp();
    probe.end(p);
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();          // the partner is done with this CTA's barriers and tensor memory
    if (threadIdx.x == 0) trace_stamp(p, 6);
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

}  // namespace

uint32_t gemm_pair_smem_bytes(uint32_t pair_n) {
    return pair_stages(pair_n) * (kAStageBytes + (pair_n / 2) * BK * 2) + 256 + 8 * kEpiStageBytes + 1024;
}

namespace {

template <uint32_t kPairN, bool B_MN>
int launch_pair_instance(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb_half, const CUtensorMap& my, KParams p, uint64_t total, uint32_t n_sms,
                         cudaStream_t stream) {
    auto kern = gemm_bf16_tcgen05_pair_kernel<kPairN, B_MN>;
    const uint32_t smem = gemm_pair_smem_bytes(kPairN);
    static bool attr_set[64] = {};
    static int max_pairs[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(T0_ERR_INVALID, "device ordinal out of range");
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(T0_ERR_CUDA, "cudaFuncSetAttribute(smem=%u): %s", smem, cudaGetErrorString(e));
        // how many two-CTA clusters the device can hold at once (SMs pair up within a GPC)
        cudaLaunchConfig_t qc = {};
        qc.gridDim = dim3(2 * (n_sms / 2), 1, 1);
        qc.blockDim = dim3(kThreads, 1, 1);
        qc.dynamicSmemBytes = smem;
        int n_clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&n_clusters, kern, &qc);
        if (e != cudaSuccess || n_clusters <= 0) { cudaGetLastError(); n_clusters = (int)n_sms / 2; }
        max_pairs[dev] = n_clusters;
        attr_set[dev] = true;
    }
    const uint32_t pairs = (uint32_t)std::min<uint64_t>(total, (uint64_t)max_pairs[dev]);
    // last wave: `rest` tiles for `pairs` pairs; cut them in two when both halves still fit in one wave
    const uint32_t rest = (uint32_t)(total % pairs);
    static const bool no_tail = getenv("T0_NO_TAIL_SPLIT") != nullptr;
    p.tail_start = (uint32_t)total;
    const bool tail_ok = !(B_MN && kPairN == 128);   // B[K,N] boxes are 64 columns wide: a quarter of a 128-wide tile is too narrow
    if (!no_tail && tail_ok && p.split_k == 1 && total > pairs && rest != 0 && 2 * rest <= pairs) p.tail_start = (uint32_t)total - rest;
    cudaError_t e = launch_pdl(kern, 2 * pairs, kThreads, smem, stream, ma, mb, mb_half, my, p);
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "pair GEMM kernel launch failed: %s", cudaGetErrorString(e));
    return T0_OK;
}

}  // namespace

// Pair-tile launch: NT layout, 256 x 256 tiles (256 x 128 when g.tile_n <= 128).  Same argument checks as the single-CTA launch.
int launch_gemm_sm100_pair(const GemmLaunch& g, cudaStream_t stream) {
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

    const uint32_t pair_n = g.tile_n && g.tile_n <= 128 ? 128 : 256;
    KParams p;
    memset(&p, 0, sizeof p);
    p.wait_limit_ns = g.wait_limit_ns ? g.wait_limit_ns : ptx::kWaitLimitNs; p.drop_load = g.drop_load ? 1 : 0;
    p.y = g.y; p.bias = g.bias; p.status = g.status; p.probe = g.probe; p.plane_stride = g.plane_stride;
    {
        // T0_GEMM_TRACE=1: a ring of eight launches' stamps behind the two clock words (printed by t0_rt_last_kernel_clock)
        static const bool tracing = getenv("T0_GEMM_TRACE") != nullptr;
        static unsigned n_traced = 0;
        p.trace = (tracing && g.probe) ? g.probe + 2 + 8 * (n_traced++ % 8) : nullptr;
    }
    p.M = g.m; p.N = g.n; p.K = g.k;
    p.tiles_m = ceil_div(g.m, kPairM); p.tiles_n = ceil_div(g.n, pair_n); p.split_k = split;
    p.kb_per_split = ceil_div(kps, BK);
    p.swap_grid = g.swap_grid ? 1 : 0; p.raster_group = 8;
    p.out_bf16 = g.out_bf16 ? 1 : 0; p.epilogue = g.epilogue; p.n_ops = g.n_ops;
    p.scale = g.scale; p.clamp_min = g.clamp_min; p.clamp_max = g.clamp_max;
    memcpy(p.ops, g.ops, sizeof p.ops);

    CUtensorMap ma, mb;
    int rc = make_map_kmajor(&ma, g.x, g.m, ldx, kps, split, BM);
    if (rc != T0_OK) return rc;
    CUtensorMap mb_half;
    if (g.nn) {
        rc = make_map_nmajor(&mb, g.b, g.n, ldb, kps, split);
        mb_half = mb;
    } else {
        rc = make_map_kmajor(&mb, g.b, g.n, ldb, kps, split, pair_n / 2);
        if (rc != T0_OK) return rc;
        rc = make_map_kmajor(&mb_half, g.b, g.n, ldb, kps, split, pair_n / 4);
    }
    if (rc != T0_OK) return rc;
    const uint64_t total = (uint64_t)p.tiles_m * p.tiles_n * split;
    if (total > 0x7FFFFFFFull) return fail(T0_ERR_UNSUPPORTED, "too many tiles");
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
    const uint32_t n_sms = g.n_sms ? g.n_sms : 148;
    if (g.nn)
        return pair_n == 256 ? launch_pair_instance<256, true>(ma, mb, mb_half, my, p, total, n_sms, stream)
                             : launch_pair_instance<128, true>(ma, mb, mb_half, my, p, total, n_sms, stream);
    return pair_n == 256 ? launch_pair_instance<256, false>(ma, mb, mb_half, my, p, total, n_sms, stream)
                         : launch_pair_instance<128, false>(ma, mb, mb_half, my, p, total, n_sms, stream);
}

}  // namespace t0

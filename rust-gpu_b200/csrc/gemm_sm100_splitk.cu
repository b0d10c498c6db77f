// K1 with split-K inside one launch: the `split_k` CTAs that share an output tile form a thread-block cluster, each
// accumulates its part of K in tensor memory, and the partial sums are added through distributed shared memory.
//
// Replaces, for results that are wanted complete (not as planes), the two-launch form "GEMM into split_k planes, then a
// reduction pass": the reference leaves the planes to the host to add (src/t0/gemm_gen.rs:447-448,
// examples/test_gemm_correctness.rs:203-207); here the sum is the same fp32 sum of the per-split partial sums in split
// order, so results are bit-identical to that form and from run to run.  The skinny, HBM-bound shapes this serves
// (128 x 4096 x 4096, 64 x 4096 x 16384) spend a third of their time in the second launch and the gap before it.
//
// Roles per CTA as in gemm_sm100.cu (TMA producer, UMMA issuer, four epilogue warps, accumulators double-buffered in
// tensor memory).  Differences:
//   * the cluster, not the CTA, walks the tile list; the CTA's rank in the cluster is its split index;
//   * the epilogue warps park the finished 128 x BN fp32 accumulator in this CTA's shared memory (row pitch BN + 4 floats:
//     neither the row-wise writes nor the reads below have bank conflicts) and tell every CTA of the cluster so (one
//     remote mbarrier arrival per warp and CTA); CTA r then owns columns [r BN/split, (r+1) BN/split) of the tile: it
//     reads that column slice from every CTA of the cluster (ld.shared::cluster, plain loads - no multicast), adds in
//     split order, applies the epilogue and stores; a second round of arrivals keeps every CTA's copy alive until all
//     have read it.  Only the epilogue warps take part, so the producer and the issuer run ahead into the next tile.
// Every wait is bounded; a wait that runs out raises the abort flag and writes the status word the host reads.
#include "kernels.h"
#include "ptx_sm100.cuh"
#include <type_traits>
#include "gemm_common.cuh"

namespace t0 {

namespace {

using namespace gemm;
constexpr uint32_t kThreads = 192;

// Shared memory holds the operand ring and the parked accumulator.  A cluster that has one tile only (the skinny shapes: the
// tile count does not exceed the clusters the device holds) parks over the ring, which is idle by then, and so affords a
// deeper ring: what bounds these HBM-bound shapes is the bytes in flight per SM.
__host__ __device__ constexpr uint32_t sk_pitch(uint32_t bn) { return bn + 4; }                 // floats per parked row
__host__ __device__ constexpr uint32_t sk_park_bytes(uint32_t bn) { return BM * sk_pitch(bn) * 4; }
__host__ __device__ constexpr uint32_t sk_stage_bytes(uint32_t bn) { return kAStageBytes + bn * BK * 2; }
__host__ __device__ constexpr uint32_t sk_stages(uint32_t bn, bool alias) { return alias ? (bn == 128 ? 7u : 9u) : (bn == 128 ? 4u : 6u); }
__host__ __device__ constexpr uint32_t sk_bars_offset(uint32_t bn) {
    return sk_stages(bn, true) * sk_stage_bytes(bn) > sk_stages(bn, false) * sk_stage_bytes(bn) + sk_park_bytes(bn)
               ? sk_stages(bn, true) * sk_stage_bytes(bn) : sk_stages(bn, false) * sk_stage_bytes(bn) + sk_park_bytes(bn);
}
constexpr uint32_t kSkMaxStages = 9;

// wait with cluster-scope acquire: the arrivals come from other CTAs and order their shared-memory writes before our reads
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint64_t limit_ns) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    uint64_t t_start = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((spin & 0xFF) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = ptx::globaltimer_ns();
            if (t_start == 0) t_start = now;
            else if (now - t_start > limit_ns) { *abort_flag = 1; return false; }
        }
    }
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t n_clusters_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// Grouped launch: the tensor maps and outputs of up to kMaxGroupedGemms problems of one shape ride in the kernel parameters
// (8.4 KB; parameters may be 32 KB).  The single-problem kernel takes an empty record instead.
struct GroupOperands {
    CUtensorMap maps[2 * kMaxGroupedGemms];     // A, B of problem i at 2i, 2i + 1
    void* y[kMaxGroupedGemms];
};

template <uint32_t BN, bool kGrouped>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05_splitk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const KParams p,
                                const __grid_constant__ std::conditional_t<kGrouped, GroupOperands, NoGroup> group) {
    const uint32_t kStages = p.sk_stages;                  // 4 (6) with a parking area of its own, 7 (9) when the accumulator is parked over the ring
    constexpr uint32_t kBStageBytes = BN * BK * 2;
    constexpr uint32_t kStageBytes = kAStageBytes + kBStageBytes;
    constexpr uint32_t kTmemCols = 2 * BN;
    constexpr uint32_t kIdesc = ptx::make_idesc_bf16_f32(BM, BN, 0u);
    constexpr uint32_t kPitch = sk_pitch(BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + kStages * kAStageBytes;
    // [128][BN + 4] f32: this CTA's partial sums of the tile, behind the ring or (one tile per cluster) over it
    const uint32_t park = ptx::smem_u32(p.sk_alias ? smem : smem + kStages * kStageBytes);
    uint64_t* bars = (uint64_t*)(smem + sk_bars_offset(BN));
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + kSkMaxStages;
    uint64_t* tmem_full_bar = bars + 2 * kSkMaxStages;
    uint64_t* tmem_empty_bar = bars + 2 * kSkMaxStages + 2;
    uint64_t* parked_bar = bars + 2 * kSkMaxStages + 4;    // every epilogue warp of every CTA of the cluster has parked its rows of the tile
    uint64_t* read_bar = bars + 2 * kSkMaxStages + 5;      // ... has read this CTA's copy
    uint32_t* tmem_holder = (uint32_t*)(bars + 2 * kSkMaxStages + 6);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t split = ptx::cluster_ctarank();          // this CTA's part of K
    const uint32_t n_tiles = p.tiles_m * p.tiles_n;                                   // of one problem
    uint32_t n_items = n_tiles;                                                        // tiles of all the problems of the launch, problem-major
    if constexpr (kGrouped) n_items = n_tiles * p.n_problems;

    if (threadIdx.x == 0) {
        trace_stamp(p, 0);
        for (uint32_t s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }
        for (uint32_t b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&tmem_full_bar[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&tmem_empty_bar[b]), 4);
        }
        ptx::mbar_init(ptx::smem_u32(parked_bar), 4 * p.split_k);
        ptx::mbar_init(ptx::smem_u32(read_bar), 4 * p.split_k);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::tma_prefetch_desc(&map_a);
        ptx::tma_prefetch_desc(&map_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_holder), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();          // every CTA's barriers exist before anyone signals across the cluster
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    if (threadIdx.x == 0) trace_stamp(p, 2);
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    if (threadIdx.x == 0) trace_stamp(p, 1);
    ClockProbe probe;
    probe.begin(p);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t w = cluster_id_x(); ok && w < n_items; w += n_clusters_x()) {
                uint32_t prob = 0, tile = w;
                if constexpr (kGrouped) { prob = w / n_tiles; tile = w - prob * n_tiles; }
                const WorkItem wi = decode_work(tile * p.split_k, p);  // (the tile list carries no split: the rank is the split)
                const CUtensorMap* ma = &map_a;
                const CUtensorMap* mb = &map_b;
                if constexpr (kGrouped) { ma = &group.maps[2 * prob]; mb = &group.maps[2 * prob + 1]; }
                for (uint32_t kb = 0; kb < p.kb_per_split; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.wait_limit_ns)) {
                        atomicCAS(p.status, 0, kStatusProducerTimeout | (int)(w & 0xFFFFFF));
                        ok = false;
                        break;
                    }
                    const uint32_t fb = ptx::smem_u32(&full_bar[stage]);
                    ptx::mbar_arrive_expect_tx(fb, kStageBytes);
                    ptx::tma_load_3d(ptx::smem_u32(a_tiles + stage * kAStageBytes), ma, fb,
                                     (int32_t)(kb * BK), (int32_t)(wi.m_blk * BM), (int32_t)split);
                    ptx::tma_load_3d(ptx::smem_u32(b_tiles + stage * kBStageBytes), mb, fb,
                                     (int32_t)(kb * BK), (int32_t)(wi.n_blk * BN), (int32_t)split);
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t w = cluster_id_x(); ok && w < n_items; w += n_clusters_x(), ++iter) {
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
                    if (kb == 0 && iter == 0) trace_stamp(p, 3);
                    const uint32_t a_addr = ptx::smem_u32(a_tiles + stage * kAStageBytes);
                    const uint32_t b_addr = ptx::smem_u32(b_tiles + stage * kBStageBytes);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < BK / 16; ++k4) {
                        const uint64_t da = ptx::make_smem_desc(a_addr + k4 * 32, 16, 1024);
                        const uint64_t db = ptx::make_smem_desc(b_addr + k4 * 32, 16, 1024);
                        ptx::umma_bf16_ss(tmem_d, da, db, kIdesc, (kb | k4) != 0 ? 1u : 0u);
                    }
                    ptx::umma_commit(ptx::smem_u32(&empty_bar[stage]));
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (ok) ptx::umma_commit(ptx::smem_u32(&tmem_full_bar[buf]));
            }
        }
    }

    else {
        // ------------------------------------------------------------ epilogue warps 2..5: park, exchange, reduce, store
        const uint32_t quarter = warp & 3;
        const uint32_t n_split = p.split_k;
        const uint32_t cols_per = BN / n_split;             // columns of the tile this CTA reduces and stores
        const bool vec_shape = (p.N % 4 == 0) && !p.out_bf16;
        const uint32_t parked = ptx::smem_u32(parked_bar), readb = ptx::smem_u32(read_bar);
        bool ok = true;
        uint32_t iter = 0;
        for (uint32_t w = cluster_id_x(); w < n_items; w += n_clusters_x(), ++iter) {
            uint32_t prob = 0, tile = w;
            if constexpr (kGrouped) { prob = w / n_tiles; tile = w - prob * n_tiles; }
            const WorkItem wi = decode_work(tile * p.split_k, p);
            void* y_out = p.y;
            if constexpr (kGrouped) y_out = group.y[prob];
            const bool vec = vec_shape && (((uintptr_t)y_out & 15) == 0);
            const uint32_t buf = iter & 1, acc_phase = (iter >> 1) & 1;
            if (ok && !ptx::mbar_wait(ptx::smem_u32(&tmem_full_bar[buf]), acc_phase, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | (int)(w & 0xFFFFFF));
                ok = false;
            }
            // the copy of the previous tile has been read by everyone before it is overwritten
            if (ok && iter > 0 && !mbar_wait_cluster(readb, (iter - 1) & 1, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0x400000 | (int)(w & 0x3FFFFF));
                ok = false;
            }
            if (!ok) break;
            ptx::tc_fence_after_sync();
            if (iter == 0 && threadIdx.x == 64) trace_stamp(p, 4);
            {
                // park the accumulator: this lane holds row quarter*32 + lane, 32 columns per tcgen05.ld
                const uint32_t row = quarter * 32 + lane;
#pragma unroll 1
                for (uint32_t c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(tmem_base + ((quarter * 32) << 16) + buf * BN + c * 32, r);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(park + (row * kPitch + c * 32 + 4 * j) * 4), "r"(r[4 * j]),
                                     "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                                     : "memory");
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(ptx::smem_u32(&tmem_empty_bar[buf]));                         // the issuer may reuse the accumulator
                for (uint32_t s = 0; s < n_split; ++s) ptx::mbar_arrive_cluster(ptx::mapa(parked, s));   // tell every CTA (release, cluster scope)
            }
            if (!mbar_wait_cluster(parked, iter & 1, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0x800000 | (int)(w & 0x3FFFFF));
                ok = false;
                break;
            }
            {
                // this CTA's column slice: 128 rows x cols_per columns, four floats per lane; a warp instruction covers
                // 128 / cols_per rows.  Splits are added in split order.
                const uint32_t lanes_per_row = cols_per / 4;
                const uint32_t rows_per_inst = 32 / lanes_per_row;
                const uint32_t col_in = split * cols_per + (lane % lanes_per_row) * 4;      // within the tile
                const uint32_t col = wi.n_blk * BN + col_in;
                // Remote shared-memory loads take hundreds of cycles: the loads of kU row groups (kU x split of them) are all
                // issued before the first is used, so the slice costs a few round trips instead of one per row group.
                constexpr uint32_t kU = 4;
                for (uint32_t r0 = quarter * 32; r0 < quarter * 32 + 32; r0 += kU * rows_per_inst) {
                    float4 part[kU][8];
#pragma unroll
                    for (uint32_t u = 0; u < kU; ++u) {
                        const uint32_t row_in = r0 + u * rows_per_inst + lane / lanes_per_row;
                        const bool live = r0 + u * rows_per_inst < quarter * 32 + 32;
#pragma unroll
                        for (uint32_t s = 0; s < 8; ++s)
                            part[u][s] = (live && s < n_split) ? ld_cluster_f4(ptx::mapa(park + (row_in * kPitch + col_in) * 4, s)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (uint32_t u = 0; u < kU; ++u) {
                        if (r0 + u * rows_per_inst >= quarter * 32 + 32) break;
                        const uint32_t row_in = r0 + u * rows_per_inst + lane / lanes_per_row;
                        const uint32_t row = wi.m_blk * BM + row_in;
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (uint32_t s = 0; s < 8; ++s)
                            if (s < n_split) { acc.x += part[u][s].x; acc.y += part[u][s].y; acc.z += part[u][s].z; acc.w += part[u][s].w; }
                        if (row >= p.M || col >= p.N) continue;
                        float o[4] = {acc.x, acc.y, acc.z, acc.w};
                        if (p.n_ops) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) o[j] = apply_chain(o[j], (p.bias && col + j < p.N) ? __ldg(p.bias + col + j) : 0.0f, p);
                        } else if (p.epilogue != T0_EPI_STORE_F32) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                o[j] += (p.bias && col + j < p.N) ? __ldg(p.bias + col + j) : 0.0f;
                                if (p.epilogue == T0_EPI_BIAS_ADD_RELU_STORE_F32) o[j] = fmaxf(o[j], 0.0f);
                            }
                        }
                        const size_t off = (size_t)row * p.N + col;
                        if (vec && col + 4 <= p.N) {
                            *(float4*)((float*)y_out + off) = make_float4(o[0], o[1], o[2], o[3]);
                        } else {
                            for (int j = 0; j < 4; ++j) {
                                if (col + j >= p.N) break;
                                if (p.out_bf16) ((__nv_bfloat16*)y_out)[off + j] = __float2bfloat16_rn(o[j]);
                                else ((float*)y_out)[off + j] = o[j];
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0)
                for (uint32_t s = 0; s < n_split; ++s) ptx::mbar_arrive_cluster(ptx::mapa(readb, s));      // this warp has read every copy
        }
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
    ptx::cluster_sync_all();          // no CTA's shared memory goes away while a peer may still read its copy or signal its barriers
    if (threadIdx.x == 0) trace_stamp(p, 6);
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

uint32_t splitk_smem_bytes(uint32_t bn) { return sk_bars_offset(bn) + 256 + 1024; }

template <uint32_t BN, bool kGrouped>
int launch_splitk_instance(const CUtensorMap& ma, const CUtensorMap& mb, KParams p, uint32_t n_sms, cudaStream_t stream,
                           const std::conditional_t<kGrouped, GroupOperands, NoGroup>& group) {
    auto kern = gemm_bf16_tcgen05_splitk_kernel<BN, kGrouped>;
    const uint32_t smem = splitk_smem_bytes(BN);
    static bool attr_set[64] = {};
    static int max_clusters[64][9] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(T0_ERR_INVALID, "device ordinal out of range");
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(T0_ERR_CUDA, "cudaFuncSetAttribute(smem=%u): %s", smem, cudaGetErrorString(e));
        attr_set[dev] = true;
    }
    const uint32_t split = p.split_k;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (!max_clusters[dev][split]) {
        // how many clusters of this size the device can hold at once
        cfg.gridDim = dim3(split * (n_sms / split), 1, 1);
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess || n <= 0) { cudaGetLastError(); n = (int)(n_sms / split) * 3 / 4; }
        max_clusters[dev][split] = std::max(n, 1);
    }
    static const bool use_pdl = getenv("T0_NO_PDL") == nullptr;
    const uint32_t tiles = p.tiles_m * p.tiles_n * (kGrouped ? p.n_problems : 1u);
    const uint32_t clusters = std::min<uint32_t>(tiles, (uint32_t)max_clusters[dev][split]);
    p.sk_alias = tiles <= clusters ? 1 : 0;                 // one tile per cluster: the accumulator is parked over the idle ring
    p.sk_stages = sk_stages(BN, p.sk_alias != 0);
    cfg.gridDim = dim3(clusters * split, 1, 1);
    cfg.numAttrs = use_pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ma, mb, p, group);
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "split-K GEMM kernel launch failed: %s", cudaGetErrorString(e));
    return T0_OK;
}

}  // namespace

// Whether the cluster form takes this request: NT layout, 2 / 4 / 8 splits of whole 64-deep k blocks, tile width 64 or 128.
bool gemm_splitk_cluster_supported(const GemmLaunch& g) {
    const uint32_t split = g.split_k;
    if (g.nn || (split != 2 && split != 4 && split != 8)) return false;
    if (g.k % split || (g.k / split) % 8) return false;
    const uint32_t bn = snap_tile_n(g.tile_n);
    if (bn != 64 && bn != 128) return false;
    if (bn / split < 4 || (bn / split) % 4) return false;
    const uint32_t ldx = g.ldx ? g.ldx : g.k, ldb = g.ldb ? g.ldb : g.k;
    if ((ldx % 8) || (ldb % 8) || ((uintptr_t)g.x & 15) || ((uintptr_t)g.b & 15)) return false;
    return true;
}

namespace {

// The launch parameters and the two operand maps of one problem (shape already accepted by gemm_splitk_cluster_supported).
int splitk_params(const GemmLaunch& g, KParams* out, CUtensorMap* ma, CUtensorMap* mb) {
    const uint32_t split = g.split_k, kps = g.k / split;
    const uint32_t ldx = g.ldx ? g.ldx : g.k, ldb = g.ldb ? g.ldb : g.k;
    const uint32_t bn = snap_tile_n(g.tile_n);
    KParams p;
    memset(&p, 0, sizeof p);
    p.wait_limit_ns = g.wait_limit_ns ? g.wait_limit_ns : ptx::kWaitLimitNs;
    p.y = g.y; p.bias = g.bias; p.status = g.status; p.probe = g.probe;
    {
        // T0_GEMM_TRACE=1 (builds with -DT0_GEMM_TRACE): a ring of eight launches' stamps behind the two clock words
        static const bool tracing = getenv("T0_GEMM_TRACE") != nullptr;
        static unsigned n_traced = 0;
        p.trace = (tracing && g.probe) ? g.probe + 2 + 8 * (n_traced++ % 8) : nullptr;
    }
    p.M = g.m; p.N = g.n; p.K = g.k;
    p.tiles_m = ceil_div(g.m, BM); p.tiles_n = ceil_div(g.n, bn); p.split_k = split;
    p.kb_per_split = ceil_div(kps, BK);
    p.swap_grid = g.swap_grid ? 1 : 0; p.raster_group = 8;
    p.out_bf16 = g.out_bf16 ? 1 : 0; p.epilogue = g.epilogue; p.n_ops = g.n_ops;
    p.scale = g.scale; p.clamp_min = g.clamp_min; p.clamp_max = g.clamp_max;
    memcpy(p.ops, g.ops, sizeof p.ops);
    int rc = make_map_kmajor(ma, g.x, g.m, ldx, kps, split, BM);
    if (rc != T0_OK) return rc;
    rc = make_map_kmajor(mb, g.b, g.n, ldb, kps, split, bn);
    if (rc != T0_OK) return rc;
    *out = p;
    return T0_OK;
}

}  // namespace

int launch_gemm_sm100_splitk(const GemmLaunch& g, cudaStream_t stream) {
    if (g.m == 0 || g.n == 0) return T0_OK;
    if (!gemm_splitk_cluster_supported(g)) return fail(T0_ERR_UNSUPPORTED, "the cluster split-K kernel does not take this request");
    KParams p;
    CUtensorMap ma, mb;
    int rc = splitk_params(g, &p, &ma, &mb);
    if (rc != T0_OK) return rc;
    if ((uint64_t)p.tiles_m * p.tiles_n > 0x7FFFFFFFull) return fail(T0_ERR_UNSUPPORTED, "too many tiles");
    const uint32_t n_sms = g.n_sms ? g.n_sms : 148;
    const NoGroup none = {0};
    return snap_tile_n(g.tile_n) == 128 ? launch_splitk_instance<128, false>(ma, mb, p, n_sms, stream, none)
                                        : launch_splitk_instance<64, false>(ma, mb, p, n_sms, stream, none);
}

int launch_gemm_sm100_splitk_grouped(const GemmLaunch* gs, uint32_t count, cudaStream_t stream) {
    if (!gs || count == 0) return T0_OK;
    if (count > kMaxGroupedGemms) return fail(T0_ERR_INVALID, "at most %u problems per grouped launch (got %u)", kMaxGroupedGemms, count);
    const GemmLaunch& g0 = gs[0];
    if (g0.m == 0 || g0.n == 0) return T0_OK;
    if (!gemm_splitk_cluster_supported(g0)) return fail(T0_ERR_UNSUPPORTED, "the cluster split-K kernel does not take this request");
    static GroupOperands group;          // 8.4 KB: kept off the stack; launches are issued under the caller's lock
    static std::mutex group_mu;
    std::lock_guard<std::mutex> lock(group_mu);
    KParams p0;
    for (uint32_t i = 0; i < count; ++i) {
        const GemmLaunch& g = gs[i];
        // one shape and one configuration: only the operand and output addresses differ
        if (g.m != g0.m || g.n != g0.n || g.k != g0.k || g.ldx != g0.ldx || g.ldb != g0.ldb || g.tile_n != g0.tile_n || g.split_k != g0.split_k ||
            g.nn != g0.nn || g.out_bf16 != g0.out_bf16 || g.swap_grid != g0.swap_grid || g.epilogue != g0.epilogue || g.n_ops != g0.n_ops ||
            memcmp(g.ops, g0.ops, sizeof g.ops) != 0 || g.scale != g0.scale || g.clamp_min != g0.clamp_min || g.clamp_max != g0.clamp_max ||
            g.bias != g0.bias)
            return fail(T0_ERR_INVALID, "grouped launch: problem %u differs from problem 0 in shape or configuration", i);
        if (!g.x || !g.b || !g.y) return fail(T0_ERR_INVALID, "grouped launch: null pointer in problem %u", i);
        if (((uintptr_t)g.x & 15) || ((uintptr_t)g.b & 15)) return fail(T0_ERR_UNSUPPORTED, "grouped launch: operands of problem %u are not 16-byte aligned", i);
        KParams pi;
        int rc = splitk_params(g, &pi, &group.maps[2 * i], &group.maps[2 * i + 1]);
        if (rc != T0_OK) return rc;
        if (i == 0) p0 = pi;
        group.y[i] = g.y;
    }
    p0.n_problems = count;
    if ((uint64_t)p0.tiles_m * p0.tiles_n * count > 0x7FFFFFFFull) return fail(T0_ERR_UNSUPPORTED, "too many tiles");
    const uint32_t n_sms = g0.n_sms ? g0.n_sms : 148;
    return snap_tile_n(g0.tile_n) == 128 ? launch_splitk_instance<128, true>(group.maps[0], group.maps[1], p0, n_sms, stream, group)
                                         : launch_splitk_instance<64, true>(group.maps[0], group.maps[1], p0, n_sms, stream, group);
}

}  // namespace t0

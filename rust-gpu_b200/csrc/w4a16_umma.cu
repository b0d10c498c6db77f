// K2 for 16 < M <= 128: the fused W4A16 GEMM on tcgen05, weights in the row layout (packed[K/8][N], scales[K/G][N],
// zeros[K/G][N/8]), dequantisation in the main loop, no K x N scratch matrix.
//
// No counterpart kernel exists in the reference (its INT4 support stops at the stand-alone dequantisation kernels,
// src/t0/quant_kernels.rs:53-171).  y[m,n] = sum_k a[m,k] * w[k,n],  w = RNE_bf16((q - z) * s),  fp32 accumulate.
//
// One CTA owns a 256-column tile of y and a range of K; the CTAs that share a tile form a cluster and add their partial
// sums through distributed shared memory (split order, deterministic), as the split-K GEMM does.  Per 64-deep k chunk:
//   * the producer lane fetches the chunk's packed words (8 rows x 256 columns), its scales and zero points with three
//     TMA boxes into a ring of raw stages, and the chunk's activations with a fourth into the operand ring;
//   * sixteen dequantisation warps turn the words into bf16 (one LOP3 per nibble pair: 0x4300 | q is the bf16 128+q,
//     minus 128+z, times s - bit-identical to the oracle because (q-z)*s is rounded once) and write them as the UMMA's B
//     operand: 256 rows (n) x 64 k, K-major, 128-byte swizzle.  A packed word holds eight consecutive k of one column
//     and the nibble pairs come out as (k, k+4); four byte permutes put them back into k order, so that the activations
//     (the 128-row A operand) can come straight from global memory through TMA (rows beyond M are zero-filled);
//   * one thread issues four tcgen05.mma (128 x 256 x 16) per chunk into a 128 x 256 fp32 accumulator in tensor memory.
// At the end the sixteen warps read the accumulator, park it in shared memory (over the rings, idle by then), exchange
// across the cluster and store.  Every wait is bounded.
#include "w4a16_common.cuh"
#include <type_traits>

using namespace t0;
using namespace t0::w4;

namespace {

constexpr uint32_t kUmDqWarps = 16;
constexpr uint32_t kUmThreads = (kUmDqWarps + 2) * 32;      // + producer warp + issuer warp
constexpr uint32_t kUmBN = 256;                             // columns of y per tile
constexpr uint32_t kUmBK = 64;                              // k per chunk: one 128-byte swizzle atom of bf16
constexpr uint32_t kUmRawStages = 6;
constexpr uint32_t kUmRawBytes = 8 * kUmBN * 4 + kUmBN * 2 + (kUmBN / 8) * 4;      // 8832: words, scales, zero points
constexpr uint32_t kUmRawStride = 9216;                     // keeps every stage 1024-byte aligned
constexpr uint32_t kUmAbStages = 3;
constexpr uint32_t kUmBBytes = kUmBN * kUmBK * 2;           // 32 KiB
constexpr uint32_t kUmABytes = 128 * kUmBK * 2;             // 16 KiB
constexpr uint32_t kUmRingBytes = kUmRawStages * kUmRawStride + kUmAbStages * (kUmABytes + kUmBBytes);   // 202752
constexpr uint32_t kUmPitch = kUmBN + 4;                    // floats per parked row
constexpr uint32_t kUmParkBytes = 128 * kUmPitch * 4;       // 133120, over the rings
static_assert(kUmParkBytes <= kUmRingBytes, "the parked accumulator must fit over the rings");
constexpr uint32_t kUmSmem = kUmRingBytes + 512 + 1024;
constexpr uint32_t kUmTmemCols = 256;

struct UmParams {
    const uint16_t* a;
    float* y;
    int* status;
    uint64_t wait_limit_ns;
    uint32_t M, N, K;
    uint32_t group;          // k per scale / zero-point row (a multiple of 64)
    uint32_t n_tiles, n_chunks, split;
    uint32_t tiled;          // the weights are in the tile-major layout (3-D maps: column in tile, row, tile) instead of the row layout
#ifdef T0_UM_TRACE
    unsigned long long* trace;   // debugging build only: nanosecond stamps of CTA 0's roles, 6 x 64 chunks
#endif
    uint32_t n_problems;     // grouped launch: problems of one shape in this launch (their maps and outputs ride in the group record)
};

__device__ __forceinline__ bool um_try_wait_cluster(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ bool um_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint64_t limit_ns) {
    if (um_try_wait_cluster(bar, parity)) return true;
    uint64_t t_start = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (um_try_wait_cluster(bar, parity)) return true;
        if ((spin & 0xFF) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = ptx::globaltimer_ns();
            if (t_start == 0) t_start = now;
            else if (now - t_start > limit_ns) { *abort_flag = 1; return false; }
        }
    }
}
__device__ __forceinline__ uint32_t um_cluster_id() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t um_n_clusters() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t um_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t um_lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void um_sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ float4 um_ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

// Grouped launch: the four tensor maps (weights, scales, zero points, activations) and the output of up to 32 problems of
// one shape in the kernel parameters (16.6 KB).
constexpr uint32_t kUmMaxGroup = 32;
struct UmGroup {
    CUtensorMap maps[4 * kUmMaxGroup];
    float* y[kUmMaxGroup];
};

template <bool kGrouped>
__global__ void __launch_bounds__(kUmThreads, 1)
w4a16_umma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                  const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_a, const UmParams p,
                  const __grid_constant__ std::conditional_t<kGrouped, UmGroup, gemm::NoGroup> group) {
    // a grouped launch (no split of K: cluster of one) walks the column tiles of all its problems, problem-major
    uint32_t n_items = p.n_tiles;
    if constexpr (kGrouped) n_items = p.n_tiles * p.n_problems;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t raw_ring = smem;
    const uint32_t a_ring = smem + kUmRawStages * kUmRawStride;
    const uint32_t b_ring = a_ring + kUmAbStages * kUmABytes;
    const uint32_t park = smem;                                   // [128][260] f32 over the rings, used when they are idle
    const uint32_t bars = smem + kUmRingBytes;
    const uint32_t raw_full = bars, raw_empty = bars + 8 * kUmRawStages;
    const uint32_t ab_full = raw_empty + 8 * kUmRawStages, ab_empty = ab_full + 8 * kUmAbStages;
    const uint32_t acc_full = ab_empty + 8 * kUmAbStages, acc_empty = acc_full + 8;
    const uint32_t parked_bar = acc_empty + 8, read_bar = parked_bar + 8;
    __shared__ uint32_t tmem_holder;
    __shared__ int s_abort;
    volatile int* abort_flag = &s_abort;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t split = ptx::cluster_ctarank();
    const uint32_t c_begin = (uint32_t)((uint64_t)split * p.n_chunks / p.split), c_end = (uint32_t)((uint64_t)(split + 1) * p.n_chunks / p.split);
    const uint32_t my_chunks = c_end - c_begin;

    if (tid == 0) {
        for (uint32_t s = 0; s < kUmRawStages; ++s) {
            ptx::mbar_init(raw_full + 8 * s, 1);
            ptx::mbar_init(raw_empty + 8 * s, kUmDqWarps / 2);    // the eight warps of the group that dequantises the chunk
        }
        for (uint32_t s = 0; s < kUmAbStages; ++s) {
            ptx::mbar_init(ab_full + 8 * s, kUmDqWarps / 2 + 1);  // eight warps' weights + the activations' bytes (producer)
            ptx::mbar_init(ab_empty + 8 * s, 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, kUmDqWarps);
        ptx::mbar_init(parked_bar, kUmDqWarps * p.split);
        ptx::mbar_init(read_bar, kUmDqWarps * p.split);
        s_abort = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::tma_prefetch_desc(&map_w);
        ptx::tma_prefetch_desc(&map_s);
        ptx::tma_prefetch_desc(&map_z);
        ptx::tma_prefetch_desc(&map_a);
    }
    if (warp == kUmDqWarps + 1) {
        ptx::tmem_alloc(ptx::smem_u32(&tmem_holder), kUmTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();          // every CTA's barriers exist before anyone signals across the cluster
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();

    if (warp == kUmDqWarps) {
        // ------------------------------------------------------------ producer: three TMA boxes per chunk
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t item = um_cluster_id(); ok && item < n_items; item += um_n_clusters(), ++iter) {
                uint32_t prob = 0, tile = item;
                if constexpr (kGrouped) { prob = item / p.n_tiles; tile = item - prob * p.n_tiles; }
                (void)prob; (void)tile;
                // the rings double as the parking area: the previous tile's copy must have been read by the whole cluster
                if (iter > 0 && !um_wait_cluster(read_bar, (iter - 1) & 1, abort_flag, p.wait_limit_ns)) {
                    atomicCAS(p.status, 0, kStatusProducerTimeout | 0x800000);
                    break;
                }
                const uint32_t n0 = tile * kUmBN;
                for (uint32_t c = c_begin; c < c_end; ++c) {
                    if (!ptx::mbar_wait_relaxed(raw_empty + 8 * stage, phase ^ 1, abort_flag, p.wait_limit_ns, 64)) {
                        atomicCAS(p.status, 0, kStatusProducerTimeout | (int)(c & 0xFFFFFF));
                        ok = false;
                        break;
                    }
                    ptx::fence_proxy_async_smem();           // the stage was read through the generic proxy, the copies write it through the async proxy
                    const uint32_t fb = raw_full + 8 * stage, dst = raw_ring + stage * kUmRawStride;
                    const uint32_t grp = c * kUmBK / p.group;
                    ptx::mbar_arrive_expect_tx(fb, kUmRawBytes);
                    const CUtensorMap* mw = &map_w;
                    const CUtensorMap* ms = &map_s;
                    const CUtensorMap* mz = &map_z;
                    if constexpr (kGrouped) { mw = &group.maps[4 * prob]; ms = &group.maps[4 * prob + 1]; mz = &group.maps[4 * prob + 2]; }
                    if (p.tiled) {
                        // tile-major layout: the chunk's 8 KB of words are contiguous, as are its scales and zero points
                        ptx::tma_load_3d(dst, mw, fb, 0, (int32_t)(c * (kUmBK / 8)), (int32_t)tile);
                        ptx::tma_load_3d(dst + 8 * kUmBN * 4, ms, fb, 0, (int32_t)grp, (int32_t)tile);
                        ptx::tma_load_3d(dst + 8 * kUmBN * 4 + kUmBN * 2, mz, fb, 0, (int32_t)grp, (int32_t)tile);
                    } else {
                        ptx::tma_load_2d(dst, mw, fb, (int32_t)n0, (int32_t)(c * (kUmBK / 8)));
                        ptx::tma_load_2d(dst + 8 * kUmBN * 4, ms, fb, (int32_t)n0, (int32_t)grp);
                        ptx::tma_load_2d(dst + 8 * kUmBN * 4 + kUmBN * 2, mz, fb, (int32_t)(n0 / 8), (int32_t)grp);
                    }
                    if (++stage == kUmRawStages) { stage = 0; phase ^= 1; }
                }
            }
        } else if (lane == 1) {
            // the activations of every chunk, one 128-row box each, as soon as the UMMAs that read the operand stage are done
            uint32_t as = 0, aphase = 0, iter = 0;
            bool ok = true;
            for (uint32_t item = um_cluster_id(); ok && item < n_items; item += um_n_clusters(), ++iter) {
                uint32_t prob = 0, tile = item;
                if constexpr (kGrouped) { prob = item / p.n_tiles; tile = item - prob * p.n_tiles; }
                (void)prob; (void)tile;
                if (iter > 0 && !um_wait_cluster(read_bar, (iter - 1) & 1, abort_flag, p.wait_limit_ns)) break;
                for (uint32_t c = c_begin; c < c_end; ++c) {
                    if (!ptx::mbar_wait_relaxed(ab_empty + 8 * as, aphase ^ 1, abort_flag, p.wait_limit_ns, 64)) {
                        atomicCAS(p.status, 0, kStatusProducerTimeout | 0x400000 | (int)(c & 0x3FFFFF));
                        ok = false;
                        break;
                    }
                    ptx::fence_proxy_async_smem();           // the rings were the parking area of the previous tile (generic proxy)
                    ptx::mbar_arrive_expect_tx(ab_full + 8 * as, kUmABytes);
                    const CUtensorMap* ma = &map_a;
                    if constexpr (kGrouped) ma = &group.maps[4 * prob + 3];
                    ptx::tma_load_3d(a_ring + as * kUmABytes, ma, ab_full + 8 * as, (int32_t)(c * kUmBK), 0, 0);
                    if (++as == kUmAbStages) { as = 0; aphase ^= 1; }
                }
            }
        }
    } else if (warp == kUmDqWarps + 1) {
        // ------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t kIdesc = ptx::make_idesc_bf16_f32(128, kUmBN, 0u);
            uint32_t stage = 0, phase = 0, iter = 0;
            bool ok = true;
            for (uint32_t item = um_cluster_id(); ok && item < n_items; item += um_n_clusters(), ++iter) {
                uint32_t prob = 0, tile = item;
                if constexpr (kGrouped) { prob = item / p.n_tiles; tile = item - prob * p.n_tiles; }
                (void)prob; (void)tile;
                if (iter > 0 && !ptx::mbar_wait(acc_empty, (iter - 1) & 1, abort_flag, p.wait_limit_ns)) {
                    atomicCAS(p.status, 0, kStatusMmaTimeout | 0x800000);
                    break;
                }
                ptx::tc_fence_after_sync();
                for (uint32_t c = 0; c < my_chunks; ++c) {
                    if (!ptx::mbar_wait(ab_full + 8 * stage, phase, abort_flag, p.wait_limit_ns)) {
                        atomicCAS(p.status, 0, kStatusMmaTimeout | (int)(c & 0x7FFFFF));
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = a_ring + stage * kUmABytes, b_addr = b_ring + stage * kUmBBytes;
#pragma unroll
                    for (uint32_t k4 = 0; k4 < kUmBK / 16; ++k4) {
                        const uint64_t da = ptx::make_smem_desc(a_addr + k4 * 32, 16, 1024);
                        const uint64_t db = ptx::make_smem_desc(b_addr + k4 * 32, 16, 1024);
                        ptx::umma_bf16_ss(tmem_base, da, db, kIdesc, (c | k4) != 0 ? 1u : 0u);
                    }
                    ptx::umma_commit(ab_empty + 8 * stage);
                    if (++stage == kUmAbStages) { stage = 0; phase ^= 1; }
                }
                if (ok) ptx::umma_commit(acc_full);
            }
        }
    } else {
        // ------------------------------------------------------------ sixteen warps: dequantise, then the epilogue
        // Two groups of eight warps take alternate chunks: a warp's chain per chunk (wait, loads, arithmetic, stores, proxy
        // fence, arrive) is longer than the UMMAs of a chunk, so with all sixteen warps on the same chunk that chain, not any
        // unit, set the pace; two chunks in flight hide it.  A thread owns one column of the tile and all eight word rows.
        const uint32_t grp = warp >> 3, n = (warp & 7) * 32 + lane;
        uint32_t mask, magic;
        asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(mask));
        asm volatile("mov.b32 %0, 0x43004300;" : "=r"(magic));
        uint32_t iter = 0, t_base = 0;                              // t_base: chunks of earlier tiles (ring positions run on across tiles)
        bool ok = true;
        const uint32_t b_off = (n >> 3) * 1024 + (n & 7) * 128;
        for (uint32_t item = um_cluster_id(); item < n_items; item += um_n_clusters(), ++iter, t_base += my_chunks) {
            uint32_t prob = 0, tile = item;
            if constexpr (kGrouped) { prob = item / p.n_tiles; tile = item - prob * p.n_tiles; }
            (void)prob;
            const uint32_t n0 = tile * kUmBN;
            if (ok && iter > 0 && !um_wait_cluster(read_bar, (iter - 1) & 1, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0x400000);
                ok = false;
            }
            for (uint32_t ci = 0; ok && ci < my_chunks; ++ci) {
                const uint32_t t = t_base + ci;
                if ((t & 1u) != grp) continue;
                const uint32_t rs = t % kUmRawStages, rphase = (t / kUmRawStages) & 1u, as = t % kUmAbStages, aphase = (t / kUmAbStages) & 1u;
                if (!ptx::mbar_wait(raw_full + 8 * rs, rphase, abort_flag, p.wait_limit_ns)) {
                    if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | (int)(ci & 0x3FFFFF));
                    ok = false;
                    break;
                }
                const uint32_t raw = raw_ring + rs * kUmRawStride;
                uint32_t words[8];
#pragma unroll
                for (uint32_t i = 0; i < 8; ++i) words[i] = um_lds32(raw + i * (kUmBN * 4) + n * 4);
                const uint32_t sbits = um_lds16(raw + 8 * kUmBN * 4 + n * 2);
                const uint32_t zword = um_lds32(raw + 8 * kUmBN * 4 + kUmBN * 2 + (n >> 3) * 4);
                const uint32_t zz = ((zword >> ((n & 7) * 4)) & 0xFu) * 0x00010001u + 0x43004300u;     // bf16x2 (128+z, 128+z)
                const uint32_t ss = sbits * 0x00010001u;                                               // (s, s)
                if (!ptx::mbar_wait(ab_empty + 8 * as, aphase ^ 1, abort_flag, p.wait_limit_ns)) {
                    if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0x800000 | (int)(ci & 0x3FFFFF));
                    ok = false;
                    break;
                }
                const uint32_t b_stage = b_ring + as * kUmBBytes + b_off;
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    const uint32_t wd = words[j];
                    const uint32_t v0 = bf16x2_mul(bf16x2_sub(and_or(wd, mask, magic), zz), ss);            // k 0, 4
                    const uint32_t v1 = bf16x2_mul(bf16x2_sub(and_or(wd >> 4, mask, magic), zz), ss);       // k 1, 5
                    const uint32_t v2 = bf16x2_mul(bf16x2_sub(and_or(wd >> 8, mask, magic), zz), ss);       // k 2, 6
                    const uint32_t v3 = bf16x2_mul(bf16x2_sub(and_or(wd >> 12, mask, magic), zz), ss);      // k 3, 7
                    if (p.tiled) {
                        // tile-major words hold their codes so that the four pairs come out as (0,1) (2,3) (4,5) (6,7)
                        um_sts128(b_stage + ((j ^ (n & 7)) << 4), v0, v1, v2, v3);
                    } else {
                        // row layout: pairs (0,4) (1,5) (2,6) (3,7); back into k order
                        um_sts128(b_stage + ((j ^ (n & 7)) << 4), __byte_perm(v0, v1, 0x5410), __byte_perm(v2, v3, 0x5410),
                                  __byte_perm(v0, v1, 0x7632), __byte_perm(v2, v3, 0x7632));
                    }
                }
                // The UMMAs read these bytes through the async proxy.  The warp's writes are ordered before lane 0 by the warp
                // barrier; lane 0's proxy fence and release-arrive then publish them (one fence per warp instead of 32:
                // the fence is the most expensive instruction of the chunk).
                __syncwarp();
                if (lane == 0) {
                    ptx::fence_proxy_async_smem();
                    ptx::mbar_arrive(raw_empty + 8 * rs);
                    ptx::mbar_arrive(ab_full + 8 * as);
                }
            }
            // ---- epilogue: the accumulator of this CTA's part of K
            if (ok && !ptx::mbar_wait(acc_full, iter & 1, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0xC00000);
                ok = false;
            }
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t q = warp & 3, cg = warp >> 2;             // tensor-memory lane quarter, 64-column group
            const uint32_t row_in = q * 32 + lane;
            if (p.split == 1) {
                // no exchange: straight from tensor memory to y
#pragma unroll 1
                for (uint32_t h = 0; h < 2; ++h) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(tmem_base + ((q * 32) << 16) + cg * 64 + h * 32, r);
                    ptx::tmem_ld_wait();
                    const uint32_t col = n0 + cg * 64 + h * 32;
                    if (row_in < p.M) {
                        float* y_out = p.y;
                        if constexpr (kGrouped) y_out = group.y[prob];
                        float* dst = y_out + (size_t)row_in * p.N + col;
                        if (col + 32 <= p.N && (p.N % 4 == 0) && (((uintptr_t)y_out & 15) == 0)) {       // every row starts on a 16-byte boundary
#pragma unroll
                            for (uint32_t j = 0; j < 8; ++j)
                                *(float4*)(dst + 4 * j) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                                                    __uint_as_float(r[4 * j + 3]));
                        } else {
#pragma unroll
                            for (uint32_t j = 0; j < 32; ++j)
                                if (col + j < p.N) dst[j] = __uint_as_float(r[j]);
                        }
                    }
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(acc_empty);
                    ptx::mbar_arrive(read_bar);          // (nothing was parked; the next tile's waits are the same either way)
                }
                continue;
            }
            // park (the rings are idle: every chunk has been consumed), tell the cluster, wait for everyone
#pragma unroll 1
            for (uint32_t h = 0; h < 2; ++h) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + ((q * 32) << 16) + cg * 64 + h * 32, r);
                ptx::tmem_ld_wait();
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j)
                    um_sts128(park + (row_in * kUmPitch + cg * 64 + h * 32 + 4 * j) * 4, r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(acc_empty);
                for (uint32_t s = 0; s < p.split; ++s) ptx::mbar_arrive_cluster(ptx::mapa(parked_bar, s));
            }
            if (!um_wait_cluster(parked_bar, iter & 1, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0xD00000);
                ok = false;
                break;
            }
            {
                // this CTA's column slice of the tile (whole float4s), every row; splits added in split order
                const uint32_t slice_w = ((kUmBN / p.split + 3) / 4) * 4;
                const uint32_t s_begin = split * slice_w, s_end = min(kUmBN, s_begin + slice_w);
                const uint32_t f4_per_row = s_end > s_begin ? (s_end - s_begin) / 4 : 0;
                const uint32_t items = 128 * f4_per_row;
                const bool vec = ((uintptr_t)p.y & 15) == 0;         // (N % 32 == 0 is a condition of this kernel)
                constexpr uint32_t kU = 2;
                for (uint32_t i0 = tid; i0 < items; i0 += kU * kUmDqWarps * 32) {
                    float4 part[kU][4];
#pragma unroll
                    for (uint32_t u = 0; u < kU; ++u) {
                        const uint32_t i = i0 + u * kUmDqWarps * 32;
                        const uint32_t row = i / f4_per_row, c4 = i - row * f4_per_row;
#pragma unroll
                        for (uint32_t s = 0; s < 4; ++s)
                            part[u][s] = (i < items && s < p.split) ? um_ld_cluster_f4(ptx::mapa(park + (row * kUmPitch + s_begin + c4 * 4) * 4, s))
                                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (uint32_t u = 0; u < kU; ++u) {
                        const uint32_t i = i0 + u * kUmDqWarps * 32;
                        if (i >= items) break;
                        const uint32_t row = i / f4_per_row, c4 = i - row * f4_per_row;
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (uint32_t s = 0; s < 4; ++s)
                            if (s < p.split) { acc.x += part[u][s].x; acc.y += part[u][s].y; acc.z += part[u][s].z; acc.w += part[u][s].w; }
                        const uint32_t col = n0 + s_begin + c4 * 4;
                        if (row >= p.M || col >= p.N) continue;
                        float* dst = p.y + (size_t)row * p.N + col;
                        if (vec && col + 4 <= p.N) *(float4*)dst = acc;
                        else {
                            const float o[4] = {acc.x, acc.y, acc.z, acc.w};
                            for (uint32_t j = 0; j < 4 && col + j < p.N; ++j) dst[j] = o[j];
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0)
                for (uint32_t s = 0; s < p.split; ++s) ptx::mbar_arrive_cluster(ptx::mapa(read_bar, s));      // this warp has read every copy
        }
    }

    // ---------------------------------------------------------------- common exit
    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();          // no CTA's shared memory goes away while a peer may still read its copy or signal its barriers
    if (warp == kUmDqWarps + 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kUmTmemCols);
    }
}

// ------------------------------------------------------------------ the same GEMM with the weights as the TENSOR-MEMORY operand
//
// For launches that do not split K (the grouped launches).  The shared-memory form above moves 114 KB through an SM's shared
// memory per 64-deep chunk (32 KB of dequantised weights written, then read again by the UMMAs, on top of the raw weights and
// the activations), which is what bounds it.  Here the roles of the operands are swapped: the dequantised weights are the
// 128-row A operand and go from registers straight into tensor memory (tcgen05.st; a warp writes the 32 lanes of its
// quadrant), the activations are the 128-column B operand in shared memory, exactly as TMA delivers them.  The accumulator is
// y transposed: lane = column of y, tensor-memory column = row of y; a tile of 256 columns is two 128-lane accumulators.
// Shared-memory traffic per chunk falls to 66 KB (raw weights in and out 18, activations in 16, read by eight UMMAs 32).
//
// Tensor memory (512 columns): accumulators 2 x 128 columns, then three A stages of 2 halves x 4 k-steps x 8 columns.
constexpr uint32_t kTsTmemCols = 512;
constexpr uint32_t kTsABase = 256;                         // first column of the A stages
constexpr uint32_t kTsAStageCols = 64;
constexpr uint32_t kTsAStages = 3;                         // (a fourth stage, which fills the 512 columns, measured no faster)
// (the request is padded past half an SM's shared memory: the kernel takes all 512 tensor-memory columns, so two of its CTAs
// must never share an SM)
constexpr uint32_t kTsXStages = 4;                         // activation stages (16 KB boxes from L2)
constexpr uint32_t kTsRawStages = 14;                      // raw weight stages: 124 KB in flight per SM; with six the kernel was bound by bytes in flight x latency
constexpr uint32_t kTsSmemUsed = kTsRawStages * kUmRawStride + kTsXStages * kUmABytes + 512 + 1024;
constexpr uint32_t kTsSmem = kTsSmemUsed > 120 * 1024 ? kTsSmemUsed : 120 * 1024;

#ifdef T0_UM_TRACE
#define UM_STAMP(row, t) do { if (p.trace && blockIdx.x == 0 && (t) < 64) p.trace[(row) * 64 + (t)] = ptx::globaltimer_ns(); } while (0)
#else
#define UM_STAMP(row, t) do { } while (0)
#endif

template <bool kGrouped>
__global__ void __launch_bounds__(kUmThreads, 1)
w4a16_umma_ts_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                     const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_a, const UmParams p,
                     const __grid_constant__ std::conditional_t<kGrouped, UmGroup, gemm::NoGroup> group) {
    uint32_t n_items = p.n_tiles;
    if constexpr (kGrouped) n_items = p.n_tiles * p.n_problems;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t raw_ring = smem;
    const uint32_t x_ring = smem + kTsRawStages * kUmRawStride;           // activations: [128 rows][64 k] bf16, 128-byte swizzle, per stage
    const uint32_t bars = x_ring + kTsXStages * kUmABytes;
    const uint32_t raw_full = bars, raw_empty = bars + 8 * kTsRawStages;
    const uint32_t ab_full = raw_empty + 8 * kTsRawStages, ab_empty = ab_full + 8 * kTsAStages;
    const uint32_t acc_full = ab_empty + 8 * kTsAStages, acc_empty = acc_full + 8;
    const uint32_t x_full = acc_empty + 8, x_empty = x_full + 8 * kTsXStages;
    __shared__ uint32_t tmem_holder;
    __shared__ int s_abort;
    volatile int* abort_flag = &s_abort;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n_chunks = p.n_chunks;

    if (tid == 0) {
        for (uint32_t s = 0; s < kTsRawStages; ++s) {
            ptx::mbar_init(raw_full + 8 * s, 1);
            ptx::mbar_init(raw_empty + 8 * s, kUmDqWarps);
        }
        for (uint32_t s = 0; s < kTsAStages; ++s) {
            ptx::mbar_init(ab_full + 8 * s, kUmDqWarps);          // sixteen warps' weights in tensor memory
            ptx::mbar_init(ab_empty + 8 * s, 1);
        }
        for (uint32_t s = 0; s < kTsXStages; ++s) {
            ptx::mbar_init(x_full + 8 * s, 1);
            ptx::mbar_init(x_empty + 8 * s, 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, kUmDqWarps);
        s_abort = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::tma_prefetch_desc(&map_w);
        ptx::tma_prefetch_desc(&map_s);
        ptx::tma_prefetch_desc(&map_z);
        ptx::tma_prefetch_desc(&map_a);
    }
    if (warp == kUmDqWarps + 1) {
        ptx::tmem_alloc(ptx::smem_u32(&tmem_holder), kTsTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_holder;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();

    if (warp == kUmDqWarps) {
        if (lane == 0) {
            // ---------------------------------------------------------- raw weights, scales, zero points: three TMA boxes per chunk
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
                uint32_t prob = 0, tile = item;
                if constexpr (kGrouped) { prob = item / p.n_tiles; tile = item - prob * p.n_tiles; }
                const CUtensorMap* mw = &map_w;
                const CUtensorMap* ms = &map_s;
                const CUtensorMap* mz = &map_z;
                if constexpr (kGrouped) { mw = &group.maps[4 * prob]; ms = &group.maps[4 * prob + 1]; mz = &group.maps[4 * prob + 2]; }
                const uint32_t n0 = tile * kUmBN;
                for (uint32_t c = 0; c < n_chunks; ++c) {
                    if (!ptx::mbar_wait_relaxed(raw_empty + 8 * stage, phase ^ 1, abort_flag, p.wait_limit_ns, 64)) {
                        atomicCAS(p.status, 0, kStatusProducerTimeout | (int)(c & 0xFFFFFF));
                        ok = false;
                        break;
                    }
                    UM_STAMP(0, c);
                    ptx::fence_proxy_async_smem();           // the stage was read through the generic proxy, the copies write it through the async proxy
                    const uint32_t fb = raw_full + 8 * stage, dst = raw_ring + stage * kUmRawStride;
                    const uint32_t grp = c * kUmBK / p.group;
                    ptx::mbar_arrive_expect_tx(fb, kUmRawBytes);
                    if (p.tiled) {
                        // tile-major layout: the chunk's 8 KB of words are contiguous, as are its scales and zero points
                        ptx::tma_load_3d(dst, mw, fb, 0, (int32_t)(c * (kUmBK / 8)), (int32_t)tile);
                        ptx::tma_load_3d(dst + 8 * kUmBN * 4, ms, fb, 0, (int32_t)grp, (int32_t)tile);
                        ptx::tma_load_3d(dst + 8 * kUmBN * 4 + kUmBN * 2, mz, fb, 0, (int32_t)grp, (int32_t)tile);
                    } else {
                        ptx::tma_load_2d(dst, mw, fb, (int32_t)n0, (int32_t)(c * (kUmBK / 8)));
                        ptx::tma_load_2d(dst + 8 * kUmBN * 4, ms, fb, (int32_t)n0, (int32_t)grp);
                        ptx::tma_load_2d(dst + 8 * kUmBN * 4 + kUmBN * 2, mz, fb, (int32_t)(n0 / 8), (int32_t)grp);
                    }
                    if (++stage == kTsRawStages) { stage = 0; phase ^= 1; }
                }
            }
        } else if (lane == 1) {
            // ---------------------------------------------------------- activations: one 128-row box per chunk (rows beyond M are zero)
            uint32_t as = 0, aphase = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
                uint32_t prob = 0;
                if constexpr (kGrouped) prob = item / p.n_tiles;
                const CUtensorMap* ma = &map_a;
                if constexpr (kGrouped) ma = &group.maps[4 * prob + 3];
                for (uint32_t c = 0; c < n_chunks; ++c) {
                    if (!ptx::mbar_wait_relaxed(x_empty + 8 * as, aphase ^ 1, abort_flag, p.wait_limit_ns, 64)) {
                        atomicCAS(p.status, 0, kStatusProducerTimeout | 0x400000 | (int)(c & 0x3FFFFF));
                        ok = false;
                        break;
                    }
                    ptx::mbar_arrive_expect_tx(x_full + 8 * as, kUmABytes);
                    ptx::tma_load_3d(x_ring + as * kUmABytes, ma, x_full + 8 * as, (int32_t)(c * kUmBK), 0, 0);
                    if (++as == kTsXStages) { as = 0; aphase ^= 1; }
                }
            }
        }
    } else if (warp == kUmDqWarps + 1) {
        // -------------------------------------------------------------- UMMA issuer: per chunk 2 halves x 4 k-steps of M 128 x N 128 x K 16
        if (lane == 0) {
            constexpr uint32_t kIdesc = ptx::make_idesc_bf16_f32(128, 128, 0u);
            uint32_t stage = 0, phase = 0, iter = 0, xs = 0, xphase = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++iter) {
                if (iter > 0 && !ptx::mbar_wait(acc_empty, (iter - 1) & 1, abort_flag, p.wait_limit_ns)) {
                    atomicCAS(p.status, 0, kStatusMmaTimeout | 0x800000);
                    break;
                }
                ptx::tc_fence_after_sync();
                for (uint32_t c = 0; c < n_chunks; ++c) {
                    if (!ptx::mbar_wait(ab_full + 8 * stage, phase, abort_flag, p.wait_limit_ns) ||
                        !ptx::mbar_wait(x_full + 8 * xs, xphase, abort_flag, p.wait_limit_ns)) {
                        atomicCAS(p.status, 0, kStatusMmaTimeout | (int)(c & 0x7FFFFF));
                        ok = false;
                        break;
                    }
                    UM_STAMP(4, c);
                    ptx::tc_fence_after_sync();
                    const uint32_t x_addr = x_ring + xs * kUmABytes;
                    const uint32_t a_cols = tmem_base + kTsABase + stage * kTsAStageCols;
#pragma unroll
                    for (uint32_t k4 = 0; k4 < kUmBK / 16; ++k4) {
                        const uint64_t db = ptx::make_smem_desc(x_addr + k4 * 32, 16, 1024);
#pragma unroll
                        for (uint32_t t = 0; t < 2; ++t)
                            ptx::umma_bf16_ts(tmem_base + t * 128, a_cols + t * 32 + k4 * 8, db, kIdesc, (c | k4) != 0 ? 1u : 0u);
                    }
                    ptx::umma_commit(ab_empty + 8 * stage);
                    ptx::umma_commit(x_empty + 8 * xs);
                    UM_STAMP(5, c);
                    if (++stage == kTsAStages) { stage = 0; phase ^= 1; }
                    if (++xs == kTsXStages) { xs = 0; xphase ^= 1; }
                }
                if (ok) ptx::umma_commit(acc_full);
            }
        }
    } else {
        // -------------------------------------------------------------- sixteen warps: dequantise into tensor memory, then the epilogue
        const uint32_t q = warp & 3, t = (warp >> 2) & 1, h = warp >> 3;   // lane quadrant, 128-column half of the tile, k half of a chunk
        const uint32_t n = t * 128 + q * 32 + lane;                          // this thread's column of the tile
        const uint32_t lane_base = (q * 32) << 16;
        uint32_t mask, magic;
        asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(mask));
        asm volatile("mov.b32 %0, 0x43004300;" : "=r"(magic));
        uint32_t rs = 0, rphase = 0, as = 0, aphase = 0, iter = 0;
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x, ++iter) {
            uint32_t prob = 0, tile = item;
            if constexpr (kGrouped) { prob = item / p.n_tiles; tile = item - prob * p.n_tiles; }
            const uint32_t n0 = tile * kUmBN;
            for (uint32_t c = 0; ok && c < n_chunks; ++c) {
                if (!ptx::mbar_wait(raw_full + 8 * rs, rphase, abort_flag, p.wait_limit_ns)) {
                    if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | (int)(c & 0x3FFFFF));
                    ok = false;
                    break;
                }
                if (tid == 0) UM_STAMP(1, c);
                const uint32_t raw = raw_ring + rs * kUmRawStride;
                uint32_t words[4];
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) words[i] = um_lds32(raw + (h * 4 + i) * (kUmBN * 4) + n * 4);
                const uint32_t sbits = um_lds16(raw + 8 * kUmBN * 4 + n * 2);
                const uint32_t zword = um_lds32(raw + 8 * kUmBN * 4 + kUmBN * 2 + (n >> 3) * 4);
                const uint32_t zz = ((zword >> ((n & 7) * 4)) & 0xFu) * 0x00010001u + 0x43004300u;     // bf16x2 (128+z, 128+z)
                const uint32_t ss = sbits * 0x00010001u;                                               // (s, s)
                // the A stage is free once the UMMAs of three chunks ago have read it
                if (!ptx::mbar_wait(ab_empty + 8 * as, aphase ^ 1, abort_flag, p.wait_limit_ns)) {
                    if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0x800000 | (int)(c & 0x3FFFFF));
                    ok = false;
                    break;
                }
                if (tid == 0) UM_STAMP(2, c);
                ptx::tc_fence_after_sync();
                const uint32_t a_cols = tmem_base + lane_base + kTsABase + as * kTsAStageCols + t * 32 + h * 16;
#pragma unroll
                for (uint32_t jj = 0; jj < 2; ++jj) {          // one k-step of 16 = two packed words = eight columns of bf16 pairs
                    uint32_t r8[8];
#pragma unroll
                    for (uint32_t half = 0; half < 2; ++half) {
                        const uint32_t wd = words[2 * jj + half];
                        const uint32_t v0 = bf16x2_mul(bf16x2_sub(and_or(wd, mask, magic), zz), ss);            // k 0, 4
                        const uint32_t v1 = bf16x2_mul(bf16x2_sub(and_or(wd >> 4, mask, magic), zz), ss);       // k 1, 5
                        const uint32_t v2 = bf16x2_mul(bf16x2_sub(and_or(wd >> 8, mask, magic), zz), ss);       // k 2, 6
                        const uint32_t v3 = bf16x2_mul(bf16x2_sub(and_or(wd >> 12, mask, magic), zz), ss);      // k 3, 7
                        // k order: (0,1) (2,3) (4,5) (6,7), two consecutive k per tensor-memory column
                        if (p.tiled) {                     // tile-major words are stored so that the pairs come out in that order
                            r8[half * 4 + 0] = v0; r8[half * 4 + 1] = v1; r8[half * 4 + 2] = v2; r8[half * 4 + 3] = v3;
                        } else {                           // row layout: pairs (0,4) (1,5) (2,6) (3,7)
                            r8[half * 4 + 0] = __byte_perm(v0, v1, 0x5410);
                            r8[half * 4 + 1] = __byte_perm(v2, v3, 0x5410);
                            r8[half * 4 + 2] = __byte_perm(v0, v1, 0x7632);
                            r8[half * 4 + 3] = __byte_perm(v2, v3, 0x7632);
                        }
                    }
                    ptx::tmem_st_32x32b_x8(a_cols + jj * 8, r8);
                }
                ptx::tmem_st_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(raw_empty + 8 * rs);
                    ptx::mbar_arrive(ab_full + 8 * as);
                }
                if (tid == 0) UM_STAMP(3, c);
                if (++rs == kTsRawStages) { rs = 0; rphase ^= 1; }
                if (++as == kTsAStages) { as = 0; aphase ^= 1; }
            }
            // ---- epilogue: y[m][n0 + n] = D[lane n][column m]; a warp stores 32 consecutive columns of one row per instruction
            if (ok && !ptx::mbar_wait(acc_full, iter & 1, abort_flag, p.wait_limit_ns)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0xC00000);
                ok = false;
            }
            if (!ok) break;
            ptx::tc_fence_after_sync();
            float* y_out = p.y;
            if constexpr (kGrouped) y_out = group.y[prob];
            const uint32_t col = n0 + n;
            // this warp: lanes of quadrant q, accumulator half t, rows (columns of the accumulator) h * 64 .. h * 64 + 63
#pragma unroll 1
            for (uint32_t mc = 0; mc < 2; ++mc) {
                const uint32_t m0 = h * 64 + mc * 32;
                if (m0 >= p.M) break;                 // warp-uniform
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(tmem_base + lane_base + t * 128 + m0, r);
                ptx::tmem_ld_wait();
                if (col < p.N) {
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j)
                        if (m0 + j < p.M) y_out[(size_t)(m0 + j) * p.N + col] = __uint_as_float(r[j]);
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(acc_empty);
        }
    }

    __syncwarp();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == kUmDqWarps + 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTsTmemCols);
    }
}

// ------------------------------------------------------------------ tile-major weight layout
//
// The row layout puts the 8 KB of packed words a CTA needs per chunk in eight 1 KB pieces 4N bytes apart; HBM serves that
// pattern at about a third of its copy bandwidth, which is then what bounds these kernels (not the arithmetic, not the
// UMMAs).  The tile-major layout stores every 256-column tile as a matrix of its own, so a chunk's words, scales and zero
// points are each one contiguous piece:
//   words  [T][K/8][256] u32, scales [T][K/G][256] bf16, zero points [T][K/G][32] u32, T = ceil(N / 256), columns past N zero;
//   within a word code k sits in nibble (k >> 1) + 4 (k & 1).
struct TiledLayout { size_t off_words, off_scales, off_zeros, total; uint32_t tiles, rows, groups; };

TiledLayout tiled_layout(uint32_t K, uint32_t N, uint32_t group) {
    TiledLayout L;
    L.tiles = ceil_div(N, kUmBN); L.rows = K / 8; L.groups = K / group;
    L.off_words = 0;
    L.off_scales = (size_t)L.tiles * L.rows * kUmBN * 4;
    L.off_zeros = L.off_scales + (size_t)L.tiles * L.groups * kUmBN * 2;
    L.total = L.off_zeros + (size_t)L.tiles * L.groups * (kUmBN / 8) * 4;
    return L;
}

// Row layout -> tile-major layout: one thread per output word / scale / zero-point word.
__global__ void w4_to_tiled_kernel(const uint32_t* __restrict__ packed, const uint16_t* __restrict__ scales, const uint32_t* __restrict__ zeros,
                                   uint8_t* __restrict__ out, uint32_t N, uint32_t nz, TiledLayout L) {
    const uint64_t n_words = (uint64_t)L.tiles * L.rows * kUmBN;
    const uint64_t n_scales = (uint64_t)L.tiles * L.groups * kUmBN;
    const uint64_t n_zwords = (uint64_t)L.tiles * L.groups * (kUmBN / 8);
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words + n_scales + n_zwords; i += stride) {
        if (i < n_words) {
            const uint32_t c = (uint32_t)(i % kUmBN);
            const uint64_t r = i / kUmBN;
            const uint32_t row = (uint32_t)(r % L.rows), tile = (uint32_t)(r / L.rows);
            const uint32_t n = tile * kUmBN + c;
            // code k of the word moves to nibble (k >> 1) + 4 (k & 1): the kernels pull nibbles i and i + 4 out together as one
            // bf16 pair, which is then (k, k + 1) with k = 2i, the order the UMMA operand wants, with no byte permutes
            uint32_t w = n < N ? packed[(size_t)row * N + n] : 0u, v = 0;
#pragma unroll
            for (uint32_t kk = 0; kk < 8; ++kk) v |= ((w >> (4 * kk)) & 0xFu) << (4 * ((kk >> 1) + 4 * (kk & 1)));
            ((uint32_t*)(out + L.off_words))[i] = v;
        } else if (i < n_words + n_scales) {
            const uint64_t j = i - n_words;
            const uint32_t c = (uint32_t)(j % kUmBN);
            const uint64_t r = j / kUmBN;
            const uint32_t g = (uint32_t)(r % L.groups), tile = (uint32_t)(r / L.groups);
            const uint32_t n = tile * kUmBN + c;
            ((uint16_t*)(out + L.off_scales))[j] = n < N ? scales[(size_t)g * N + n] : (uint16_t)0;
        } else {
            const uint64_t j = i - n_words - n_scales;
            const uint32_t wz = (uint32_t)(j % (kUmBN / 8));
            const uint64_t r = j / (kUmBN / 8);
            const uint32_t g = (uint32_t)(r % L.groups), tile = (uint32_t)(r / L.groups);
            const uint32_t n0 = tile * kUmBN + wz * 8;
            ((uint32_t*)(out + L.off_zeros))[j] = n0 < N ? zeros[(size_t)g * nz + (n0 >> 3)] : 0u;
        }
    }
}

}  // namespace

namespace t0 {

// Whether the fused tcgen05 kernel takes this W4A16 problem.
bool w4a16_umma_supported(uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group) {
    if (M == 0 || M > 128 || N % 32 || K == 0 || K % kUmBK || group == 0 || group % kUmBK || K % group) return false;
    if (((a | packed | scales | zeros) & 15) != 0 || (y & 3) != 0) return false;
    return true;
}

// The four tensor maps of one problem: packed words, scales, zero points, and the activations as the 128-row operand
// (K-major boxes of 64, 128-byte swizzle, rows beyond M read as zero).
static int um_maps(uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint32_t M, uint32_t N, uint32_t K, uint32_t group, CUtensorMap* out4) {
    int rc = gemm::make_map_2d_plain(&out4[0], (const void*)packed, 4, K / 8, N, kUmBN, kUmBK / 8);
    if (rc == T0_OK) rc = gemm::make_map_2d_plain(&out4[1], (const void*)scales, 2, K / group, N, kUmBN, 1);
    if (rc == T0_OK) rc = gemm::make_map_2d_plain(&out4[2], (const void*)zeros, 4, K / group, N / 8, kUmBN / 8, 1);
    if (rc == T0_OK) rc = gemm::make_map_kmajor(&out4[3], (const void*)a, M, K, K, 1, 128);
    return rc;
}

// The same four maps over the tile-major buffer: 3-D views (column in tile, row, tile).
static int um_maps_tiled(uint64_t a, uint64_t tiled, uint32_t M, uint32_t N, uint32_t K, uint32_t group, CUtensorMap* out4) {
    const TiledLayout L = tiled_layout(K, N, group);
    const uint8_t* base = (const uint8_t*)tiled;
    int rc = gemm::make_map_3d_plain(&out4[0], base + L.off_words, 4, kUmBN, L.rows, L.tiles, kUmBN * 4, (uint64_t)L.rows * kUmBN * 4, kUmBN, kUmBK / 8);
    if (rc == T0_OK) rc = gemm::make_map_3d_plain(&out4[1], base + L.off_scales, 2, kUmBN, L.groups, L.tiles, kUmBN * 2, (uint64_t)L.groups * kUmBN * 2, kUmBN, 1);
    if (rc == T0_OK) rc = gemm::make_map_3d_plain(&out4[2], base + L.off_zeros, 4, kUmBN / 8, L.groups, L.tiles, (kUmBN / 8) * 4, (uint64_t)L.groups * (kUmBN / 8) * 4, kUmBN / 8, 1);
    if (rc == T0_OK) rc = gemm::make_map_kmajor(&out4[3], (const void*)a, M, K, K, 1, 128);
    return rc;
}

static bool um_tiled_supported(uint64_t a, uint64_t tiled, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group) {
    if (M == 0 || M > 128 || N == 0 || K == 0 || K % kUmBK || group == 0 || group % kUmBK || K % group) return false;
    return ((a | tiled) & 15) == 0 && (y & 3) == 0;
}

template <bool kGrouped, bool kTs = false>
static int um_launch(t0_runtime* rt, const CUtensorMap* m4, UmParams p, uint32_t split, const std::conditional_t<kGrouped, UmGroup, gemm::NoGroup>& group) {
    auto kern = kTs ? w4a16_umma_ts_kernel<kGrouped> : w4a16_umma_kernel<kGrouped>;     // kTs: weights as the tensor-memory operand (K not split)
    constexpr uint32_t kSmemBytes = kTs ? kTsSmem : kUmSmem;
    static bool attr_set[64] = {};
    static int max_clusters[64][5] = {};
    if (rt->device >= 64) return fail(T0_ERR_INVALID, "device ordinal out of range");
    if (!attr_set[rt->device]) {
        T0_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_set[rt->device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kUmThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = rt->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (!max_clusters[rt->device][split]) {
        cfg.gridDim = dim3(split * ((uint32_t)rt->sm_count / split), 1, 1);
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess || n <= 0) { cudaGetLastError(); n = (int)((uint32_t)rt->sm_count / split) * 3 / 4; }
        max_clusters[rt->device][split] = std::max(n, 1);
    }
    p.split = split;
    static const bool use_pdl = getenv("T0_NO_PDL") == nullptr;
    const uint32_t items = p.n_tiles * (kGrouped ? p.n_problems : 1u);
    const uint32_t clusters = std::min<uint32_t>(items, (uint32_t)max_clusters[rt->device][split]);
    cfg.gridDim = dim3(clusters * split, 1, 1);
    cfg.numAttrs = use_pdl ? 2 : 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, kern, m4[0], m4[1], m4[2], m4[3], p, group);
    if (le != cudaSuccess) return fail(T0_ERR_CUDA, "W4A16 kernel launch failed: %s", cudaGetErrorString(le));
    rt->launches.fetch_add(1);
    return T0_OK;
}

static UmParams um_params(t0_runtime* rt, uint64_t a, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group) {
    UmParams p;
    memset(&p, 0, sizeof p);
    p.a = (const uint16_t*)a; p.y = (float*)y; p.status = rt->d_status;
    const uint64_t limit = rt->wait_limit_ns.load(std::memory_order_relaxed);
    p.wait_limit_ns = limit ? limit : ptx::kWaitLimitNs;
    p.M = M; p.N = N; p.K = K; p.group = group;
    p.n_tiles = ceil_div(N, kUmBN);
    p.n_chunks = K / kUmBK;
    return p;
}

int launch_w4a16_umma(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N, uint32_t K,
                      uint32_t group) {
    UmParams p = um_params(rt, a, y, M, N, K, group);
    // as many parts of K as fill the machine (the parts of a tile form a cluster of at most four CTAs)
    uint32_t split = std::max<uint32_t>(1, std::min<uint32_t>(4, (uint32_t)rt->sm_count / std::max<uint32_t>(1, p.n_tiles)));
    split = std::min(split, p.n_chunks);
    CUtensorMap m4[4];
    int rc = um_maps(a, packed, scales, zeros, M, N, K, group, m4);
    if (rc != T0_OK) return rc;
    const gemm::NoGroup none = {0};
    return um_launch<false>(rt, m4, p, split, none);
}

int launch_w4a16_umma_tiled(t0_runtime* rt, uint64_t a, uint64_t tiled, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group) {
    UmParams p = um_params(rt, a, y, M, N, K, group);
    p.tiled = 1;
    uint32_t split = std::max<uint32_t>(1, std::min<uint32_t>(4, (uint32_t)rt->sm_count / std::max<uint32_t>(1, p.n_tiles)));
    split = std::min(split, p.n_chunks);
    CUtensorMap m4[4];
    int rc = um_maps_tiled(a, tiled, M, N, K, group, m4);
    if (rc != T0_OK) return rc;
    const gemm::NoGroup none = {0};
    return split == 1 ? um_launch<false, true>(rt, m4, p, 1, none) : um_launch<false, false>(rt, m4, p, split, none);
}

int launch_w4a16_umma_tiled_grouped(t0_runtime* rt, const t0_w4a16_args* args, uint32_t count) {
    if (count == 0) return T0_OK;
    if (count > kUmMaxGroup) return fail(T0_ERR_INVALID, "at most %u problems per grouped launch (got %u)", kUmMaxGroup, count);
    const t0_w4a16_args& a0 = args[0];
    static UmGroup grp;
    static std::mutex grp_mu;
    std::lock_guard<std::mutex> lock(grp_mu);
    for (uint32_t i = 0; i < count; ++i) {
        const t0_w4a16_args& a = args[i];
        if (a.m != a0.m || a.n != a0.n || a.k != a0.k || a.group != a0.group) return fail(T0_ERR_INVALID, "grouped launch: problem %u differs from problem 0 in shape", i);
        if (!um_tiled_supported(a.a, a.packed, a.y, a.m, a.n, a.k, a.group)) return fail(T0_ERR_UNSUPPORTED, "grouped launch: problem %u is not a shape of the fused tcgen05 kernel", i);
        int rc = um_maps_tiled(a.a, a.packed, a.m, a.n, a.k, a.group, &grp.maps[4 * i]);
        if (rc != T0_OK) return rc;
        grp.y[i] = (float*)a.y;
    }
    UmParams p = um_params(rt, a0.a, a0.y, a0.m, a0.n, a0.k, a0.group);
    p.n_problems = count;
    p.tiled = 1;
#ifdef T0_UM_TRACE
    {
        static unsigned long long* d_trace = nullptr;
        static int calls = 0;
        if (!d_trace) { cudaMalloc(&d_trace, 6 * 64 * 8); cudaMemset(d_trace, 0, 6 * 64 * 8); }
        p.trace = d_trace;
        int rc2 = um_launch<true, true>(rt, grp.maps, p, 1, grp);
        if (++calls == 6) {
            cudaStreamSynchronize(rt->stream);
            unsigned long long h[6 * 64];
            cudaMemcpy(h, d_trace, sizeof h, cudaMemcpyDeviceToHost);
            const unsigned long long t0 = h[0];
            fprintf(stderr, "[um trace] chunk: producer-free raw-seen stage-free arrived | mma-ready committed   (us after the first)\n");
            for (int c = 0; c < 64; ++c)
                fprintf(stderr, "[um trace] %2d: %7.2f %7.2f %7.2f %7.2f | %7.2f %7.2f\n", c, (h[c] - t0) * 1e-3, (h[64 + c] - t0) * 1e-3, (h[128 + c] - t0) * 1e-3,
                        (h[192 + c] - t0) * 1e-3, (h[256 + c] - t0) * 1e-3, (h[320 + c] - t0) * 1e-3);
        }
        return rc2;
    }
#endif
    return um_launch<true, true>(rt, grp.maps, p, 1, grp);
}

// Up to 32 problems of one shape in one launch, K not split: the CTAs walk the column tiles of all the problems, so launch,
// prologue and the exchange between the parts of K disappear from the per-problem cost.  The problems run concurrently.
int launch_w4a16_umma_grouped(t0_runtime* rt, const t0_w4a16_args* args, uint32_t count) {
    if (count == 0) return T0_OK;
    if (count > kUmMaxGroup) return fail(T0_ERR_INVALID, "at most %u problems per grouped launch (got %u)", kUmMaxGroup, count);
    const t0_w4a16_args& a0 = args[0];
    static UmGroup grp;                  // 16.6 KB: kept off the stack, filled under the lock, copied by the launch
    static std::mutex grp_mu;
    std::lock_guard<std::mutex> lock(grp_mu);
    for (uint32_t i = 0; i < count; ++i) {
        const t0_w4a16_args& a = args[i];
        if (a.m != a0.m || a.n != a0.n || a.k != a0.k || a.group != a0.group) return fail(T0_ERR_INVALID, "grouped launch: problem %u differs from problem 0 in shape", i);
        if (!w4a16_umma_supported(a.a, a.packed, a.scales, a.zeros, a.y, a.m, a.n, a.k, a.group))
            return fail(T0_ERR_UNSUPPORTED, "grouped launch: problem %u is not a shape of the fused tcgen05 kernel", i);
        int rc = um_maps(a.a, a.packed, a.scales, a.zeros, a.m, a.n, a.k, a.group, &grp.maps[4 * i]);
        if (rc != T0_OK) return rc;
        grp.y[i] = (float*)a.y;
    }
    UmParams p = um_params(rt, a0.a, a0.y, a0.m, a0.n, a0.k, a0.group);
    p.n_problems = count;
    static const bool smem_form = getenv("T0_W4_UMMA_SS") != nullptr;     // comparison switch: dequantised weights through shared memory
    return smem_form ? um_launch<true, false>(rt, grp.maps, p, 1, grp) : um_launch<true, true>(rt, grp.maps, p, 1, grp);
}

}  // namespace t0

extern "C" {

size_t t0_w4_tiled_bytes(uint32_t K, uint32_t N, uint32_t group) {
    if (K == 0 || N == 0 || group == 0 || K % kUmBK || group % kUmBK || K % group) return 0;
    return tiled_layout(K, N, group).total;
}

int t0_w4_to_tiled(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out, uint32_t K, uint32_t N, uint32_t group) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!packed || !scales || !zeros || !out) return fail(T0_ERR_INVALID, "null device pointer");
    if (K == 0 || N == 0 || group == 0 || K % kUmBK || group % kUmBK || K % group)
        return fail(T0_ERR_UNSUPPORTED, "the tile-major layout needs K %% 64 == 0 and group %% 64 == 0 with group | K (K=%u, group=%u)", K, group);
    if (out & 127) return fail(T0_ERR_INVALID, "the output buffer must be 128-byte aligned");
    DeviceGuard guard(rt->device);
    const TiledLayout L = tiled_layout(K, N, group);
    const uint64_t n = L.total / 2;
    const uint32_t grid = (uint32_t)std::min<uint64_t>((n + 255) / 256, 148ull * 16);
    w4_to_tiled_kernel<<<grid, 256, 0, rt->stream>>>((const uint32_t*)packed, (const uint16_t*)scales, (const uint32_t*)zeros, (uint8_t*)out, N, (N + 7) / 8, L);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "layout conversion launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

int t0_w4a16_gemm_tiled(t0_runtime* rt, uint64_t a, uint64_t tiled, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (M == 0 || N == 0) return T0_OK;
    if (!a || !tiled || !y) return fail(T0_ERR_INVALID, "null device pointer");
    if (!um_tiled_supported(a, tiled, y, M, N, K, group))
        return fail(T0_ERR_UNSUPPORTED, "shape M=%u N=%u K=%u group=%u: needs M <= 128, K %% 64 == 0, group %% 64 == 0, group | K, a and the weights 16-byte aligned", M, N, K, group);
    DeviceGuard guard(rt->device);
    return launch_w4a16_umma_tiled(rt, a, tiled, y, M, N, K, group);
}

int t0_w4a16_gemm_tiled_grouped(t0_runtime* rt, const t0_w4a16_args* args, size_t count) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!args && count) return fail(T0_ERR_INVALID, "null arguments");
    for (size_t i = 0; i < count; ++i) {
        const t0_w4a16_args& a = args[i];
        if (a.m == 0 || a.n == 0) return fail(T0_ERR_INVALID, "grouped launch: problem %zu is empty", i);
        if (!a.a || !a.packed || !a.y) return fail(T0_ERR_INVALID, "null device pointer in problem %zu", i);
        if (!um_tiled_supported(a.a, a.packed, a.y, a.m, a.n, a.k, a.group))
            return fail(T0_ERR_UNSUPPORTED, "problem %zu: needs M <= 128, K %% 64 == 0, group %% 64 == 0, group | K, a and the weights 16-byte aligned", i);
        // the problems run at the same time: no output may be an activation or the output of another problem
        const uint64_t y_lo = a.y, y_hi = a.y + (uint64_t)a.m * a.n * 4;
        for (size_t j = 0; j < count; ++j) {
            if (j == i) continue;
            const t0_w4a16_args& b = args[j];
            const uint64_t by_hi = b.y + (uint64_t)b.m * b.n * 4, ba_hi = b.a + (uint64_t)b.m * b.k * 2;
            if ((y_lo < by_hi && b.y < y_hi) || (y_lo < ba_hi && b.a < y_hi))
                return fail(T0_ERR_INVALID, "grouped launch: the output of problem %zu overlaps the activations or the output of problem %zu (the problems run concurrently)", i, j);
        }
    }
    DeviceGuard guard(rt->device);
    // runs of equal shapes share a launch (up to 32 problems each)
    size_t i = 0;
    while (i < count) {
        size_t n = 1;
        while (i + n < count && n < kUmMaxGroup && args[i + n].m == args[i].m && args[i + n].n == args[i].n && args[i + n].k == args[i].k && args[i + n].group == args[i].group) ++n;
        rc = n == 1 ? launch_w4a16_umma_tiled(rt, args[i].a, args[i].packed, args[i].y, args[i].m, args[i].n, args[i].k, args[i].group)
                    : launch_w4a16_umma_tiled_grouped(rt, args + i, (uint32_t)n);
        if (rc != T0_OK) return rc;
        i += n;
    }
    return T0_OK;
}

}  // extern "C"


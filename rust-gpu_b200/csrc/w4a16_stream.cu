// K2, streaming form: the fused W4A16 GEMM for M <= 16 on weights in the streaming layout, one persistent launch for a
// whole list of problems.
//
// No counterpart kernel exists in the reference (its INT4 support stops at the stand-alone dequantisation kernels,
// src/t0/quant_kernels.rs:53-171); the batching idea is the reference's DispatchQueue (src/t0/prefill_dispatch.rs:61-206):
// a decode step submits one projection after another and waits once.
//
// y[m,n] = sum_k a[m,k] * w[k,n],  w = RNE_bf16((q - z) * s),  fp32 accumulate.  The int4 weights are ~97 % of the bytes,
// so the kernel is organised around streaming them exactly once at HBM rate:
//   * weights come in the layout of t0_w4_prepack: per (256-column band, 128-deep k step) one contiguous 16 KiB tile whose
//     words are already in mma.sync fragment order; a "unit" is one such tile.  The units of ALL problems of a launch form
//     one list, cut into equal contiguous ranges, one per CTA (one CTA per SM), so that launch, pipeline fill and the band
//     fix-up at the end of a range are paid once per launch instead of once per problem;
//   * warp 16 (one lane) streams the tiles of the range into a ring of stages with one 16 KiB bulk copy each;
//   * warps 17..20 prepare, one step each in turn and a few steps ahead of the consumers, what else a step needs in the
//     same stage: the activations of the step as mma.sync B fragments, and per column pair the words {128+z, s} the
//     dequantisation uses, so that a consumer gets them with one 16-byte load and no decoding;
//   * warps 0..15 (consumers) own 16 columns of the band each: two LDS.128 fetch a lane's eight packed words of a step;
//     nibble pairs become bf16x2 with one LOP3 (0x4300 | q is the bf16 128+q), minus (128+z), times s - bit-identical
//     to the oracle because (q-z)*s is rounded once - and every dequantised word IS the 16 x 16 A fragment of one
//     mma.sync.m16n8k16 whose 8-column B operand is the activations;
//   * a band that lies wholly inside a range is stored directly; a band shared by several CTAs is finished by whichever
//     CTA arrives last (per-band arrival counter, partial pieces in scratch, added in k order: deterministic, repeated
//     calls agree bit for bit); no CTA ever waits for another.  A spare lane of the producer warp counts a range's leading
//     partial band in while the consumers go on.
// Every barrier wait is bounded; a wait that runs out raises the CTA's abort flag, the roles unwind, the status word is
// written and the host reports T0_ERR_TIMEOUT.
#include "w4a16_common.cuh"

using namespace t0;
using namespace t0::w4;

namespace {

constexpr int kStConsumers = 16;                      // consumer warps: warp w owns columns 16w .. 16w+15 of the band, all k of a step
constexpr int kStHelpers = 4;                         // warps that prepare activations and scale / zero-point words
constexpr int kStProducerWarp = kStConsumers;
constexpr int kStHelperWarp0 = kStConsumers + 1;
constexpr int kStThreads = (kStHelperWarp0 + kStHelpers) * 32;    // 672 = 21 warps
constexpr int kStSzBytes = 2048;                      // per stage: [16 warps][8 g] uint4 {128+z(col), s(col), 128+z(col+8), s(col+8)} as bf16x2 pairs
constexpr int kStAFragBytes = 2048;                   // per stage and group of eight rows: [2 j][2 pr][32 lanes] uint4 B fragments
constexpr int kStMaxProblems = 32;                    // problems per launch (the table travels as a kernel parameter)

__host__ __device__ constexpr int st_stage_bytes(int m_groups) { return kWeightBytes + kStSzBytes + m_groups * kStAFragBytes; }
__host__ __device__ constexpr int st_stages(int m_groups) { return m_groups == 1 ? 11 : 10; }
__host__ __device__ constexpr size_t st_smem_bytes(int m_groups) { return 128 + (size_t)st_stages(m_groups) * st_stage_bytes(m_groups) + 512; }

struct StProblem {
    const uint16_t* a;         // [M][K] bf16
    float* y;                  // [M][N] f32
    const uint8_t* tiles;      // [band][kstep][16][256] u32
    const uint8_t* scales_t;   // [band][K/G][256] bf16
    const uint8_t* zeros_t;    // [band][K/G][32] u32
    uint32_t M, N, K;
    uint32_t ksteps, groups, units_per_group, n_bands;
    uint32_t unit_begin;       // first unit of this problem in the launch's list
    uint32_t band_begin;       // first arrival counter of this problem
    uint32_t _pad;
};

struct StParams {
    StProblem prob[kStMaxProblems];
    float* partials;           // [grid][2][16*256]
    int* counters;             // one per band of the launch, zero between launches
    int* status;               // error word of the runtime (bounded waits)
    unsigned long long* stamps;   // optional trace: 4 nanosecond stamps per CTA (entry, first step landed, loop done, exit)
    uint64_t wait_limit_ns;
    uint32_t n_problems, total_units;
    uint32_t probe;            // timing experiments, only in builds with -DT0_W4_PROBE (results are then wrong on purpose):
                               // 1 = consumers skip the arithmetic, 2 = the producer copies nothing, 3 = both
};

struct Cursor { uint32_t p, band, ks; };

__device__ __forceinline__ Cursor locate(const StParams& P, uint32_t unit) {
    Cursor c;
    c.p = 0;
    while (c.p + 1 < P.n_problems && P.prob[c.p + 1].unit_begin <= unit) ++c.p;
    const uint32_t r = unit - P.prob[c.p].unit_begin, ks = P.prob[c.p].ksteps;
    c.band = r / ks;
    c.ks = r - c.band * ks;
    return c;
}
__device__ __forceinline__ void advance(const StParams& P, Cursor& c) {
    if (++c.ks == P.prob[c.p].ksteps) {
        c.ks = 0;
        if (++c.band == P.prob[c.p].n_bands) { c.band = 0; ++c.p; }
    }
}

__device__ __forceinline__ void st_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kStConsumers * 32) : "memory"); }
// explicit shared-space accesses: the ring's address went through an integer for alignment, so plain pointers would make
// the compiler use generic loads and 64-bit address arithmetic
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int kMGroups>    // 1: every M <= 8, 2: M <= 16
__global__ void __launch_bounds__(kStThreads, 1)
w4a16_stream_kernel(const __grid_constant__ StParams P) {
    constexpr int kSt = st_stages(kMGroups);
    constexpr int kSB = st_stage_bytes(kMGroups);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t ring = (ptx::smem_u32(smem_raw) + 127u) & ~127u;      // kSt x {16 KiB tile, 2 KiB scale/zero words, kMGroups x 2 KiB B fragments}
    const uint32_t full_bar = ring + kSt * kSB;                          // [kSt] x 8 bytes
    const uint32_t empty_bar = full_bar + kSt * 8;
    const uint32_t head_written_bar = empty_bar + kSt * 8;               // all 16 consumer warps have stored their part of the head piece
    const uint32_t head_counted_bar = head_written_bar + 8;              // the head piece is counted in and s_head_last is valid
    __shared__ int s_flags[4];
    volatile int* abort_flag = &s_flags[0];
    int* s_last = &s_flags[1];
    int* s_head_last = &s_flags[2];                                      // 1 when this CTA turned out to be the last contributor of its head band

#ifdef T0_W4_PROBE
    const uint32_t probe = P.probe;
#else
    constexpr uint32_t probe = 0;
#endif
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t U0 = range_begin(blockIdx.x, gridDim.x, P.total_units);
    const uint32_t U1 = range_begin(blockIdx.x + 1, gridDim.x, P.total_units);
    if (U0 >= U1) return;
    auto stamp = [&](int i) {
        if (P.stamps) P.stamps[blockIdx.x * 4 + i] = ptx::globaltimer_ns();
    };
    if (tid == 0) {
        for (int s = 0; s < kSt; ++s) {
            ptx::mbar_init(full_bar + s * 8, 2);                 // the tile's bytes (producer) + the prepared words (a helper warp)
            ptx::mbar_init(empty_bar + s * 8, kStConsumers);
        }
        ptx::mbar_init(head_written_bar, kStConsumers);
        ptx::mbar_init(head_counted_bar, 1);
        *abort_flag = 0;
        *s_head_last = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    __syncthreads();
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();      // global memory is touched only after the previous grid in the stream is done
    if (tid == 0) stamp(0);
    const Cursor c0 = locate(P, U0);
    const uint32_t n_units = U1 - U0;
    // A head piece: the range starts inside a band and goes on into the next one.  Counting it in (fence, atomic round
    // trip) is the head warp's job, so no consumer warp falls behind the others while the range goes on.
    const uint32_t head_end = U0 - c0.ks + P.prob[c0.p].ksteps;    // one past the last unit of the first band
    const bool has_head = c0.ks != 0 && head_end < U1;

    if (warp == kStProducerWarp) {
        if (lane == 1 && has_head) {
            // ------------------------------------------------------------ lane 1 counts the head piece in (while lane 0 streams)
            int last = 0;
            if (ptx::mbar_wait_relaxed(head_written_bar, 0, abort_flag, P.wait_limit_ns, 1000)) {
                const uint32_t first_unit = head_end - P.prob[c0.p].ksteps;
                const uint32_t c_first = owner_of(first_unit, gridDim.x, P.total_units);
                const uint32_t c_last = owner_of(head_end - 1, gridDim.x, P.total_units);
                __threadfence();                   // the piece is visible before this CTA is counted
                last = atomicAdd(&P.counters[P.prob[c0.p].band_begin + c0.band], 1) == (int)(c_last - c_first);
                if (last) __threadfence();
            } else {
                atomicCAS(P.status, 0, kStatusEpilogueTimeout | 0xD00000);
            }
            *s_head_last = last;                   // looked at when the range is done
            ptx::mbar_arrive(head_counted_bar);
        }
        // ------------------------------------------------------------ lane 0, producer: one 16 KiB bulk copy per step
        if (lane == 0) {
            Cursor c = c0;
            uint32_t stage = 0, phase = 0;
            const uint8_t* src = P.prob[c.p].tiles + ((size_t)c.band * P.prob[c.p].ksteps + c.ks) * kWeightBytes;
            for (uint32_t u = U0; u < U1; ++u) {
                if (!ptx::mbar_wait_relaxed(empty_bar + stage * 8, phase ^ 1, abort_flag, P.wait_limit_ns, 100)) {
                    atomicCAS(P.status, 0, kStatusProducerTimeout | (int)(u & 0xFFFFFF));
                    break;
                }
                // The consumers read the stage through the generic proxy (their reads are ordered before this point by
                // their release-arrive and the acquire-wait above); the copy overwrites it through the async proxy, and
                // this fence orders the two.  Without a proxy fence, launches with cold TLBs consumed sectors of the
                // step loaded into the same stage a ring later.
                ptx::fence_proxy_async_smem();
                const uint32_t fb = full_bar + stage * 8;
                if (probe & 2) {
                    ptx::mbar_arrive(fb);
                } else {
                    ptx::mbar_arrive_expect_tx(fb, kWeightBytes);
                    ptx::bulk_load(ring + stage * kSB, src, kWeightBytes, fb);
                }
                if (++stage == kSt) { stage = 0; phase ^= 1; }
                // the tiles of one problem are consecutive in memory in the order the range walks them
                src += kWeightBytes;
                if (++c.ks == P.prob[c.p].ksteps) {
                    c.ks = 0;
                    if (++c.band == P.prob[c.p].n_bands) { c.band = 0; ++c.p; if (u + 1 < U1) src = P.prob[c.p].tiles; }
                }
            }
        }
        return;
    }
    if (warp >= kStHelperWarp0) {
        // ------------------------------------------------------------ helpers: step i of the range is prepared by helper i % 4
        const uint32_t h = warp - kStHelperWarp0;
        if (h >= n_units) return;
        Cursor c = c0;
        for (uint32_t k = 0; k < h; ++k) advance(P, c);
        const uint32_t g = lane >> 2, t = lane & 3;
        const uint32_t w2 = lane >> 1, hh = lane & 1;          // scale / zero-point words: this lane makes entries 8 w2 + 4 hh + 0..3
        uint32_t cur_p = 0xFFFFFFFFu, ksteps = 1, n_bands = 1, upg = 1, groups = 1, M = 0;
        const uint16_t* arow[kMGroups];                        // this lane's row of the activations per group of eight rows, at k = 2t
        const uint8_t* sbase = nullptr; const uint8_t* zbase = nullptr;
        for (uint32_t i = h;;) {
            if (c.p != cur_p) {
                const StProblem& pr = P.prob[c.p];
                cur_p = c.p; ksteps = pr.ksteps; n_bands = pr.n_bands; upg = pr.units_per_group; groups = pr.groups; M = pr.M;
#pragma unroll
                for (int mg = 0; mg < kMGroups; ++mg) arow[mg] = pr.a + (size_t)(mg * 8 + g) * pr.K + 2 * t;
                sbase = pr.scales_t + w2 * 32 + hh * 8;
                zbase = pr.zeros_t + w2 * 8;
            }
            const uint32_t stage = i % kSt, round = i / kSt;
            if (probe & 4) {      // timing experiment: no preparation, only the hand-off
                uint32_t okp = 1;
                if (lane == 0 && !ptx::mbar_wait_relaxed(empty_bar + stage * 8, (round & 1) ^ 1, abort_flag, P.wait_limit_ns, 400)) okp = 0;
                okp = __shfl_sync(0xFFFFFFFFu, okp, 0);
                if (!okp) break;
                if (lane == 0) ptx::mbar_arrive(full_bar + stage * 8);
                i += kStHelpers;
                if (i >= n_units) break;
                continue;
            }
            // loads first (they do not touch the stage), then the wait for the stage, then the stores
            // -- scale / zero-point words: entry e = 8w + g serves consumer warp w, lanes g: columns 16w + g and 16w + g + 8
            const size_t sz_row = (size_t)c.band * groups + c.ks / upg;
            const uint2 sa = __ldg((const uint2*)(sbase + sz_row * kScaleBytes));            // scales of columns 16 w2 + 4 hh + 0..3
            const uint2 sb = __ldg((const uint2*)(sbase + sz_row * kScaleBytes + 16));       // ... of columns 16 w2 + 8 + 4 hh + 0..3
            const uint2 zz = __ldg((const uint2*)(zbase + sz_row * kZeroBytes));             // zero points of columns 16 w2 + 0..7, 16 w2 + 8..15
            // -- activations of the step as B fragments: for row group mg, half j, pair pr2, lane (g, t) one uint4
            // {b0(s), b1(s), b0(s+1), b1(s+1)}, s = 4j + 2 pr2, b0(s) = a[m][k0 + 16s + 2t .. +1], b1(s) = a[m][k0 + 16s + 2t + 8 .. +9], m = 8 mg + g
            uint4 av[kMGroups * 4];
#pragma unroll
            for (int mg = 0; mg < kMGroups; ++mg) {
                const uint32_t* row = (const uint32_t*)(arow[mg] + c.ks * kUnitK);   // 4-byte aligned
                const bool in = (uint32_t)(mg * 8) + g < M;
#pragma unroll
                for (int f = 0; f < 4; ++f) {       // f = 2j + pr2: the step's k range in quarters of 32
                    av[mg * 4 + f] = make_uint4(0, 0, 0, 0);
                    if (in) {
                        av[mg * 4 + f].x = __ldg(row + f * 16); av[mg * 4 + f].y = __ldg(row + f * 16 + 4);
                        av[mg * 4 + f].z = __ldg(row + f * 16 + 8); av[mg * 4 + f].w = __ldg(row + f * 16 + 12);
                    }
                }
            }
            uint32_t okw = 1;
            if (lane == 0 && !ptx::mbar_wait_relaxed(empty_bar + stage * 8, (round & 1) ^ 1, abort_flag, P.wait_limit_ns, 400)) {
                atomicCAS(P.status, 0, kStatusProducerTimeout | 0x800000 | (int)((U0 + i) & 0x7FFFFF));
                okw = 0;
            }
            okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
            if (!okw) break;
            const uint32_t st = ring + stage * kSB + kWeightBytes;
            {
                const uint32_t sc0[4] = {sa.x & 0xFFFFu, sa.x >> 16, sa.y & 0xFFFFu, sa.y >> 16};
                const uint32_t sc1[4] = {sb.x & 0xFFFFu, sb.x >> 16, sb.y & 0xFFFFu, sb.y >> 16};
                const uint32_t z0 = zz.x >> (16 * hh), z1 = zz.y >> (16 * hh);      // the lane's four columns' zero points in the low 16 bits
#pragma unroll
                for (uint32_t q = 0; q < 4; ++q) {
                    uint4 o;
                    o.x = ((z0 >> (4 * q)) & 0xFu) * 0x00010001u + 0x43004300u;     // bf16x2 (128+z, 128+z)
                    o.y = sc0[q] * 0x00010001u;                                     // (s, s)
                    o.z = ((z1 >> (4 * q)) & 0xFu) * 0x00010001u + 0x43004300u;
                    o.w = sc1[q] * 0x00010001u;
                    sts128(st + (lane * 4 + q) * 16, o);
                }
            }
#pragma unroll
            for (uint32_t f = 0; f < kMGroups * 4; ++f)
                if ((f >> 2) * 8 + g < M) sts128(st + kStSzBytes + f * 512 + lane * 16, av[f]);      // (rows that do not exist are left as they are: their products are never stored)
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(full_bar + stage * 8);
            i += kStHelpers;
            if (i >= n_units) break;
            c.ks += kStHelpers;
            while (c.ks >= ksteps) {
                c.ks -= ksteps;
                if (++c.band == n_bands) {
                    c.band = 0; ++c.p;
                    ksteps = P.prob[c.p].ksteps; n_bands = P.prob[c.p].n_bands;     // (the other fields follow at the top of the loop)
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers (16 warps)
    const uint32_t g = lane >> 2, t = lane & 3;
    // four accumulator sets, one per k step modulo 4: consecutive MMAs must not wait for each other's result
    constexpr int kAccSets = 4;
    float acc[kMGroups][kAccSets][4];
#pragma unroll
    for (int mg = 0; mg < kMGroups; ++mg)
#pragma unroll
        for (int a = 0; a < kAccSets; ++a)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mg][a][j] = 0.0f;
    uint32_t mask, magic;
    asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(mask));
    asm volatile("mov.b32 %0, 0x43004300;" : "=r"(magic));
    Cursor c = c0;
    bool ok = true;    // false after a wait expired: the warps keep walking (barriers stay matched) but do no work
    const uint32_t col0 = warp * 16 + g;                      // this lane's two columns within the band: col0 and col0 + 8
    // a lane's places in the current stage: eight packed words [w][j][lane] uint4, the scale / zero words of its column pair,
    // its B fragments; the stage's barriers
    uint32_t st_w = ring + warp * 1024 + lane * 16;
    uint32_t st_sz = ring + kWeightBytes + (warp * 8 + g) * 16;
    uint32_t st_af = ring + kWeightBytes + kStSzBytes + lane * 16;
    uint32_t fb = full_bar, eb = empty_bar, stage = 0, phase = 0;
#ifdef T0_W4_PROBE
    bool first_step = true;
    long long wait_cycles = 0;
    const long long cyc0 = clock64();
#endif

    // The CTA that contributes last to a band adds the pieces in k order (CTA order) and stores; nobody waits for anybody.
    // Only the first contributor can hold the band in slot 1 (its range began in the band before).
    auto reduce_band = [&](uint32_t rp, uint32_t rb) {
        const StProblem& pr = P.prob[rp];
        const uint32_t first_unit = pr.unit_begin + rb * pr.ksteps;
        const uint32_t c_first = owner_of(first_unit, gridDim.x, P.total_units);
        const uint32_t c_last = owner_of(first_unit + pr.ksteps - 1, gridDim.x, P.total_units);
        const uint32_t first_slot = range_begin(c_first, gridDim.x, P.total_units) < first_unit ? 1u : 0u;
        constexpr int kPer = kMGroups * 8 * kBandCols / (kStConsumers * 32);   // outputs per thread: 4 for M <= 8, 8 for M <= 16
        constexpr int kCo = 4;                                                  // contributors whose pieces are in flight together
        float total[kPer];
#pragma unroll
        for (int j = 0; j < kPer; ++j) total[j] = 0.0f;
        for (uint32_t cc0 = c_first; cc0 <= c_last; cc0 += kCo) {
            float v[kCo][kPer];
#pragma unroll
            for (int b = 0; b < kCo; ++b) {
                const uint32_t cc = cc0 + b;
                const float* src = P.partials + ((size_t)cc * 2 + (cc == c_first ? first_slot : 0u)) * kPieceFloats;
#pragma unroll
                for (int j = 0; j < kPer; ++j) {
                    const uint32_t idx = tid + j * (kStConsumers * 32);
                    v[b][j] = (cc <= c_last && idx < pr.M * kBandCols) ? __ldcg(src + idx) : 0.0f;
                }
            }
#pragma unroll
            for (int b = 0; b < kCo; ++b)       // still added in CTA order, one contributor after the other
#pragma unroll
                for (int j = 0; j < kPer; ++j) total[j] += v[b][j];
        }
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const uint32_t idx = tid + j * (kStConsumers * 32);
            if (idx < pr.M * kBandCols) {
                const uint32_t row = idx / kBandCols, col = idx - row * kBandCols;
                const uint32_t nc = rb * kBandCols + col;
                if (nc < pr.N) pr.y[(size_t)row * pr.N + nc] = total[j];
            }
        }
        if (tid == 0) P.counters[pr.band_begin + rb] = 0;   // ready for the next launch
    };

    // The end of a piece (the steps of one band this CTA owns; `u_next` is the unit after it): a band that lies wholly in
    // the range is stored, a partial one goes to scratch and is counted in.
    auto flush_piece = [&](uint32_t u_next) {
        const StProblem& pr = P.prob[c.p];
        const uint32_t first_unit = pr.unit_begin + c.band * pr.ksteps, last_unit = first_unit + pr.ksteps;   // [first, last)
        const bool whole = first_unit >= U0 && last_unit <= U1;
        const uint32_t c_first = owner_of(first_unit, gridDim.x, P.total_units);
        const uint32_t c_last = owner_of(last_unit - 1, gridDim.x, P.total_units);
        const uint32_t slot = (first_unit <= U0) ? 0u : 1u;   // the piece of the band holding this CTA's first unit is slot 0
        float* piece = P.partials + ((size_t)blockIdx.x * 2 + slot) * kPieceFloats;
        // accumulator fragment: c0,c1 = (column col0, rows 2t, 2t+1), c2,c3 = (column col0 + 8, same rows)
#pragma unroll
        for (int mg = 0; mg < kMGroups; ++mg) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t m = mg * 8 + 2 * t + (j & 1), col = col0 + (j >> 1) * 8;
                const uint32_t ncol = c.band * kBandCols + col;
                const float v = (acc[mg][0][j] + acc[mg][1][j]) + (acc[mg][2][j] + acc[mg][3][j]);
                if (m < pr.M) {
                    if (!whole) piece[m * kBandCols + col] = v;
                    else if (ncol < pr.N) pr.y[(size_t)m * pr.N + ncol] = v;
                }
#pragma unroll
                for (int a = 0; a < kAccSets; ++a) acc[mg][a][j] = 0.0f;
            }
        }
        if (!whole) {
            if (u_next < U1) {
                // head piece, more steps follow: hand it to the counting lane and go on
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(head_written_bar);
            } else {
                st_consumer_sync();                    // every thread's part of the piece is written ...
                if (tid == 0) {
                    __threadfence();                   // ... and made visible before this CTA is counted
                    *s_last = atomicAdd(&P.counters[pr.band_begin + c.band], 1) == (int)(c_last - c_first);
                    if (*s_last) __threadfence();
                }
                st_consumer_sync();
                if (*s_last) reduce_band(c.p, c.band);
            }
        }
        c.ks = 0;          // a further piece starts a new band
        if (++c.band == pr.n_bands) { c.band = 0; ++c.p; }
    };

    // every warp walks the ring at its own pace: it waits for the stage, reads its words, and tells the producer when it is done
    uint32_t ksteps_cur = P.prob[c.p].ksteps;
    for (uint32_t u = U0; u < U1; ++u) {
#ifdef T0_W4_PROBE
        const long long tw0 = clock64();
#endif
        if (ok && !ptx::mbar_wait(fb, phase, abort_flag, P.wait_limit_ns)) {
            if (lane == 0) atomicCAS(P.status, 0, kStatusMmaTimeout | (int)(u & 0xFFFFFF));
            ok = false;
        }
#ifdef T0_W4_PROBE
        if (!first_step) wait_cycles += clock64() - tw0;      // (the first step's wait is the pipeline fill)
        if (first_step && tid == 0) stamp(1);
        first_step = false;
#endif
        if (ok && !(probe & 1)) {
            const uint4 q0 = lds128(st_w);
            const uint4 q1 = lds128(st_w + 512);
            const uint4 sz = lds128(st_sz);          // {128+z, s} of column col0, then of col0 + 8
            const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int p2 = 0; p2 < 2; ++p2) {
                    uint4 bf[kMGroups];
#pragma unroll
                    for (int mg = 0; mg < kMGroups; ++mg) {
                        bf[mg] = lds128(st_af + ((mg * 2 + j) * 2 + p2) * 512);     // (rows that do not exist: stale bytes, whose products are never stored)
                    }
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const uint32_t wd = words[j * 4 + p2 * 2 + e];
                        const uint32_t a0 = bf16x2_mul(bf16x2_sub(and_or(wd, mask, magic), sz.x), sz.y);
                        const uint32_t a1 = bf16x2_mul(bf16x2_sub(and_or(wd >> 4, mask, magic), sz.z), sz.w);
                        const uint32_t a2 = bf16x2_mul(bf16x2_sub(and_or(wd >> 8, mask, magic), sz.x), sz.y);
                        const uint32_t a3 = bf16x2_mul(bf16x2_sub(and_or(wd >> 12, mask, magic), sz.z), sz.w);
#pragma unroll
                        for (int mg = 0; mg < kMGroups; ++mg)
                            mma_bf16_16816(acc[mg][p2 * 2 + e], a0, a1, a2, a3, e ? bf[mg].z : bf[mg].x, e ? bf[mg].w : bf[mg].y);
                    }
                }
            }
        }
        if (ok) {
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(eb);          // this warp has read the stage
        }
        st_w += kSB; st_sz += kSB; st_af += kSB; fb += 8; eb += 8;
        if (++stage == kSt) {
            stage = 0; phase ^= 1;
            st_w -= kSt * kSB; st_sz -= kSt * kSB; st_af -= kSt * kSB; fb -= kSt * 8; eb -= kSt * 8;
        }
        if (++c.ks == ksteps_cur || u + 1 == U1) {
#ifdef T0_W4_PROBE
            if (u + 1 == U1 && tid == 0 && P.stamps) { P.stamps[gridDim.x * 4 + blockIdx.x] = (unsigned long long)(clock64() - cyc0); P.stamps[gridDim.x * 5 + blockIdx.x] = (unsigned long long)wait_cycles; }
#endif
            if (u + 1 == U1 && tid == 0) stamp(2);
            flush_piece(u + 1);
            if (u + 1 < U1) ksteps_cur = P.prob[c.p].ksteps;
        }
    }
    if (has_head) {
        if (!ptx::mbar_wait(head_counted_bar, 0, abort_flag, P.wait_limit_ns) && lane == 0) atomicCAS(P.status, 0, kStatusEpilogueTimeout | 0xE00000);
        st_consumer_sync();
        if (*s_head_last) reduce_band(c0.p, c0.band);
    }
    if (*abort_flag) {
        // give bulk copies already in flight time to land before shared memory goes away
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if (tid == 0) stamp(3);
}

// ------------------------------------------------------------------ streaming (tile-major) weight layout

struct PrepackLayout { size_t off_tiles, off_scales, off_zeros, total; uint32_t bands, ksteps, groups; };

PrepackLayout prepack_layout(uint32_t K, uint32_t N, uint32_t group) {
    PrepackLayout L;
    L.bands = ceil_div(N, kBandCols); L.ksteps = K / kUnitK; L.groups = K / group;
    L.off_tiles = 0;
    L.off_scales = (size_t)L.bands * L.ksteps * kWeightBytes;
    L.off_zeros = L.off_scales + (size_t)L.bands * L.groups * kScaleBytes;
    L.total = L.off_zeros + (size_t)L.bands * L.groups * kZeroBytes;
    return L;
}

// Row layout -> streaming layout.  One thread per four tile words (the four words that draw on the same four source words),
// per scale, or per word of eight zero points.  Columns past N are written as zero.
__global__ void w4_prepack_kernel(const uint32_t* __restrict__ packed, const uint16_t* __restrict__ scales, const uint32_t* __restrict__ zeros,
                                  uint8_t* __restrict__ out, uint32_t K, uint32_t N, uint32_t nz, PrepackLayout L) {
    const uint64_t n_words = (uint64_t)L.bands * L.ksteps * 16 * kBandCols / 4;      // units of four words
    const uint64_t n_scales = (uint64_t)L.bands * L.groups * kBandCols;
    const uint64_t n_zwords = (uint64_t)L.bands * L.groups * (kBandCols / 8);
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words + n_scales + n_zwords; i += stride) {
        if (i < n_words) {
            // Word (tile, w, j, lane, e) of the fragment order: k step s = 4j + e of column tile w, lane (g, t); nibble c / c+4 =
            // codes (k, k+1) of column n = 16w + g + 8(c & 1) at k = 16s + 2t + 8(c >> 1).  The four words t = 0..3 of one
            // (tile, w, j, g, e) take nibble pair t of the same four source words (two rows x two columns).
            const uint32_t e = (uint32_t)(i & 3), g = (uint32_t)((i >> 2) & 7), j = (uint32_t)((i >> 5) & 1), w = (uint32_t)((i >> 6) & 15);
            const uint64_t tile = i >> 10;
            const uint32_t ks = (uint32_t)(tile % L.ksteps), band = (uint32_t)(tile / L.ksteps);
            const uint32_t sstep = 4 * j + e;
            const uint32_t n0 = band * kBandCols + w * 16 + g, n1 = n0 + 8;
            const size_t r0 = (size_t)(ks * (kUnitK / 8) + 2 * sstep) * N;
            uint32_t src[4];
            src[0] = n0 < N ? __ldg(packed + r0 + n0) : 0u;
            src[1] = n1 < N ? __ldg(packed + r0 + n1) : 0u;
            src[2] = n0 < N ? __ldg(packed + r0 + N + n0) : 0u;
            src[3] = n1 < N ? __ldg(packed + r0 + N + n1) : 0u;
            uint32_t* dst = (uint32_t*)(out + L.off_tiles) + ((tile << 12) | ((uint64_t)w << 8) | ((uint64_t)j << 7) | ((uint64_t)g << 4) | e);
#pragma unroll
            for (uint32_t t = 0; t < 4; ++t) {
                uint32_t v = 0;
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) {
                    const uint32_t pair = src[c] >> (8 * t);
                    v |= (pair & 0xFu) << (4 * c);
                    v |= ((pair >> 4) & 0xFu) << (4 * (c + 4));
                }
                dst[t * 4] = v;                       // lane 4g + t: sixteen bytes further on
            }
        } else if (i < n_words + n_scales) {
            const uint64_t j = i - n_words;
            const uint32_t c = (uint32_t)(j % kBandCols);
            const uint64_t row = j / kBandCols;
            const uint32_t g = (uint32_t)(row % L.groups), band = (uint32_t)(row / L.groups);
            const uint32_t n = band * kBandCols + c;
            ((uint16_t*)(out + L.off_scales))[j] = n < N ? scales[(size_t)g * N + n] : (uint16_t)0;
        } else {
            const uint64_t j = i - n_words - n_scales;
            const uint32_t wz = (uint32_t)(j % (kBandCols / 8));
            const uint64_t row = j / (kBandCols / 8);
            const uint32_t g = (uint32_t)(row % L.groups), band = (uint32_t)(row / L.groups);
            const uint32_t n0 = band * kBandCols + wz * 8;     // eight columns, aligned to a source word
            ((uint32_t*)(out + L.off_zeros))[j] = n0 < N ? zeros[(size_t)g * nz + (n0 >> 3)] : 0u;
        }
    }
}

uint32_t prepack_grid_for(uint64_t n, uint32_t block) {
    uint64_t gsz = (n + block - 1) / block;
    const uint64_t cap = 148ull * 16;
    return (uint32_t)(gsz < 1 ? 1 : (gsz > cap ? cap : gsz));
}

// One launch for up to kStMaxProblems problems (already validated).
int launch_stream_chunk(t0_runtime* rt, const t0_w4a16_args* args, size_t count) {
    StParams P;
    memset(&P, 0, sizeof P);
    uint64_t total = 0, bands = 0;
    uint32_t max_m = 0;
    for (size_t i = 0; i < count; ++i) {
        const t0_w4a16_args& a = args[i];
        const PrepackLayout L = prepack_layout(a.k, a.n, a.group);
        StProblem& q = P.prob[i];
        q.a = (const uint16_t*)a.a;
        q.y = (float*)a.y;
        q.tiles = (const uint8_t*)a.packed + L.off_tiles;
        q.scales_t = (const uint8_t*)a.packed + L.off_scales;
        q.zeros_t = (const uint8_t*)a.packed + L.off_zeros;
        q.M = a.m; q.N = a.n; q.K = a.k;
        q.ksteps = L.ksteps; q.groups = L.groups; q.units_per_group = a.group / kUnitK; q.n_bands = L.bands;
        q.unit_begin = (uint32_t)total; q.band_begin = (uint32_t)bands;
        total += (uint64_t)L.bands * L.ksteps;
        bands += L.bands;
        max_m = std::max(max_m, a.m);
    }
    if (total == 0) return T0_OK;
    if (total > 0x7FFFFFFFull || bands * sizeof(int) > kCounterRegion) return fail(T0_ERR_UNSUPPORTED, "batch too large: %llu steps, %llu bands", (unsigned long long)total, (unsigned long long)bands);
    const uint32_t grid = (uint32_t)std::min<uint64_t>(total, (uint64_t)rt->sm_count);
    const size_t need = kCounterRegion + (size_t)grid * 2 * kPieceFloats * sizeof(float);
    if (need > rt->scratch_w4.size) {
        int rc = ensure_scratch(rt, rt->scratch_w4, need);
        if (rc != T0_OK) return rc;
        T0_CUDA(cudaMemsetAsync(rt->scratch_w4.ptr, 0, kCounterRegion, rt->stream));
    }
    P.counters = (int*)rt->scratch_w4.ptr;
    P.partials = (float*)((uint8_t*)rt->scratch_w4.ptr + kCounterRegion);
    P.status = rt->d_status;
    const uint64_t limit = rt->wait_limit_ns.load(std::memory_order_relaxed);
    P.wait_limit_ns = limit ? limit : ptx::kWaitLimitNs;
    P.n_problems = (uint32_t)count; P.total_units = (uint32_t)total;
#ifdef T0_W4_PROBE
    if (const char* pm = getenv("T0_W4_PROBE")) P.probe = (uint32_t)atoi(pm);
#endif
    const int m_groups = max_m <= 8 ? 1 : 2;
    static bool attr_set[64] = {};
    if (rt->device < 64 && !attr_set[rt->device]) {
        T0_CUDA(cudaFuncSetAttribute(w4a16_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st_smem_bytes(1)));
        T0_CUDA(cudaFuncSetAttribute(w4a16_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st_smem_bytes(2)));
        attr_set[rt->device] = true;
    }
    // T0_W4_TRACE=1: per-CTA stamps, summarised on stderr after a blocking wait (a debugging aid, off by default)
    static const bool trace = getenv("T0_W4_TRACE") != nullptr;
    StampBuffer stamps;
    if (trace) {
        int rc = stamps.make(grid);
        if (rc != T0_OK) return rc;
        P.stamps = stamps.d;
    }
    static const bool use_pdl = getenv("T0_NO_PDL") == nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kStThreads, 1, 1);
    cfg.dynamicSmemBytes = st_smem_bytes(m_groups);
    cfg.stream = rt->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    cudaError_t le = m_groups == 1 ? cudaLaunchKernelEx(&cfg, w4a16_stream_kernel<1>, P) : cudaLaunchKernelEx(&cfg, w4a16_stream_kernel<2>, P);
    if (le != cudaSuccess) return fail(T0_ERR_CUDA, "W4A16 kernel launch failed: %s", cudaGetErrorString(le));
    rt->launches.fetch_add(1);
    if (trace) {
        std::vector<unsigned long long> h((size_t)grid * 4);
        T0_CUDA(cudaStreamSynchronize(rt->stream));
        T0_CUDA(cudaMemcpy(h.data(), stamps.d, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        unsigned long long t_min = ~0ull, t_max = 0;
        double fill = 0, loop = 0, tail = 0;
        uint32_t slow = 0;
        for (uint32_t c = 0; c < grid; ++c) {
            t_min = std::min(t_min, h[c * 4]); t_max = std::max(t_max, h[c * 4 + 3]);
            fill += (double)(h[c * 4 + 1] - h[c * 4]); loop += (double)(h[c * 4 + 2] - h[c * 4 + 1]); tail += (double)(h[c * 4 + 3] - h[c * 4 + 2]);
            if (h[c * 4 + 3] - h[c * 4] > h[slow * 4 + 3] - h[slow * 4]) slow = c;
        }
#ifdef T0_W4_PROBE
        {
            std::vector<unsigned long long> cy(grid);
            T0_CUDA(cudaMemcpy(cy.data(), stamps.d + (size_t)grid * 4, cy.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
            std::vector<unsigned long long> wt(grid);
            T0_CUDA(cudaMemcpy(wt.data(), stamps.d + (size_t)grid * 5, wt.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
            double csum = 0, wsum = 0;
            for (uint32_t c = 0; c < grid; ++c) { csum += (double)cy[c]; wsum += (double)wt[c]; }
            fprintf(stderr, "[w4a16 stream trace] main loop %.0f SM cycles per step (mean over CTAs), of which warp 0 waits %.0f for the stage; %.3f GHz\n",
                    csum / grid / ((double)total / grid), wsum / grid / ((double)total / grid), csum / grid / (loop / grid));
        }
#endif
        fprintf(stderr, "[w4a16 stream trace] %zu problems, %llu steps on %u CTAs: first entry -> last exit %.2f us; per CTA mean: first step landed after %.2f us, "
                "main loop %.2f us (%.3f us per step), flush+exit %.2f us; slowest CTA %u entered %.2f us after the first, loop %.2f us, flush+exit %.2f us\n",
                count, (unsigned long long)total, grid, (t_max - t_min) * 1e-3, fill / grid * 1e-3, loop / grid * 1e-3, loop / grid * 1e-3 / ((double)total / grid),
                tail / grid * 1e-3, slow, (h[slow * 4] - t_min) * 1e-3, (h[slow * 4 + 2] - h[slow * 4 + 1]) * 1e-3, (h[slow * 4 + 3] - h[slow * 4 + 2]) * 1e-3);
    }
    return T0_OK;
}

int check_stream_problem(const t0_w4a16_args& a) {
    if (!a.a || !a.packed || !a.y) return fail(T0_ERR_INVALID, "null device pointer");
    if (a.m > 16) return fail(T0_ERR_UNSUPPORTED, "M=%u: the streaming-layout kernel takes M <= 16; use t0_w4a16_gemm on the row layout for larger M", a.m);
    if (a.k == 0 || a.k % kUnitK || a.group == 0 || a.group % kUnitK || a.k % a.group || a.n % 8)
        return fail(T0_ERR_UNSUPPORTED, "shape K=%u N=%u group=%u: needs K %% 128 == 0, group %% 128 == 0, group | K, N %% 8 == 0", a.k, a.n, a.group);
    if ((a.a & 15) || (a.packed & 127) || (a.y & 3)) return fail(T0_ERR_INVALID, "a must be 16-byte, the weights 128-byte and y 4-byte aligned");
    return T0_OK;
}

}  // namespace

extern "C" {

size_t t0_w4_prepacked_bytes(uint32_t K, uint32_t N, uint32_t group) {
    if (K == 0 || N == 0 || group == 0 || K % kUnitK || group % kUnitK || K % group) return 0;
    return prepack_layout(K, N, group).total;
}

int t0_w4_prepack(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out, uint32_t K, uint32_t N, uint32_t group) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!packed || !scales || !zeros || !out) return fail(T0_ERR_INVALID, "null device pointer");
    if (K == 0 || N == 0 || group == 0 || K % kUnitK || group % kUnitK || K % group)
        return fail(T0_ERR_UNSUPPORTED, "the streaming layout needs K %% 128 == 0 and group %% 128 == 0 with group | K (K=%u, group=%u)", K, group);
    if (N % 8) return fail(T0_ERR_UNSUPPORTED, "N=%u must be a multiple of 8 (eight zero points per word)", N);
    if (out & 127) return fail(T0_ERR_INVALID, "the output buffer must be 128-byte aligned");
    DeviceGuard guard(rt->device);
    const PrepackLayout L = prepack_layout(K, N, group);
    const uint64_t n = L.total / 2;
    w4_prepack_kernel<<<prepack_grid_for(n, 256), 256, 0, rt->stream>>>((const uint32_t*)packed, (const uint16_t*)scales, (const uint32_t*)zeros,
                                                                       (uint8_t*)out, K, N, (N + 7) / 8, L);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "prepack launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

int t0_w4a16_gemm_prepacked_batch(t0_runtime* rt, const t0_w4a16_args* args, size_t count) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!args && count) return fail(T0_ERR_INVALID, "null arguments");
    DeviceGuard guard(rt->device);
    // every problem is checked before anything is launched; empty problems are dropped
    std::vector<t0_w4a16_args> live;
    live.reserve(count);
    for (size_t i = 0; i < count; ++i) {
        if (args[i].m == 0 || args[i].n == 0) continue;
        rc = check_stream_problem(args[i]);
        if (rc != T0_OK) return rc;
        live.push_back(args[i]);
    }
    // launches of up to kStMaxProblems problems; a launch also ends where the band counters or the step index would overflow
    size_t i = 0;
    while (i < live.size()) {
        size_t n = 0;
        uint64_t bands = 0, units = 0;
        while (i + n < live.size() && n < (size_t)kStMaxProblems) {
            const PrepackLayout L = prepack_layout(live[i + n].k, live[i + n].n, live[i + n].group);
            if (n > 0 && ((bands + L.bands) * sizeof(int) > kCounterRegion || units + (uint64_t)L.bands * L.ksteps > 0x7FFFFFFFull)) break;
            bands += L.bands; units += (uint64_t)L.bands * L.ksteps;
            ++n;
        }
        rc = launch_stream_chunk(rt, live.data() + i, n);
        if (rc != T0_OK) return rc;
        i += n;
    }
    return T0_OK;
}

int t0_w4a16_gemm_prepacked(t0_runtime* rt, uint64_t a, uint64_t prepacked, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group) {
    t0_w4a16_args one;
    memset(&one, 0, sizeof one);
    one.a = a; one.packed = prepacked; one.y = y; one.m = M; one.n = N; one.k = K; one.group = group;
    return t0_w4a16_gemm_prepacked_batch(rt, &one, 1);
}

}  // extern "C"

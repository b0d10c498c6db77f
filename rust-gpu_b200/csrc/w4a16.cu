// INT4 weights: K3 (stand-alone dequantisation) and K2 (fused W4A16 GEMM, dequant in the main loop).
//
// Reference: src/t0/quant_kernels.rs — `build_dequant_int4_f32/bf16` (:53-171) compute
// out[e] = f32(code(e) - zp[e >> g]) * scale[e >> g] with two codes per byte, low nibble first (:5-9);
// `GptqWeight` (:188-294) is the container and wire format.  The reference has no fused INT4 GEMM; the
// fused kernel here computes  y[m,n] = sum_k a[m,k] * w[k,n],  w = RNE_bf16((q - z) * s),  fp32 accumulate,
// on the B200 weight layout: codes packed eight per u32 along K (packed[K/8][N]), bf16 scales [K/G][N],
// uint4 zero points packed eight per u32 along N (zeros[K/G][N/8]).
//
// K2 is HBM-bound for M <= 16 (the int4 weights are ~97% of the bytes), so it is organised around the
// weight stream:
//   * 148 persistent CTAs of 16 warps = 8 column slabs side by side x 2 k slices: one step of a CTA reads
//     eight packed rows of 1 KiB each (a DRAM page is used whole while it is open; 128-byte pieces 44 KiB
//     apart measured 11% of the copy bandwidth); the flattened space (256-column band) x (64-deep k step)
//     is cut into equal contiguous ranges, one per CTA (a band straddles several CTAs);
//   * per step every lane issues ONE 16-byte load (4 columns x 8 codes); loads for the next steps are
//     already in flight (register queue);
//   * codes become bf16 with one logic op (0x4300 | q is the bf16 128+q), minus (128+z), times s: two
//     bf16x2 ops per pair, bit-identical to the oracle's fp32 formula because (q-z)*s is exact in fp32;
//   * mma.sync m16n8k16 (bf16 in, fp32 out) does the dot products: the activations are the 16-row
//     operand, read from shared memory where they sit pre-permuted to match the code order in a word;
//   * the k slices of a slab are summed through shared memory in a fixed order; a band finished by one
//     CTA is stored directly, otherwise each CTA leaves its M x 256 piece in a scratch area and the CTA
//     that arrives last adds the pieces in k order (no CTA ever waits for another).
#include "w4a16_common.cuh"

using namespace t0;
using namespace t0::w4;

namespace {

// 32 k of one lane: 4 columns x 8 codes against the matching activation quads
__device__ __forceinline__ void consume_word4(float (&acc)[4][4], const uint4& wq, const uint32_t (&zz)[4], const uint32_t (&ss)[4],
                                              const uint4& qa0, const uint4& qa1, uint32_t mask, uint32_t magic) {
    const uint32_t words[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t wv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t v = and_or(words[c] >> (4 * i), mask, magic);   // bf16x2 (128+q_i, 128+q_{i+4})
            wv[i] = bf16x2_mul(bf16x2_sub(v, zz[c]), ss[c]);
        }
        mma_bf16_16816(acc[c], qa0.x, qa0.y, qa0.z, qa0.w, wv[0], wv[1]);
        mma_bf16_16816(acc[c], qa1.x, qa1.y, qa1.z, qa1.w, wv[2], wv[3]);
    }
}

constexpr int kConsumers = kWarps * 32;
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

__global__ void __launch_bounds__(kThreads, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                  const __grid_constant__ CUtensorMap map_z, const W4Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    uint8_t* ring = smem;                                             // kStages x {16 KiB codes, 512 B scales, 128 B zero points}
    float* red = (float*)(smem + kStages * kStageBytes);              // [kWarps][16][33]
    uint64_t* full_bar = (uint64_t*)(smem + kStages * kStageBytes + kRedBytes);
    uint64_t* empty_bar = full_bar + kStages;
    volatile int* abort_flag = (volatile int*)(empty_bar + kStages);
    int* s_last = (int*)(abort_flag + 1);
    // activations of this CTA's steps, in the order it walks them: one 288-byte record per group of eight k, eight
    // 16-byte quads {row g, row g+8} x {k0 k4 | k1 k5} then eight for {k2 k6 | k3 k7}: each quad is the A fragment of one MMA
    uint8_t* a_smem = smem + kStages * kStageBytes + kRedBytes + 256;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t u0 = range_begin(blockIdx.x, gridDim.x, p.total_units);
    const uint32_t u1 = range_begin(blockIdx.x + 1, gridDim.x, p.total_units);
    if (u0 >= u1) return;
    auto stamp = [&](int i) {
        if (p.stamps && tid == 0) { unsigned long long t_ns; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_ns)); p.stamps[blockIdx.x * 4 + i] = t_ns; }
    };
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), kWarps);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::tma_prefetch_desc(&map_w);
        ptx::tma_prefetch_desc(&map_s);
        ptx::tma_prefetch_desc(&map_z);
    }
    __syncthreads();
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();      // global memory is touched only after the previous grid in the stream is done
    stamp(0);
    const uint32_t band_first = u0 / p.ksteps;
    const uint32_t ks_first = u0 - band_first * p.ksteps;

    if (warp == kWarps) {
        // ------------------------------------------------------------ producer: one elected lane streams the steps in
        if (lane == 0) {
            uint32_t band = band_first, ks = ks_first, stage = 0, phase = 0;
            for (uint32_t u = u0; u < u1; ++u) {
                if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag)) {
                    atomicCAS(p.status, 0, kStatusProducerTimeout | (int)(u & 0xFFFFFF));
                    break;
                }
                const uint32_t fb = ptx::smem_u32(&full_bar[stage]);
                uint8_t* dst = ring + stage * kStageBytes;
                const uint32_t grp = ks / p.units_per_group;
                ptx::mbar_arrive_expect_tx(fb, kWeightBytes + kScaleBytes + kZeroBytes);
                ptx::tma_load_2d(ptx::smem_u32(dst), &map_w, fb, (int32_t)(band * kBandCols), (int32_t)(ks * (kUnitK / 8)));
                ptx::tma_load_2d(ptx::smem_u32(dst + kWeightBytes), &map_s, fb, (int32_t)(band * kBandCols), (int32_t)grp);
                ptx::tma_load_2d(ptx::smem_u32(dst + kWeightBytes + kScaleBytes), &map_z, fb, (int32_t)(band * (kBandCols / 8)), (int32_t)grp);
                if (++stage == kStages) { stage = 0; phase ^= 1; }
                if (++ks == p.ksteps) { ks = 0; ++band; }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers (16 warps)
    const uint32_t slab = warp & (kBandSlabs - 1), slice = warp / kBandSlabs;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t row_in_unit = slice * 8 + t;               // first packed row of this lane within a 128-deep step
    const uint32_t zshift = (g & 1) * 16;

    // Activations are staged for a_units steps at a time (all of this CTA's steps when they fit).  Within every group
    // of eight k the order becomes 0,4,1,5,2,6,3,7 so that the pair (code i, code i+4) a single mask pulls out of a
    // word lines up with the two bf16 of one register.  While the consumers restage, the ring keeps filling.
    auto stage_activations = [&](uint32_t ks_at, uint32_t count) {
        const uint32_t n_items = count * (kUnitK / 8) * 8;      // (record, row pair)
        for (uint32_t i0 = tid; i0 < n_items; i0 += 4 * kConsumers) {
            uint4 lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t i = i0 + j * kConsumers, rec = i >> 3, r = i & 7;
                const uint32_t unit = rec / (kUnitK / 8), kks = (ks_at + unit) % p.ksteps;
                const uint32_t kk = kks * kUnitK + (rec - unit * (kUnitK / 8)) * 8;
                lo[j] = make_uint4(0, 0, 0, 0); hi[j] = make_uint4(0, 0, 0, 0);
                if (i < n_items && r < p.M) lo[j] = __ldg((const uint4*)(p.a + (size_t)r * p.K + kk));
                if (i < n_items && r + 8 < p.M) hi[j] = __ldg((const uint4*)(p.a + (size_t)(r + 8) * p.K + kk));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t i = i0 + j * kConsumers, rec = i >> 3, r = i & 7;
                if (i >= n_items) break;
                uint4 q0, q1;
                q0.x = __byte_perm(lo[j].x, lo[j].z, 0x5410); q0.y = __byte_perm(hi[j].x, hi[j].z, 0x5410);   // k0 k4: rows r, r+8
                q0.z = __byte_perm(lo[j].x, lo[j].z, 0x7632); q0.w = __byte_perm(hi[j].x, hi[j].z, 0x7632);   // k1 k5
                q1.x = __byte_perm(lo[j].y, lo[j].w, 0x5410); q1.y = __byte_perm(hi[j].y, hi[j].w, 0x5410);   // k2 k6
                q1.z = __byte_perm(lo[j].y, lo[j].w, 0x7632); q1.w = __byte_perm(hi[j].y, hi[j].w, 0x7632);   // k3 k7
                *(uint4*)(a_smem + (size_t)rec * kARecord + r * 16) = q0;
                *(uint4*)(a_smem + (size_t)rec * kARecord + 128 + r * 16) = q1;
            }
        }
    };

    float acc[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[c][j] = 0.0f;
    // constants the compiler must keep in registers (see and_or)
    uint32_t mask, magic;
    asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(mask));
    asm volatile("mov.b32 %0, 0x43004300;" : "=r"(magic));

    uint32_t band = band_first, ks = ks_first, stage = 0, phase = 0;
    bool ok = true;    // false after a wait expired: the warp keeps walking (barriers stay matched) but does no work
    const uint8_t* const arec0 = a_smem + (size_t)row_in_unit * kARecord + g * 16;
    const uint8_t* arec = arec0;
    // this lane's places inside a stage
    const uint32_t w_off = row_in_unit * (kBandCols * 4) + slab * (kSlabCols * 4) + g * 16;
    const uint32_t s_off = kWeightBytes + (slab * kSlabCols + 4 * g) * 2;
    const uint32_t z_off = kWeightBytes + kScaleBytes + (slab * (kSlabCols / 8) + (g >> 1)) * 4;

    for (uint32_t u = u0; u < u1; ++u) {
        if ((u - u0) % p.a_units == 0) {
            if (u != u0) consumer_sync();          // everyone is done reading the previous batch
            stage_activations(ks, min(p.a_units, u1 - u));
            consumer_sync();
            if (u == u0) stamp(1);
            arec = arec0;
        }
        if (ok && !ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) {
            if (lane == 0) atomicCAS(p.status, 0, kStatusMmaTimeout | (int)(u & 0xFFFFFF));
            ok = false;
        }
        if (ok) {
            const uint8_t* st = ring + stage * kStageBytes;
            const uint4 w0 = *(const uint4*)(st + w_off);
            const uint4 w1 = *(const uint4*)(st + w_off + 4 * (kBandCols * 4));
            const uint2 sc = *(const uint2*)(st + s_off);
            const uint32_t zw = *(const uint32_t*)(st + z_off) >> zshift;
            uint32_t zz[4], ss[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t z = (zw >> (4 * c)) & 0xFu;
                zz[c] = z * 0x00010001u + 0x43004300u;                                   // bf16x2 (128+z, 128+z)
                ss[c] = __byte_perm((c & 2) ? sc.y : sc.x, 0, (c & 1) ? 0x3232 : 0x1010);   // (s, s)
            }
            consume_word4(acc, w0, zz, ss, *(const uint4*)arec, *(const uint4*)(arec + 128), mask, magic);
            consume_word4(acc, w1, zz, ss, *(const uint4*)(arec + 4 * kARecord), *(const uint4*)(arec + 4 * kARecord + 128), mask, magic);
            // The stage was read through the generic proxy and TMA (async proxy) will overwrite it: the reads are fenced
            // against the async proxy before the producer is told the stage is free.  Without the fence, launches that
            // ran with cold TLBs were seen consuming 32-byte sectors of the step loaded into the same stage eight steps later.
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&empty_bar[stage]));          // this warp is done with the stage
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
        arec += (kUnitK / 8) * kARecord;

        const bool band_ends = (ks + 1 == p.ksteps) || (u + 1 == u1);
        if (u + 1 == u1) stamp(2);
        if (band_ends) {
            // every warp parks its 16 x 32 partial; the k slices of a slab are then added in slice order
            float* mine = red + (size_t)warp * 16 * 33;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                mine[g * 33 + 4 * (2 * t) + c] = acc[c][0];
                mine[g * 33 + 4 * (2 * t + 1) + c] = acc[c][1];
                mine[(g + 8) * 33 + 4 * (2 * t) + c] = acc[c][2];
                mine[(g + 8) * 33 + 4 * (2 * t + 1) + c] = acc[c][3];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[c][j] = 0.0f;
            }
            consumer_sync();
            const uint32_t first_unit = band * p.ksteps, last_unit = first_unit + p.ksteps;   // [first, last)
            const bool whole = first_unit >= u0 && last_unit <= u1;
            const uint32_t c_first = owner_of(first_unit, gridDim.x, p.total_units);
            const uint32_t c_last = owner_of(last_unit - 1, gridDim.x, p.total_units);
            const uint32_t slot = (first_unit <= u0) ? 0u : 1u;   // the piece of the band holding this CTA's first unit is slot 0
            float* piece = p.partials + ((size_t)blockIdx.x * 2 + slot) * kPieceFloats;
            for (uint32_t idx = tid; idx < p.M * kBandCols; idx += kConsumers) {
                const uint32_t row = idx / kBandCols, col = idx - row * kBandCols;
                const uint32_t sl = col / kSlabCols, c32 = col - sl * kSlabCols;
                float sum = 0.0f;
#pragma unroll
                for (int s = 0; s < kSlices; ++s) sum += red[(size_t)(s * kBandSlabs + sl) * 16 * 33 + row * 33 + c32];
                const uint32_t ncol = band * kBandCols + col;
                if (whole) { if (ncol < p.N) p.y[(size_t)row * p.N + ncol] = sum; }
                else piece[idx] = sum;
            }
            if (!whole) {
                consumer_sync();                       // every thread's part of the piece is written ...
                if (tid == 0) {
                    __threadfence();                   // ... and made visible before this CTA is counted
                    *s_last = (atomicAdd(&p.counters[band], 1) == (int)(c_last - c_first)) ? 1 : 0;
                    if (*s_last) __threadfence();
                }
                consumer_sync();
                if (*s_last) {
                    // last to arrive: add the pieces in k order (CTA order) and store; nobody waits for anybody.
                    // Only the first contributor can hold this band in slot 1 (its range began in the band before).
                    const uint32_t first_slot = range_begin(c_first, gridDim.x, p.total_units) < first_unit ? 1u : 0u;
                    constexpr int kPer = kPieceFloats / kConsumers;   // 8 outputs per thread when M = 16
                    float total[kPer];
#pragma unroll
                    for (int j = 0; j < kPer; ++j) total[j] = 0.0f;
                    for (uint32_t c = c_first; c <= c_last; ++c) {
                        const float* src = p.partials + ((size_t)c * 2 + (c == c_first ? first_slot : 0u)) * kPieceFloats;
                        float v[kPer];
#pragma unroll
                        for (int j = 0; j < kPer; ++j) {
                            const uint32_t idx = tid + j * kConsumers;
                            v[j] = idx < p.M * kBandCols ? __ldcg(src + idx) : 0.0f;
                        }
#pragma unroll
                        for (int j = 0; j < kPer; ++j) total[j] += v[j];
                    }
#pragma unroll
                    for (int j = 0; j < kPer; ++j) {
                        const uint32_t idx = tid + j * kConsumers;
                        if (idx < p.M * kBandCols) {
                            const uint32_t row = idx / kBandCols, col = idx - row * kBandCols;
                            const uint32_t ncol = band * kBandCols + col;
                            if (ncol < p.N) p.y[(size_t)row * p.N + ncol] = total[j];
                        }
                    }
                    if (tid == 0) p.counters[band] = 0;   // ready for the next call
                }
            }
            consumer_sync();
        }
        if (++ks == p.ksteps) { ks = 0; ++band; }
    }
    stamp(3);
}

// ------------------------------------------------------------------ K2, tensor-memory form
//
// Same work split, ring and band fix-up as the kernel above, but the dot products run on tcgen05: the dequantised
// weights are the 128-row A operand and live in tensor memory (each of 16 dequant warps writes the rows of its lane
// quadrant with tcgen05.st), the activations are the 16-column B operand in shared memory (128-byte swizzle, K-major,
// pre-permuted to the order a single mask pulls codes out of a word), accumulators are 128 lanes x 16 columns per
// 128-column half band.  One UMMA (M 128, N 16, K 16) replaces 32 mma.sync; the k halves of a step accumulate into
// the same tensor-memory tile, so no cross-warp reduction is left.
constexpr int kTcWarps = 16;                         // dequant + epilogue warps
constexpr int kTcIssuers = 4;                        // UMMA issuer warps.  A 128 x 16 x 16 UMMA with its A tile in tensor memory costs about
                                                     // 100 cycles whatever its N and however many threads issue (measured); four issuers
                                                     // shorten the tail of a band a little, no more
constexpr int kTcThreads = (kTcWarps + 1 + kTcIssuers) * 32;   // + TMA producer warp + UMMA issuer warps
constexpr int kTcBUnitBytes = 2 * 16 * 128;          // activations of one step: two 64-deep atoms of 16 rows x 128 B
constexpr int kTcMaxUnits = 20;                      // steps of one CTA whose activations fit beside the ring
constexpr uint32_t kTcTmemCols = 512;
constexpr uint32_t kTcACols = 128;                   // A columns per step: 2 half bands x 8 k steps x 8 columns
constexpr uint32_t kTcABufs = 3;                     // A buffers: the dequant warps may run two steps ahead of the UMMAs
constexpr uint32_t kTcDBase = kTcABufs * kTcACols;   // then the accumulators: 2 half bands x 4 partial sums x 16 columns
constexpr uint32_t kTcDParts = 4;                    // k step j accumulates into partial sum j % 4, so every issuer owns its accumulators
constexpr uint32_t kTcIdesc = ptx::make_idesc_bf16_f32(128, 16, 0u);
__device__ __forceinline__ void tc_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kTcWarps * 32) : "memory"); }

// Weights in the row layout packed[K/8][N], fetched with 2-D TMA boxes; activations staged by the dequant warps in the
// permuted order.
__global__ void __launch_bounds__(kTcThreads, 1)
w4a16_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                const __grid_constant__ CUtensorMap map_z, const W4Params p) {
    constexpr uint32_t kRingStage = kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* b_area = smem;                                            // [a_units][2 atoms][16 rows][128 B], swizzled
    uint8_t* ring = smem + (size_t)p.a_units * kTcBUnitBytes;          // kStages x {16 KiB codes, 512 B scales, 128 B zero points}
    uint64_t* full_bar = (uint64_t*)(ring + kStages * kRingStage);
    uint64_t* empty_bar = full_bar + kStages;
    uint64_t* a_ready_bar = empty_bar + kStages;       // [kTcABufs] all 16 warps wrote their part of an A buffer
    uint64_t* a_free_bar = a_ready_bar + kTcABufs;     // [kTcABufs] the UMMAs that read an A buffer are done
    uint64_t* acc_full_bar = a_free_bar + kTcABufs;    // [2] a band piece is accumulated
    uint64_t* acc_empty_bar = acc_full_bar + 2;        // [2] all 16 warps have read an accumulator buffer
    uint32_t* tmem_holder = (uint32_t*)(acc_empty_bar + 2);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
    int* s_last = (int*)(tmem_holder + 2);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t u0 = range_begin(blockIdx.x, gridDim.x, p.total_units);
    const uint32_t u1 = range_begin(blockIdx.x + 1, gridDim.x, p.total_units);
    if (u0 >= u1) return;
    auto stamp = [&](int i) {
        if (p.stamps && tid == 0) { unsigned long long t_ns; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_ns)); p.stamps[blockIdx.x * 4 + i] = t_ns; }
    };
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), kTcWarps);
        }
        for (uint32_t b = 0; b < kTcABufs; ++b) {
            ptx::mbar_init(ptx::smem_u32(&a_ready_bar[b]), kTcWarps);
            ptx::mbar_init(ptx::smem_u32(&a_free_bar[b]), kTcIssuers);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&acc_full_bar[b]), kTcIssuers);
            ptx::mbar_init(ptx::smem_u32(&acc_empty_bar[b]), kTcWarps);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::tma_prefetch_desc(&map_w);
        ptx::tma_prefetch_desc(&map_s);
        ptx::tma_prefetch_desc(&map_z);
    }
    if (warp == kTcWarps + 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_holder), kTcTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();      // global memory is touched only after the previous grid in the stream is done
    stamp(0);
    const uint32_t band_first = u0 / p.ksteps;
    const uint32_t ks_first = u0 - band_first * p.ksteps;

    if (warp == kTcWarps) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t band = band_first, ks = ks_first, stage = 0, phase = 0;
            for (uint32_t u = u0; u < u1; ++u) {
                if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag)) {
                    atomicCAS(p.status, 0, kStatusProducerTimeout | (int)(u & 0xFFFFFF));
                    break;
                }
                const uint32_t fb = ptx::smem_u32(&full_bar[stage]);
                uint8_t* dst = ring + stage * kRingStage;
                const uint32_t grp = ks / p.units_per_group;
                ptx::mbar_arrive_expect_tx(fb, kWeightBytes + kScaleBytes + kZeroBytes);
                ptx::tma_load_2d(ptx::smem_u32(dst), &map_w, fb, (int32_t)(band * kBandCols), (int32_t)(ks * (kUnitK / 8)));
                ptx::tma_load_2d(ptx::smem_u32(dst + kWeightBytes), &map_s, fb, (int32_t)(band * kBandCols), (int32_t)grp);
                ptx::tma_load_2d(ptx::smem_u32(dst + kWeightBytes + kScaleBytes), &map_z, fb, (int32_t)(band * (kBandCols / 8)), (int32_t)grp);
            
                if (++stage == kStages) { stage = 0; phase ^= 1; }
                if (++ks == p.ksteps) { ks = 0; ++band; }
            }
        }
    } else if (warp > kTcWarps) {
        // ------------------------------------------------------------ UMMA issuers: issuer w owns k steps w and w + 4 of
        // every step and partial accumulator w of both half bands
        const uint32_t issuer = warp - kTcWarps - 1;
        if (lane == 0) {
            uint32_t ks = ks_first, piece = 0;
            bool piece_start = true;
            for (uint32_t u = u0; u < u1; ++u) {
                const uint32_t i = u - u0, ab = i % kTcABufs, a_round = i / kTcABufs;
                if (piece_start) {
                    // the accumulators have been read by everyone (previous piece)
                    if (!ptx::mbar_wait(ptx::smem_u32(&acc_empty_bar[0]), (piece & 1) ^ 1, abort_flag)) {
                        atomicCAS(p.status, 0, kStatusMmaTimeout | 0x800000 | (int)(u & 0x7FFFFF));
                        break;
                    }
                }
                const long long t_w = p.stamps ? clock64() : 0;
                if (!ptx::mbar_wait(ptx::smem_u32(&a_ready_bar[ab]), a_round & 1, abort_flag)) {
                    atomicCAS(p.status, 0, kStatusMmaTimeout | (int)(u & 0xFFFFFF));
                    break;
                }
                if (p.stamps && issuer == 0) p.stamps[gridDim.x * 4 + blockIdx.x * 4 + 3] += (unsigned long long)(clock64() - t_w);   // trace: idle time of issuer 0
                ptx::tc_fence_after_sync();
                const uint32_t b_addr = ptx::smem_u32(b_area + (size_t)i * kTcBUnitBytes);
#pragma unroll
                for (uint32_t jh = 0; jh < 2; ++jh) {
                    const uint32_t j = issuer + jh * kTcDParts;
                    const uint64_t db = ptx::make_smem_desc(b_addr + jh * 2048 + issuer * 32, 16, 1024);
#pragma unroll
                    for (uint32_t t = 0; t < 2; ++t)
                        ptx::umma_bf16_ts(tmem_base + kTcDBase + (t * kTcDParts + issuer) * 16, tmem_base + ab * kTcACols + t * 64 + j * 8, db, kTcIdesc,
                                          (piece_start && jh == 0) ? 0u : 1u);
                }
                ptx::umma_commit(ptx::smem_u32(&a_free_bar[ab]));
                const bool band_ends = (ks + 1 == p.ksteps) || (u + 1 == u1);
                piece_start = false;
                if (band_ends) {
                    ptx::umma_commit(ptx::smem_u32(&acc_full_bar[0]));
                    ++piece;
                    piece_start = true;
                }
                if (++ks == p.ksteps) ks = 0;
            }
        }
    } else {
        // ------------------------------------------------------------ dequant + epilogue warps (16)
        const uint32_t q = warp & 3, t = (warp >> 2) & 1, h = warp >> 3;   // lane quadrant, half band, k half of a step
        const uint32_t n_local = t * 128 + q * 32 + lane;                   // this thread's column within the band
        const uint32_t lane_base = (q * 32) << 16;
        const uint32_t n_units = u1 - u0;

        // Activations -> shared memory as the B operand: 16 rows (m) x 64 k per 128-byte-swizzled atom.  Within every
        // group of eight k the order becomes 0,4,1,5,2,6,3,7: the pair (code i, code i+4) one mask pulls out of a
        // packed word is then one 32-bit column of the A tile.
        for (uint32_t i = tid; i < n_units * 256; i += kTcWarps * 32) {
            const uint32_t unit = i >> 8, m = (i >> 4) & 15, g8 = i & 15;
            const uint32_t kks = (ks_first + unit) % p.ksteps;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < p.M) v = __ldg((const uint4*)(p.a + (size_t)m * p.K + kks * kUnitK + g8 * 8));
            uint4 o;
            o.x = __byte_perm(v.x, v.z, 0x5410);   // k0 k4
            o.y = __byte_perm(v.x, v.z, 0x7632);   // k1 k5
            o.z = __byte_perm(v.y, v.w, 0x5410);   // k2 k6
            o.w = __byte_perm(v.y, v.w, 0x7632);   // k3 k7
            *(uint4*)(b_area + (size_t)unit * kTcBUnitBytes + (g8 >> 3) * 2048 + m * 128 + (((g8 & 7) ^ (m & 7)) << 4)) = o;
        }
        ptx::fence_proxy_async_smem();            // the UMMAs read these bytes through the async proxy
        tc_consumer_sync();
        stamp(1);

        uint32_t mask, magic;
        asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(mask));
        asm volatile("mov.b32 %0, 0x43004300;" : "=r"(magic));
        uint32_t band = band_first, ks = ks_first, stage = 0, phase = 0, piece_idx = 0;
        long long w_full = 0, w_afree = 0, w_acc = 0, t_mark = 0;   // trace only: cycles this warp waited on each barrier
        const bool tracing = p.stamps != nullptr;
        bool ok = true;    // false after a wait expired: the warp keeps walking (barriers stay matched) but does no work
        const uint32_t w_off = (h * 8) * (kBandCols * 4) + n_local * 4;
        const uint32_t s_off = kWeightBytes + n_local * 2;
        const uint32_t z_off = kWeightBytes + kScaleBytes + (n_local >> 3) * 4;
        const uint32_t z_shift = (n_local & 7) * 4;

        for (uint32_t u = u0; u < u1; ++u) {
            const uint32_t i = u - u0, ab = i % kTcABufs, a_round = i / kTcABufs;
            if (tracing) t_mark = clock64();
            if (ok && !ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | (int)(u & 0xFFFFFF));
                ok = false;
            }
            if (tracing) { const long long now = clock64(); w_full += now - t_mark; t_mark = now; }
            uint32_t words[8];
            uint32_t zz = 0, ss = 0;
            if (ok) {
                const uint8_t* st = ring + stage * kRingStage;
#pragma unroll
                for (int r = 0; r < 8; ++r) words[r] = *(const uint32_t*)(st + w_off + r * (kBandCols * 4));
                uint32_t s, z;
                s = *(const uint16_t*)(st + s_off);
                z = (*(const uint32_t*)(st + z_off) >> z_shift) & 0xFu;
            
                zz = z * 0x00010001u + 0x43004300u;     // bf16x2 (128+z, 128+z)
                ss = s * 0x00010001u;                    // (s, s)
            }
            // the A buffer is free once the UMMAs of two steps ago have read it
            if (tracing) t_mark = clock64();
            if (ok && !ptx::mbar_wait(ptx::smem_u32(&a_free_bar[ab]), (a_round & 1) ^ 1, abort_flag)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0x400000 | (int)(u & 0x3FFFFF));
                ok = false;
            }
            if (tracing) w_afree += clock64() - t_mark;
            if (ok) {
                ptx::tc_fence_after_sync();
#pragma unroll
                for (uint32_t jj = 0; jj < 4; ++jj) {
                    uint32_t r8[8];
#pragma unroll
                    for (uint32_t half = 0; half < 2; ++half) {
                        const uint32_t wd = words[2 * jj + half];
#pragma unroll
                        for (uint32_t c = 0; c < 4; ++c) {
                            const uint32_t v = and_or(wd >> (4 * c), mask, magic);          // bf16x2 (128 + nibble c, 128 + nibble c+4)
                            r8[half * 4 + c] = bf16x2_mul(bf16x2_sub(v, zz), ss);
                        }
                    }
                    ptx::tmem_st_32x32b_x8(tmem_base + lane_base + ab * kTcACols + t * 64 + (h * 4 + jj) * 8, r8);
                }
                // the stage was read through the generic proxy and TMA (async proxy) will overwrite it
                ptx::fence_proxy_async_smem();
                ptx::tmem_st_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(ptx::smem_u32(&empty_bar[stage]));
                    ptx::mbar_arrive(ptx::smem_u32(&a_ready_bar[ab]));
                }
            }
            if (++stage == kStages) { stage = 0; phase ^= 1; }

            const bool band_ends = (ks + 1 == p.ksteps) || (u + 1 == u1);
            if (u + 1 == u1) stamp(2);
            if (band_ends) {
                if (tracing) t_mark = clock64();
                if (ok && !ptx::mbar_wait(ptx::smem_u32(&acc_full_bar[0]), piece_idx & 1, abort_flag)) {
                    if (lane == 0) atomicCAS(p.status, 0, kStatusEpilogueTimeout | 0x800000 | (int)(u & 0x3FFFFF));
                    ok = false;
                }
                if (tracing) w_acc += clock64() - t_mark;
                uint32_t d[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) d[j] = 0;
                if (ok) {
                    ptx::tc_fence_after_sync();
                    // rows m = 8h .. 8h+7 of column n_local: the four partial sums, added in k order
                    uint32_t part[kTcDParts][8];
#pragma unroll
                    for (uint32_t jq = 0; jq < kTcDParts; ++jq)
                        ptx::tmem_ld_32x32b_x8(tmem_base + lane_base + kTcDBase + (t * kTcDParts + jq) * 16 + h * 8, part[jq]);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        d[j] = __float_as_uint((__uint_as_float(part[0][j]) + __uint_as_float(part[1][j])) +
                                               (__uint_as_float(part[2][j]) + __uint_as_float(part[3][j])));
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&acc_empty_bar[0]));
                }
                ++piece_idx;
                const uint32_t first_unit = band * p.ksteps, last_unit = first_unit + p.ksteps;   // [first, last)
                const bool whole = first_unit >= u0 && last_unit <= u1;
                const uint32_t c_first = owner_of(first_unit, gridDim.x, p.total_units);
                const uint32_t c_last = owner_of(last_unit - 1, gridDim.x, p.total_units);
                const uint32_t slot = (first_unit <= u0) ? 0u : 1u;   // the piece of the band holding this CTA's first unit is slot 0
                float* piece = p.partials + ((size_t)blockIdx.x * 2 + slot) * kPieceFloats;
                const uint32_t ncol = band * kBandCols + n_local;
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    const uint32_t m = h * 8 + j;
                    if (m < p.M) {
                        if (!whole) piece[m * kBandCols + n_local] = __uint_as_float(d[j]);
                        else if (ncol < p.N) p.y[(size_t)m * p.N + ncol] = __uint_as_float(d[j]);
                    }
                }
                if (!whole) {
                    tc_consumer_sync();                    // every thread's part of the piece is written ...
                    if (tid == 0) {
                        __threadfence();                   // ... and made visible before this CTA is counted
                        *s_last = (atomicAdd(&p.counters[band], 1) == (int)(c_last - c_first)) ? 1 : 0;
                        if (*s_last) __threadfence();
                    }
                    tc_consumer_sync();
                    if (*s_last) {
                        // last to arrive: add the pieces in k order (CTA order) and store; nobody waits for anybody.
                        // Only the first contributor can hold this band in slot 1 (its range began in the band before).
                        const uint32_t first_slot = range_begin(c_first, gridDim.x, p.total_units) < first_unit ? 1u : 0u;
                        constexpr int kPer = kPieceFloats / (kTcWarps * 32);   // 8 outputs per thread when M = 16
                        constexpr int kCo = 2;                                  // contributors whose pieces are in flight together
                        float total[kPer];
#pragma unroll
                        for (int j = 0; j < kPer; ++j) total[j] = 0.0f;
                        for (uint32_t c = c_first; c <= c_last; c += kCo) {
                            float v[kCo][kPer];
#pragma unroll
                            for (int b = 0; b < kCo; ++b) {
                                const uint32_t cc = c + b;
                                const float* src = p.partials + ((size_t)cc * 2 + (cc == c_first ? first_slot : 0u)) * kPieceFloats;
#pragma unroll
                                for (int j = 0; j < kPer; ++j) {
                                    const uint32_t idx = tid + j * (kTcWarps * 32);
                                    v[b][j] = (cc <= c_last && idx < p.M * kBandCols) ? __ldcg(src + idx) : 0.0f;
                                }
                            }
#pragma unroll
                            for (int b = 0; b < kCo; ++b)       // still added in CTA order, one contributor after the other
#pragma unroll
                                for (int j = 0; j < kPer; ++j) total[j] += v[b][j];
                        }
#pragma unroll
                        for (int j = 0; j < kPer; ++j) {
                            const uint32_t idx = tid + j * (kTcWarps * 32);
                            if (idx < p.M * kBandCols) {
                                const uint32_t row = idx / kBandCols, col = idx - row * kBandCols;
                                const uint32_t nc = band * kBandCols + col;
                                if (nc < p.N) p.y[(size_t)row * p.N + nc] = total[j];
                            }
                        }
                        if (tid == 0) p.counters[band] = 0;   // ready for the next call
                    }
                    tc_consumer_sync();
                }
            }
            if (++ks == p.ksteps) { ks = 0; ++band; }
        }
        if (tracing && tid == 0) { p.stamps[gridDim.x * 4 + blockIdx.x * 4 + 0] = w_full; p.stamps[gridDim.x * 4 + blockIdx.x * 4 + 1] = w_afree; p.stamps[gridDim.x * 4 + blockIdx.x * 4 + 2] = w_acc; }
    }

    // ---------------------------------------------------------------- common exit
    __syncwarp();
    stamp(3);
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == kTcWarps + 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTcTmemCols);
    }
}

// ------------------------------------------------------------------ K3: stand-alone dequantisation

// Eight elements of the reference wire format from one packed word: value = (code - zero point) * scale in f32
// (quant_kernels.rs:53-171); bf16 output keeps the upper 16 bits (truncation, quant_kernels.rs:167-168).
__device__ __forceinline__ void dequant_ref_word(uint32_t word, int32_t zp, float sc, void* out, uint64_t e0, uint32_t out_bf16) {
    uint32_t bits[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) bits[i] = __float_as_uint(__fmul_rn((float)((int32_t)((word >> (4 * i)) & 0xFu) - zp), sc));
    if (out_bf16) {
        uint4 o;
        o.x = __byte_perm(bits[0], bits[1], 0x7632); o.y = __byte_perm(bits[2], bits[3], 0x7632);
        o.z = __byte_perm(bits[4], bits[5], 0x7632); o.w = __byte_perm(bits[6], bits[7], 0x7632);
        __stcs((uint4*)((uint16_t*)out + e0), o);
    } else {
        __stcs((uint4*)((float*)out + e0), make_uint4(bits[0], bits[1], bits[2], bits[3]));
        __stcs((uint4*)((float*)out + e0) + 1, make_uint4(bits[4], bits[5], bits[6], bits[7]));
    }
}

// The f32 form for a full warp: a thread's eight values are 32 bytes, so two plain 16-byte stores per thread would each
// touch half of every 32-byte sector.  Neighbouring lanes swap one half instead (the even lane gives its upper four values
// and takes the odd lane's lower four), after which each store instruction writes whole sectors.
__device__ __forceinline__ void dequant_ref_word_f32_paired(uint32_t word, int32_t zp, float sc, float* out, uint64_t e0, uint32_t lane) {
    uint32_t bits[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) bits[i] = __float_as_uint(__fmul_rn((float)((int32_t)((word >> (4 * i)) & 0xFu) - zp), sc));
    const bool odd = lane & 1;
    uint32_t got[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) got[i] = __shfl_xor_sync(0xFFFFFFFFu, odd ? bits[i] : bits[4 + i], 1);
    // even lane: own values 0..3 at e0, the neighbour's 0..3 at e0 + 8; odd lane: the neighbour's 4..7 at e0 - 4, own 4..7 at e0 + 4
    float* base = out + e0;
    uint4 v1, v2;
    v1.x = odd ? got[0] : bits[0]; v1.y = odd ? got[1] : bits[1]; v1.z = odd ? got[2] : bits[2]; v1.w = odd ? got[3] : bits[3];
    v2.x = odd ? bits[4] : got[0]; v2.y = odd ? bits[5] : got[1]; v2.z = odd ? bits[6] : got[2]; v2.w = odd ? bits[7] : got[3];
    __stcs((uint4*)(odd ? base - 4 : base), v1);
    __stcs((uint4*)(odd ? base + 4 : base + 8), v2);
}

// Reference wire format (quant_kernels.rs:53-171): byte e/2 holds element e in its low nibble for even e, one f32 scale and
// one i32 zero point per group of 2^group_log2 elements.  One thread per packed 32-bit word (eight elements): a warp reads
// 128 contiguous bytes and writes 1 KiB (f32) or 512 bytes (bf16) contiguous, 16 bytes per store.
__global__ void dequant_int4_ref_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                        const int32_t* __restrict__ zps, void* __restrict__ out, uint64_t total,
                                        uint32_t group_log2, uint32_t out_bf16) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t units = (total + 7) / 8;
    // a group of at least eight elements never splits a word; the 16-byte stores need the output aligned
    const bool vec = group_log2 >= 3 && (((uintptr_t)packed & 3) == 0) && (((uintptr_t)out & 15) == 0);
    uint64_t u = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        // four independent words per round: all twelve loads are issued before the first is used
        const uint64_t full = total / 8;
        const uint32_t lane = threadIdx.x & 31;
        // (the condition is the same for all lanes of a warp: the f32 stores exchange halves between neighbouring lanes)
        for (; u - lane + 31 + 3 * stride < full; u += 4 * stride) {
            uint32_t word[4];
            int32_t zp[4];
            float sc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint64_t e0 = (u + j * stride) * 8, grp = e0 >> group_log2;
                word[j] = __ldcs((const uint32_t*)(packed + (e0 >> 1)));
                zp[j] = __ldg(zps + grp);
                sc[j] = __ldg(scales + grp);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (out_bf16) dequant_ref_word(word[j], zp[j], sc[j], out, (u + j * stride) * 8, 1u);
                else dequant_ref_word_f32_paired(word[j], zp[j], sc[j], (float*)out, (u + j * stride) * 8, lane);
            }
        }
    }
    for (; u < units; u += stride) {
        const uint64_t e0 = u * 8;
        if (vec && e0 + 8 <= total) {
            const uint64_t grp = e0 >> group_log2;
            dequant_ref_word(__ldcs((const uint32_t*)(packed + (e0 >> 1))), __ldg(zps + grp), __ldg(scales + grp), out, e0, out_bf16);
            continue;
        }
        for (uint64_t e = e0; e < e0 + 8 && e < total; ++e) {
            const uint8_t b = packed[e >> 1];
            const uint32_t code = (e & 1) ? (b >> 4) : (b & 0xFu);
            const uint64_t grp = e >> group_log2;
            const float v = __fmul_rn((float)((int32_t)code - __ldg(zps + grp)), __ldg(scales + grp));
            if (out_bf16) ((uint16_t*)out)[e] = (uint16_t)(__float_as_uint(v) >> 16);
            else ((float*)out)[e] = v;
        }
    }
}

// B200 layout -> bf16 [K][N]: one thread per (k group of 8, 8 columns): reads eight packed words (32 bytes), writes eight
// rows of 16 bytes, so a warp stores 512 contiguous bytes per row.  Ragged N (not a multiple of 8) takes the scalar tail.
__global__ void dequant_w4_b200_kernel(const uint32_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                                       const uint32_t* __restrict__ zeros, uint16_t* __restrict__ out, uint32_t K, uint32_t N,
                                       uint32_t group, uint32_t nz) {
    const uint32_t n8 = (N + 7) / 8;
    const uint64_t total = (uint64_t)(K / 8) * n8;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool vec = (N % 8 == 0) && (((uintptr_t)packed & 15) == 0) && (((uintptr_t)scales & 15) == 0) && (((uintptr_t)out & 15) == 0);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t kg = (uint32_t)(i / n8), col = (uint32_t)(i % n8) * 8;
        const uint32_t grp = (kg * 8) / group;
        const uint32_t zword = zeros[(size_t)grp * nz + (col >> 3)];        // the zero points of these eight columns
        uint32_t words[8];
        uint16_t sbits[8];
        if (vec) {
            // Two columns at a time in bf16x2: (code | 0x4300) is the bf16 128 + code, so (128 + q) - (128 + z) and the product with
            // the scale, rounded once to nearest even, are the same bits as the scalar path below.
            const uint4 w0 = __ldcs((const uint4*)(packed + (size_t)kg * N + col)), w1 = __ldcs((const uint4*)(packed + (size_t)kg * N + col + 4));
            const uint4 sv = __ldg((const uint4*)(scales + (size_t)grp * N + col));
            const uint32_t wp[4][2] = {{w0.x, w0.y}, {w0.z, w0.w}, {w1.x, w1.y}, {w1.z, w1.w}};
            const uint32_t sp[4] = {sv.x, sv.y, sv.z, sv.w};
            uint32_t o[8][4];
#pragma unroll
            for (uint32_t pr = 0; pr < 4; ++pr) {
                const uint32_t zz = (((zword >> (8 * pr)) & 0xFu) | (((zword >> (8 * pr + 4)) & 0xFu) << 16)) + 0x43004300u;
                const uint32_t lo = __byte_perm(wp[pr][0], wp[pr][1], 0x5410), hi = __byte_perm(wp[pr][0], wp[pr][1], 0x7632);   // k 0..3, k 4..7
#pragma unroll
                for (uint32_t kk = 0; kk < 4; ++kk) {
                    o[kk][pr] = bf16x2_mul(bf16x2_sub(((lo >> (4 * kk)) & 0x000F000Fu) | 0x43004300u, zz), sp[pr]);
                    o[kk + 4][pr] = bf16x2_mul(bf16x2_sub(((hi >> (4 * kk)) & 0x000F000Fu) | 0x43004300u, zz), sp[pr]);
                }
            }
#pragma unroll
            for (uint32_t kk = 0; kk < 8; ++kk)
                __stcs((uint4*)(out + (size_t)(kg * 8 + kk) * N + col), make_uint4(o[kk][0], o[kk][1], o[kk][2], o[kk][3]));
            continue;
        }
#pragma unroll
        for (uint32_t c = 0; c < 8; ++c) {
            const bool in = col + c < N;
            words[c] = in ? packed[(size_t)kg * N + col + c] : 0u;
            sbits[c] = in ? scales[(size_t)grp * N + col + c] : (uint16_t)0;
        }
        float s[8];
        int32_t z[8];
#pragma unroll
        for (uint32_t c = 0; c < 8; ++c) {
            s[c] = __uint_as_float((uint32_t)sbits[c] << 16);
            z[c] = (int32_t)((zword >> (4 * c)) & 0xFu);
        }
#pragma unroll
        for (uint32_t kk = 0; kk < 8; ++kk) {
            uint16_t o[8];
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) {
                const int32_t qv = (int32_t)((words[c] >> (4 * kk)) & 0xFu);
                const float v = __fmul_rn((float)(qv - z[c]), s[c]);
                const uint32_t bits = __float_as_uint(v);
                o[c] = (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
            }
            uint16_t* dst = out + (size_t)(kg * 8 + kk) * N + col;
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c)
                if (col + c < N) dst[c] = o[c];
        }
    }
}

uint32_t grid_for(uint64_t n, uint32_t block) {
    uint64_t gsz = (n + block - 1) / block;
    const uint64_t cap = 148ull * 16;
    return (uint32_t)(gsz < 1 ? 1 : (gsz > cap ? cap : gsz));
}

int launch_w4_dequant(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out, uint32_t K, uint32_t N,
                      uint32_t group) {
    if (K == 0 || N == 0) return T0_OK;
    if (K % 8) return fail(T0_ERR_INVALID, "K=%u must be a multiple of 8 (eight codes per word)", K);
    if (group == 0 || group % 8) return fail(T0_ERR_INVALID, "group size %u must be a positive multiple of 8", group);
    const uint64_t total = (uint64_t)(K / 8) * ((N + 7) / 8);
    dequant_w4_b200_kernel<<<grid_for(total, 256), 256, 0, rt->stream>>>((const uint32_t*)packed, (const uint16_t*)scales,
                                                                        (const uint32_t*)zeros, (uint16_t*)out, K, N, group, (N + 7) / 8);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "dequant launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

}  // namespace

namespace t0 {

// Bytes of caller-provided scratch the fused kernel needs for a grid of `ctas` CTAs: the arrival counters, then two
// 16 x 256 pieces per CTA.
size_t w4a16_fixed_scratch_bytes(uint32_t ctas) { return kCounterRegion + (size_t)ctas * 2 * kPieceFloats * sizeof(float); }
size_t w4a16_counter_region_bytes() { return kCounterRegion; }

// The one launch of the row-layout fused kernel (shapes already checked by the caller): tensor maps over the three weight
// arrays, kernel choice by steps per CTA, programmatic dependent launch.  `scratch` starts with kCounterRegion bytes of
// arrival counters (zero between calls) followed by two pieces per CTA; `stamps` is the optional trace buffer.
static int launch_w4_row_fused(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N,
                        uint32_t K, uint32_t group, void* scratch, uint32_t grid, unsigned long long* stamps) {
    const uint32_t n_bands = ceil_div(N, kBandCols), ksteps = K / kUnitK;
    const uint64_t total = (uint64_t)n_bands * ksteps;
    W4Params p;
    memset(&p, 0, sizeof p);
    p.a = (const uint16_t*)a;
    p.y = (float*)y;
    p.counters = (int*)scratch;
    p.partials = (float*)((uint8_t*)scratch + kCounterRegion);
    p.status = rt->d_status;
    p.M = M; p.N = N; p.K = K;
    p.units_per_group = group / kUnitK;
    p.n_bands = n_bands; p.ksteps = ksteps; p.total_units = (uint32_t)total;
    p.stamps = stamps;
    // the tensor-memory kernel needs the activations of all of a CTA's steps resident beside the ring
    static const bool legacy = getenv("T0_W4_LEGACY") != nullptr;
    const uint32_t units_per_cta = (uint32_t)ceil_div((uint32_t)total, grid);
    const bool use_tc = !legacy && units_per_cta <= (uint32_t)kTcMaxUnits;
    p.a_units = use_tc ? units_per_cta : std::min<uint32_t>(units_per_cta, kMaxAUnits);
    const size_t smem = use_tc ? 1024 + (size_t)p.a_units * kTcBUnitBytes + (size_t)kStages * kStageBytes + 256
                               : 128 + (size_t)kStages * kStageBytes + kRedBytes + 256 + (size_t)p.a_units * (kUnitK / 8) * kARecord;
    CUtensorMap map_w, map_s, map_z;
    int rc = gemm::make_map_2d_plain(&map_w, (const void*)packed, 4, K / 8, N, kBandCols, kUnitK / 8);
    if (rc != T0_OK) return rc;
    rc = gemm::make_map_2d_plain(&map_s, (const void*)scales, 2, K / group, N, kBandCols, 1);
    if (rc != T0_OK) return rc;
    rc = gemm::make_map_2d_plain(&map_z, (const void*)zeros, 4, K / group, N / 8, kBandCols / 8, 1);
    if (rc != T0_OK) return rc;
    static bool attr_set[64] = {};
    if (rt->device < 64 && !attr_set[rt->device]) {
        T0_CUDA(cudaFuncSetAttribute(w4a16_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem));
        T0_CUDA(cudaFuncSetAttribute(w4a16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)(1024 + (size_t)kTcMaxUnits * kTcBUnitBytes + (size_t)kStages * kStageBytes + 256)));
        attr_set[rt->device] = true;
    }
    // programmatic dependent launch: the next kernel's launch and barrier set-up overlap this one's tail; the kernel
    // touches global memory only after griddepcontrol.wait
    static const bool use_pdl = getenv("T0_NO_PDL") == nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(use_tc ? kTcThreads : kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = rt->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    cudaError_t le = use_tc ? cudaLaunchKernelEx(&cfg, w4a16_tc_kernel, map_w, map_s, map_z, p)
                            : cudaLaunchKernelEx(&cfg, w4a16_gemm_kernel, map_w, map_s, map_z, p);
    if (le != cudaSuccess) return fail(T0_ERR_CUDA, "W4A16 kernel launch failed: %s", cudaGetErrorString(le));
    rt->launches.fetch_add(1);
    return T0_OK;
}

// The fused kernel on scratch memory the caller owns (first kCounterRegion bytes: counters, zero before the first use;
// the kernel leaves them zero).  Takes only the shapes the fused kernel handles and never allocates: there is no
// two-step fallback here.
int w4a16_fused_launch_fixed(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N,
                             uint32_t K, uint32_t group, void* scratch, size_t scratch_bytes) {
    if (M == 0 || N == 0) return T0_OK;
    if (!a || !packed || !scales || !zeros || !y || !scratch) return fail(T0_ERR_INVALID, "null device pointer");
    if (M > 16) return fail(T0_ERR_UNSUPPORTED, "M=%u: this entry takes M <= 16 only (larger M needs a K x N scratch matrix)", M);
    if (K == 0 || K % kUnitK || group == 0 || group % kUnitK || K % group || N % 32)
        return fail(T0_ERR_UNSUPPORTED, "shape K=%u N=%u group=%u: this entry needs K %% 128 == 0, group %% 128 == 0, group | K, N %% 32 == 0", K, N, group);
    if (((a | packed | scales | zeros) & 15) != 0 || (y & 3) != 0) return fail(T0_ERR_INVALID, "operands must be 16-byte aligned (y: 4-byte)");
    const uint32_t n_bands = ceil_div(N, kBandCols), ksteps = K / kUnitK;
    const uint64_t total = (uint64_t)n_bands * ksteps;
    if (total > 0x7FFFFFFFull || n_bands * sizeof(int) > kCounterRegion)
        return fail(T0_ERR_UNSUPPORTED, "N=%u is beyond the fixed scratch: at most %zu bands of 256 columns", N, kCounterRegion / sizeof(int));
    const uint32_t grid = (uint32_t)std::min<uint64_t>(total, (uint64_t)rt->sm_count);
    if (w4a16_fixed_scratch_bytes(grid) > scratch_bytes)
        return fail(T0_ERR_UNSUPPORTED, "a grid of %u CTAs needs %zu bytes of scratch, the fixed area holds %zu", grid, w4a16_fixed_scratch_bytes(grid), scratch_bytes);
    return launch_w4_row_fused(rt, a, packed, scales, zeros, y, M, N, K, group, scratch, grid, nullptr);
}

}  // namespace t0

namespace t0 {
bool w4a16_umma_supported(uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N, uint32_t K, uint32_t group);
int launch_w4a16_umma(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N, uint32_t K,
                      uint32_t group);
int launch_w4a16_umma_grouped(t0_runtime* rt, const t0_w4a16_args* args, uint32_t count);
}  // namespace t0

extern "C" {

int t0_w4_dequant(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t out_bf16, uint32_t K, uint32_t N, uint32_t group) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!packed || !scales || !zeros || !out_bf16) return fail(T0_ERR_INVALID, "null device pointer");
    DeviceGuard guard(rt->device);
    return launch_w4_dequant(rt, packed, scales, zeros, out_bf16, K, N, group);
}

int t0_dequant_int4(t0_runtime* rt, uint64_t packed, uint64_t scales, uint64_t zero_points, uint64_t out, uint32_t rows, uint32_t cols,
                    uint32_t group_size_log2, int out_bf16) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    const uint64_t total = (uint64_t)rows * cols;
    if (total == 0) return T0_OK;
    if (!packed || !scales || !zero_points || !out) return fail(T0_ERR_INVALID, "null device pointer");
    if (group_size_log2 > 31) return fail(T0_ERR_INVALID, "group_size_log2=%u out of range", group_size_log2);
    DeviceGuard guard(rt->device);
    dequant_int4_ref_kernel<<<grid_for((total + 7) / 8, 256), 256, 0, rt->stream>>>(
        (const uint8_t*)packed, (const float*)scales, (const int32_t*)zero_points, (void*)out, total, group_size_log2, out_bf16 ? 1u : 0u);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "dequant launch failed: %s", cudaGetErrorString(e));
    rt->launches.fetch_add(1);
    return T0_OK;
}

int t0_w4a16_gemm(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N,
                  uint32_t K, uint32_t group) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (M == 0 || N == 0) return T0_OK;
    if (!a || !packed || !scales || !zeros || !y) return fail(T0_ERR_INVALID, "null device pointer");
    if (K == 0 || K % 8) return fail(T0_ERR_INVALID, "K=%u must be a positive multiple of 8 (eight codes per word)", K);
    if (group == 0 || group % 8 || K % group) return fail(T0_ERR_INVALID, "group size %u must divide K=%u and be a multiple of 8", group, K);
    DeviceGuard guard(rt->device);

    const uint32_t n_bands = ceil_div(N, kBandCols), ksteps = ceil_div(K, kUnitK);
    const uint64_t total = (uint64_t)n_bands * ksteps;
    const uint32_t grid = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(total, 1), (uint64_t)rt->sm_count);
    // the TMA views need 16-byte row pitches: N % 32 for the zero points (N/8 words per row)
    const bool fused = M <= 16 && (N % 32 == 0) && (K % kUnitK == 0) && (group % kUnitK == 0) && total <= 0x7FFFFFFFull &&
                       n_bands * sizeof(int) <= kCounterRegion &&
                       ((a | packed | scales | zeros) & 15) == 0 && (y & 3) == 0;
    static const bool two_step = getenv("T0_W4_TWO_STEP") != nullptr;     // comparison switch: never the fused tcgen05 kernel
    if (!fused && !two_step && M > 16 && w4a16_umma_supported(a, packed, scales, zeros, y, M, N, K, group))
        return launch_w4a16_umma(rt, a, packed, scales, zeros, y, M, N, K, group);     // 16 < M <= 128: dequantisation in the main loop of a tcgen05 GEMM
    if (!fused) {
        // general shapes: dequantise once into scratch, then the tcgen05 GEMM on B[K,N]
        rc = ensure_scratch(rt, rt->scratch_w, (size_t)K * N * 2);
        if (rc != T0_OK) return rc;
        rc = launch_w4_dequant(rt, packed, scales, zeros, (uint64_t)(uintptr_t)rt->scratch_w.ptr, K, N, group);
        if (rc != T0_OK) return rc;
        t0_gemm_args ga;
        memset(&ga, 0, sizeof ga);
        ga.x = a; ga.b = (uint64_t)(uintptr_t)rt->scratch_w.ptr; ga.y = y;
        ga.m = M; ga.n = N; ga.k = K; ga.transpose = T0_NN; ga.swap_grid = 1;
        return t0_gemm_launch(rt, &ga);
    }

    // scratch: one arrival counter per band (zero between calls) in a fixed region, then two M x 256 pieces per CTA
    const size_t piece_bytes = (size_t)grid * 2 * kPieceFloats * sizeof(float);
    const size_t need = kCounterRegion + piece_bytes;
    if (need > rt->scratch_w4.size) {
        rc = ensure_scratch(rt, rt->scratch_w4, need);
        if (rc != T0_OK) return rc;
        T0_CUDA(cudaMemsetAsync(rt->scratch_w4.ptr, 0, kCounterRegion, rt->stream));
    }
    // T0_W4_TRACE=1: per-CTA stage stamps, summarised on stderr after a blocking wait (a debugging aid, off by default)
    static const bool trace = getenv("T0_W4_TRACE") != nullptr;
    StampBuffer stamps;
    if (trace) {
        rc = stamps.make(grid);
        if (rc != T0_OK) return rc;
    }
    rc = launch_w4_row_fused(rt, a, packed, scales, zeros, y, M, N, K, group, rt->scratch_w4.ptr, grid, stamps.d);
    if (rc != T0_OK) return rc;
    if (trace) {
        std::vector<unsigned long long> h(stamps.words);
        T0_CUDA(cudaStreamSynchronize(rt->stream));
        T0_CUDA(cudaMemcpy(h.data(), stamps.d, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        unsigned long long t_min = ~0ull, t_max = 0;
        double stage = 0, loop = 0, tail = 0;
        for (uint32_t c = 0; c < grid; ++c) {
            t_min = std::min(t_min, h[c * 4]); t_max = std::max(t_max, h[c * 4 + 3]);
            stage += (double)(h[c * 4 + 1] - h[c * 4]); loop += (double)(h[c * 4 + 2] - h[c * 4 + 1]); tail += (double)(h[c * 4 + 3] - h[c * 4 + 2]);
        }
        fprintf(stderr, "[w4a16 trace] M=%u N=%u K=%u: first entry -> last exit %.2f us; per CTA mean: staging %.2f us, main loop %.2f us, flush+exit %.2f us\n",
                M, N, K, (t_max - t_min) * 1e-3, stage / grid * 1e-3, loop / grid * 1e-3, tail / grid * 1e-3);
    }
    return T0_OK;
}

int t0_w4a16_gemm_batch(t0_runtime* rt, const t0_w4a16_args* args, size_t count) {
    if (!args && count) return fail(T0_ERR_INVALID, "null arguments");
    for (size_t i = 0; i < count; ++i) {
        const t0_w4a16_args& a = args[i];
        int rc = t0_w4a16_gemm(rt, a.a, a.packed, a.scales, a.zeros, a.y, a.m, a.n, a.k, a.group);
        if (rc != T0_OK) return rc;
    }
    return T0_OK;
}

int t0_w4a16_gemm_grouped(t0_runtime* rt, const t0_w4a16_args* args, size_t count) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!args && count) return fail(T0_ERR_INVALID, "null arguments");
    if (count == 0) return T0_OK;
    const t0_w4a16_args& a0 = args[0];
    bool same = true;
    for (size_t i = 0; i < count; ++i) {
        const t0_w4a16_args& a = args[i];
        if (!a.a || !a.packed || !a.scales || !a.zeros || !a.y) return fail(T0_ERR_INVALID, "null device pointer in problem %zu", i);
        if (a.m != a0.m || a.n != a0.n || a.k != a0.k || a.group != a0.group) same = false;
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
    static const bool two_step = getenv("T0_W4_TWO_STEP") != nullptr;
    const bool grouped = same && count > 1 && !two_step && a0.m > 16 &&
                         w4a16_umma_supported(a0.a, a0.packed, a0.scales, a0.zeros, a0.y, a0.m, a0.n, a0.k, a0.group);
    if (!grouped) return t0_w4a16_gemm_batch(rt, args, count);
    DeviceGuard guard(rt->device);
    for (size_t i = 0; i < count; i += 32) {
        const size_t n = std::min<size_t>(32, count - i);
        bool ok = true;
        for (size_t j = 0; j < n; ++j) {
            const t0_w4a16_args& a = args[i + j];
            ok = ok && w4a16_umma_supported(a.a, a.packed, a.scales, a.zeros, a.y, a.m, a.n, a.k, a.group);
        }
        rc = ok ? launch_w4a16_umma_grouped(rt, args + i, (uint32_t)n) : t0_w4a16_gemm_batch(rt, args + i, n);
        if (rc != T0_OK) return rc;
    }
    return T0_OK;
}

// ------------------------------------------------------------------ GptqWeight container (host side)

int t0_gptq_parse(const uint8_t* raw, size_t len, uint32_t* rows, uint32_t* cols, uint32_t* group_size, size_t* packed_off,
                  size_t* scales_off, size_t* zero_points_off) {
    // quant_kernels.rs:251-286 (`from_bytes` asserts become error codes)
    if (!raw || !rows || !cols || !group_size || !packed_off || !scales_off || !zero_points_off) return fail(T0_ERR_INVALID, "null argument");
    if (len < 12) return fail(T0_ERR_INVALID, "GPTQ data too short (need at least 12 bytes header)");
    auto rd = [&](size_t o) { return (uint32_t)raw[o] | ((uint32_t)raw[o + 1] << 8) | ((uint32_t)raw[o + 2] << 16) | ((uint32_t)raw[o + 3] << 24); };
    *rows = rd(0); *cols = rd(4); *group_size = rd(8);
    if (*group_size == 0) return fail(T0_ERR_INVALID, "GPTQ group size is zero");
    // the sizes below come from an untrusted header: every product and sum is checked for overflow before it is compared
    // with `len`, and the shapes t0_gptq_to_b200 cannot repack are refused here already
    if (*cols % *group_size) return fail(T0_ERR_INVALID, "GPTQ cols=%u is not a multiple of the group size %u", *cols, *group_size);
    size_t n_elems = 0, n_params = 0, param_bytes = 0, expected = 0;
    if (__builtin_mul_overflow((size_t)*rows, (size_t)*cols, &n_elems)) return fail(T0_ERR_BOUNDS, "GPTQ header: rows*cols overflows");
    if (n_elems & 1) return fail(T0_ERR_INVALID, "GPTQ rows*cols=%zu is odd: two codes share a byte", n_elems);
    if (__builtin_mul_overflow((size_t)(*cols / *group_size), (size_t)*rows, &n_params) || __builtin_mul_overflow(n_params, (size_t)8, &param_bytes))
        return fail(T0_ERR_BOUNDS, "GPTQ header: parameter count overflows");
    const size_t packed_len = n_elems / 2;
    if (__builtin_add_overflow(packed_len, param_bytes, &expected) || __builtin_add_overflow(expected, (size_t)12, &expected))
        return fail(T0_ERR_BOUNDS, "GPTQ header: total size overflows");
    if (len < expected) return fail(T0_ERR_BOUNDS, "GPTQ data truncated: need %zu bytes, got %zu", expected, len);
    *packed_off = 12; *scales_off = 12 + packed_len; *zero_points_off = 12 + packed_len + n_params * 4;
    return T0_OK;
}

size_t t0_gptq_gpu_buffer_size(uint32_t rows, uint32_t cols, uint32_t group_size) {
    // quant_kernels.rs:289-293
    if (group_size == 0) return 0;
    const size_t n_params = (size_t)(cols / group_size) * rows;
    return (size_t)rows * cols / 2 + n_params * 8;
}

long t0_gptq_to_b200(const uint8_t* packed, const float* scales, const int32_t* zero_points, uint32_t rows, uint32_t cols,
                     uint32_t group_size, uint32_t* packed_out, uint16_t* scales_out, uint32_t* zeros_out) {
    if (!packed || !scales || !zero_points || !packed_out || !scales_out || !zeros_out) { fail(T0_ERR_INVALID, "null argument"); return -1; }
    if (group_size == 0 || cols % group_size || cols % 8) { fail(T0_ERR_INVALID, "cols=%u must be a multiple of 8 and of the group size %u", cols, group_size); return -1; }
    const uint32_t N = rows, K = cols, n_groups = cols / group_size, nz = (N + 7) / 8;
    memset(packed_out, 0, (size_t)(K / 8) * N * 4);
    memset(zeros_out, 0, (size_t)n_groups * nz * 4);
    long inexact = 0;
    for (uint32_t n = 0; n < N; ++n) {
        for (uint32_t k = 0; k < K; ++k) {
            const uint64_t e = (uint64_t)n * K + k;
            const uint8_t b = packed[e >> 1];
            const uint32_t code = (e & 1) ? (b >> 4) : (b & 0xFu);
            packed_out[(size_t)(k >> 3) * N + n] |= code << (4 * (k & 7));
        }
        for (uint32_t gi = 0; gi < n_groups; ++gi) {
            const int32_t z = zero_points[(size_t)n * n_groups + gi];
            if (z < 0 || z > 15) { fail(T0_ERR_UNSUPPORTED, "zero point %d of row %u group %u does not fit four bits", z, n, gi); return -1; }
            zeros_out[(size_t)gi * nz + (n >> 3)] |= (uint32_t)z << (4 * (n & 7));
            uint32_t bits;
            const float s = scales[(size_t)n * n_groups + gi];
            memcpy(&bits, &s, 4);
            const uint16_t sb = (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
            if (((uint32_t)sb << 16) != bits) ++inexact;
            scales_out[(size_t)gi * N + n] = sb;
        }
    }
    return inexact;
}

}  // extern "C"

// CUDA-runtime shim behind the reference's GpuRuntime / GpuBuffer / GpuKernel API
// (src/ignis/gpu_context.rs:31-92,99-119,151-597; src/kfd/buffer.rs:9-146; src/kfd/kernel.rs:8-19):
// one in-order stream stands in for the AQL queue, a size-keyed pool for BufferPool, a name-keyed
// table of precompiled sm_100a kernels for the JIT kernel cache, and a poison flag with the same
// fail-fast meaning.  The kernarg blobs the reference's builders produce are decoded here.
#include "runtime_internal.h"

using namespace t0;

namespace {

struct GemmRequest {
    uint64_t x, b, y, bias;
    uint32_t m, n, k;
    uint32_t tile_n, split_k;
    bool nn, out_bf16, planes, swap_grid;
    int pair;                  // 0 = choose by shape, 1 = CTA-pair kernel, 2 = single-CTA kernel
    uint64_t plane_stride;     // elements; only when planes
    uint8_t epilogue, n_ops;
    uint8_t ops[T0_TILE_MAX_EPILOGUE];
    float scale, clamp_min, clamp_max;
    uint64_t peer_y[kMaxPeerY];   // gathered output: further f32 [M,N] destinations (other GPUs' memory), see t0_gemm_launch_gather
    uint32_t n_peer_y;
};

uint32_t choose_tile_n(const t0_runtime* rt, uint32_t m, uint32_t n, uint32_t k, uint32_t split) {
    // widest tile that still gives every SM work; HBM-bound skinny shapes want many CTAs in flight
    const uint32_t tiles_m = ceil_div(m, 128);
    static const uint32_t tns[] = {256, 128, 64, 32};
    for (uint32_t tn : tns) {
        if (tn > 32 && n <= tn / 2) continue;
        if ((uint64_t)tiles_m * ceil_div(n, tn) * split >= (uint64_t)rt->sm_count) return tn;
    }
    (void)k;
    return 32;   // nothing fills the machine: take the most CTAs
}

// The common path of every GEMM entry point: staging for shapes TMA cannot address, the tcgen05
// kernel, and the device-side split-K reduction when the caller did not ask for planes.
int run_gemm(t0_runtime* rt, const GemmRequest& q_in) {
    GemmRequest q = q_in;
    if (q.m == 0 || q.n == 0) return T0_OK;
    // A caller that fixed nothing (tile width 0, kernel 0, no split, complete result wanted) gets the cost model's choice
    // for the shape: tile, CTA pair or not, and split-K with the device-side reduction.  (The "widest tile that fills the
    // machine" rule below picked 64-wide tiles for 128 x 11008 x 4096, 45 us against 28 us for the model's 128 x 128.)
    if (q.tile_n == 0 && q.pair == 0 && q.split_k <= 1 && !q.planes && q.k >= 64) {
        t0_gemm_config c;
        if (t0_cached_auto_select(q.m, q.k, q.n, &c) == T0_OK) {
            const uint32_t s = c.split_k > 1 ? c.split_k : 1;
            const bool split_ok = s == 1 || (q.k % s == 0 && (q.k / s) % 8 == 0 && q.k % 8 == 0 && !(q.x & 15) && !(q.b & 15) && (!q.nn || q.n % 8 == 0));
            if (split_ok) {
                q.tile_n = c.tile_n;
                q.split_k = s;
                q.pair = c.wgp_mode ? 1 : 2;
            }
        }
    }
    if (!q.x || !q.b || !q.y) return fail(T0_ERR_INVALID, "null device pointer in GEMM arguments");
    const bool needs_bias = q.n_ops ? std::find(q.ops, q.ops + q.n_ops, (uint8_t)T0_TEPI_BIAS_ADD) != q.ops + q.n_ops
                                    : q.epilogue != T0_EPI_STORE_F32;
    if (needs_bias && !q.bias) return fail(T0_ERR_INVALID, "epilogue needs a bias vector but bias is null");
    uint32_t split = q.split_k > 1 ? q.split_k : 1;
    if (q.n_peer_y && (split > 1 || q.k == 0 || q.out_bf16 || q.planes))
        return fail(T0_ERR_UNSUPPORTED, "a gathered output takes a plain f32 product: no split-K, no bf16 output, K > 0");
    if (q.k == 0) {
        // empty contraction: the sum is zero, the epilogue still applies
        int rc0 = launch_splitk_reduce(nullptr, (void*)q.y, (const float*)q.bias, q.m, q.n, 0, q.out_bf16, q.epilogue, q.n_ops,
                                       q.ops, q.scale, q.clamp_min, q.clamp_max, rt->stream);
        if (rc0 == T0_OK) rt->launches.fetch_add(1);
        return rc0;
    }
    if (q.k % split) return fail(T0_ERR_INVALID, "K=%u is not divisible by split_k=%u", q.k, split);   // gemm_gen callers filter this
    if (q.planes && (q.out_bf16 || q.n_ops || q.epilogue != T0_EPI_STORE_F32) && split > 1)
        return fail(T0_ERR_INVALID, "split-K planes are raw f32 partial sums: no epilogue or bf16 output");

    GemmLaunch g;
    memset(&g, 0, sizeof g);
    g.x = (const void*)q.x; g.b = (const void*)q.b;
    g.m = q.m; g.n = q.n; g.k = q.k;
    g.nn = q.nn; g.swap_grid = q.swap_grid;
    g.status = rt->d_status; g.probe = rt->d_probe; g.n_sms = (uint32_t)rt->sm_count;
    g.wait_limit_ns = rt->wait_limit_ns.load(std::memory_order_relaxed);
    g.drop_load = rt->drop_next_load.exchange(0) != 0;
    g.split_k = split;
    g.tile_n = q.tile_n ? snap_tile_n(q.tile_n) : choose_tile_n(rt, q.m, q.n, q.k, split);
    if (q.nn && g.tile_n < 64) g.tile_n = 64;
    // the CTA-pair kernel (256 x 256 tiles) pays off once there are enough tiles to fill the machine
    const bool pair_fits = (uint64_t)ceil_div(q.m, 256) * ceil_div(q.n, 256) * split >= (uint64_t)rt->sm_count / 2;
    // (with B[K,N] the half tiles of a 128-wide pair tile would be 32 columns per CTA, under the 64-column box: 256-wide only)
    const bool pair_ok = !q.nn || q.tile_n == 0 || q.tile_n >= 256;
    const bool use_pair = pair_ok && (q.pair == 1 || (q.pair == 0 && pair_fits && (q.tile_n == 0 || q.tile_n >= 256)));
    if (use_pair) g.tile_n = q.tile_n;   // 0/256 -> 256-wide pair tiles, <= 128 -> 128-wide
    auto launch = [&](const GemmLaunch& gl) { return use_pair ? launch_gemm_sm100_pair(gl, rt->stream) : launch_gemm_sm100(gl, rt->stream); };

    // --- staging for shapes the TMA path cannot address (row stride or base not 16-byte aligned)
    const uint32_t kps = q.k / split;
    const bool x_bad = (q.k % 8) || (q.x & 15);
    const bool b_bad = q.nn ? ((q.n % 8) || (q.b & 15)) : ((q.k % 8) || (q.b & 15));
    if ((x_bad || b_bad || (kps % 8)) && split > 1)
        return fail(T0_ERR_UNSUPPORTED, "split-K needs K/split_k %% 8 == 0 and 16-byte aligned operands (K=%u, split_k=%u)", q.k, split);
    const uint32_t k_pad = (q.k + 7) & ~7u;
    if (x_bad) {
        int rc = ensure_scratch(rt, rt->scratch_a, (size_t)q.m * k_pad * 2);
        if (rc != T0_OK) return rc;
        rc = launch_pad_copy_u16((const void*)q.x, rt->scratch_a.ptr, q.m, q.k, k_pad, rt->stream);
        if (rc != T0_OK) return rc;
        rt->launches.fetch_add(1);
        g.x = rt->scratch_a.ptr; g.ldx = k_pad;
    }
    if (b_bad) {
        if (q.nn) {
            const uint32_t n_pad = (q.n + 7) & ~7u;
            int rc = ensure_scratch(rt, rt->scratch_b, (size_t)q.k * n_pad * 2);
            if (rc != T0_OK) return rc;
            rc = launch_pad_copy_u16((const void*)q.b, rt->scratch_b.ptr, q.k, q.n, n_pad, rt->stream);
            if (rc != T0_OK) return rc;
            g.b = rt->scratch_b.ptr; g.ldb = n_pad;
        } else {
            int rc = ensure_scratch(rt, rt->scratch_b, (size_t)q.n * k_pad * 2);
            if (rc != T0_OK) return rc;
            rc = launch_pad_copy_u16((const void*)q.b, rt->scratch_b.ptr, q.n, q.k, k_pad, rt->stream);
            if (rc != T0_OK) return rc;
            g.b = rt->scratch_b.ptr; g.ldb = k_pad;
        }
        rt->launches.fetch_add(1);
    }

    const bool fused_reduce = split > 1 && !q.planes;
    if (fused_reduce && !use_pair) {
        // one launch: the CTAs that share a tile form a cluster and add their partial sums through distributed shared
        // memory (T0_NO_CLUSTER_SPLITK=1 keeps the two-launch form below for comparison)
        static const bool no_cluster = getenv("T0_NO_CLUSTER_SPLITK") != nullptr;
        GemmLaunch gc = g;
        gc.y = (void*)q.y; gc.plane_stride = 0; gc.bias = (const float*)q.bias;
        gc.out_bf16 = q.out_bf16; gc.epilogue = q.epilogue; gc.n_ops = q.n_ops;
        memcpy(gc.ops, q.ops, sizeof gc.ops);
        gc.scale = q.scale; gc.clamp_min = q.clamp_min; gc.clamp_max = q.clamp_max;
        if (!no_cluster && !x_bad && !b_bad && gemm_splitk_cluster_supported(gc)) {
            int rc = launch_gemm_sm100_splitk(gc, rt->stream);
            if (rc != T0_OK) return rc;
            rt->launches.fetch_add(1);
            return T0_OK;
        }
    }
    if (fused_reduce) {
        // partial planes go to scratch; K4 sums them in split order and applies the epilogue
        const size_t mn = (size_t)q.m * q.n;
        int rc = ensure_scratch(rt, rt->scratch_planes, mn * split * sizeof(float));
        if (rc != T0_OK) return rc;
        g.y = rt->scratch_planes.ptr; g.plane_stride = mn;
        g.out_bf16 = false; g.epilogue = T0_EPI_STORE_F32; g.n_ops = 0;
        rc = launch(g);
        if (rc != T0_OK) return rc;
        rt->launches.fetch_add(1);
        rc = launch_splitk_reduce((const float*)rt->scratch_planes.ptr, (void*)q.y, (const float*)q.bias, q.m, q.n, split,
                                  q.out_bf16, q.epilogue, q.n_ops, q.ops, q.scale, q.clamp_min, q.clamp_max, rt->stream);
        if (rc != T0_OK) return rc;
        rt->launches.fetch_add(1);
        return T0_OK;
    }
    if (q.n_peer_y) {
        // the destinations' tensor maps live in a per-runtime device slot; they are rewritten (stream-ordered) only when the
        // destinations or the shape differ from the launch before
        std::vector<uint64_t> key(q.peer_y, q.peer_y + q.n_peer_y);
        key.push_back(((uint64_t)q.m << 32) | q.n);
        if (!rt->d_peer_maps) T0_CUDA(cudaMalloc(&rt->d_peer_maps, kMaxPeerY * 128));
        g.n_peer_y = q.n_peer_y;
        for (uint32_t i = 0; i < q.n_peer_y; ++i) g.peer_y[i] = (void*)q.peer_y[i];
        g.peer_map_slot = rt->d_peer_maps;
        g.peer_maps_staged = key == rt->peer_maps_key;
        rt->peer_maps_key = key;
    }
    g.y = (void*)q.y;
    g.plane_stride = split > 1 ? (q.plane_stride ? q.plane_stride : (uint64_t)q.m * q.n) : 0;
    g.bias = (const float*)q.bias;
    g.out_bf16 = q.out_bf16; g.epilogue = q.epilogue; g.n_ops = q.n_ops;
    memcpy(g.ops, q.ops, sizeof g.ops);
    g.scale = q.scale; g.clamp_min = q.clamp_min; g.clamp_max = q.clamp_max;
    int rc = launch(g);
    if (rc != T0_OK) return rc;
    rt->launches.fetch_add(1);
    return T0_OK;
}

// Bytes available from `addr` to the end of the live allocation containing it, or SIZE_MAX when the
// address belongs to no allocation of this runtime (foreign device memory).
size_t extent_from(t0_runtime* rt, uint64_t addr) {
    std::lock_guard<std::mutex> g(rt->mu);
    auto it = rt->live.upper_bound((uintptr_t)addr);
    if (it == rt->live.begin()) return SIZE_MAX;
    --it;
    if (addr >= it->first + it->second) return SIZE_MAX;
    return (size_t)(it->first + it->second - addr);
}

uint32_t rd_u32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
uint64_t rd_u64(const uint8_t* p) { return (uint64_t)rd_u32(p) | ((uint64_t)rd_u32(p + 4) << 32); }
float rd_f32(const uint8_t* p) { uint32_t b = rd_u32(p); float f; memcpy(&f, &b, 4); return f; }

// Decode a kernarg blob + grid into a GEMM request (the work the reference's kernel would do).
int decode_dispatch(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* ka, size_t len, bool validate,
                    GemmRequest* out) {
    // gpu_context.rs:319-322: assert_eq!(kernargs.len(), kernel.kernarg_size)
    if (len != k->kernarg_size)
        return fail(T0_ERR_INVALID, "kernarg mismatch: builder produced %zuB, kernel declares %uB", len, k->kernarg_size);
    GemmRequest q;
    memset(&q, 0, sizeof q);
    q.x = rd_u64(ka); q.b = rd_u64(ka + 8); q.y = rd_u64(ka + 16);
    q.k = rd_u32(ka + 24); q.n = rd_u32(ka + 28);
    const uint32_t y_split_stride = rd_u32(ka + 36);
    q.scale = 1.0f;
    uint32_t tile_m, tile_n, wg, sk;
    bool swap;
    if (k->kind == 0) {
        const t0_gemm_config& c = k->cfg;
        tile_m = c.tile_m; tile_n = c.tile_n; wg = c.wg_size; sk = split_of(&c); swap = c.swap_grid;
        q.nn = c.transpose == T0_NN; q.epilogue = c.epilogue;
        // wgp_mode on a 256 x 256 tile is the CTA pair; every other config runs the single-CTA kernel
        q.pair = (c.wgp_mode && c.tile_m == 256 && c.tile_n == 256) ? 1 : 2;
        if (c.epilogue != T0_EPI_STORE_F32) q.bias = rd_u64(ka + 40);
    } else {
        const t0_tile_gemm& s = k->spec;
        tile_m = s.tile_m; tile_n = s.tile_n; wg = t0_tile_gemm_wg_size(&s); sk = s.split_k ? s.split_k : 1; swap = s.swap_grid;
        q.nn = s.transpose == T0_NN;
        q.pair = 2;
        q.m = rd_u32(ka + 40);
        q.n_ops = s.n_epilogue;
        memcpy(q.ops, s.epilogue, sizeof q.ops);
        size_t off = s.persistent ? 64 : 44;
        bool has_bias = false, has_scale = false, has_clamp = false;
        for (uint32_t i = 0; i < s.n_epilogue; ++i) {
            has_bias |= s.epilogue[i] == T0_TEPI_BIAS_ADD;
            has_scale |= s.epilogue[i] == T0_TEPI_SCALE;
            has_clamp |= s.epilogue[i] == T0_TEPI_CLAMP;
        }
        if (has_bias) { off = (off + 7) & ~(size_t)7; q.bias = rd_u64(ka + off); off += 8; }
        if (has_scale) { q.scale = rd_f32(ka + off); off += 4; }
        if (has_clamp) { q.clamp_min = rd_f32(ka + off); q.clamp_max = rd_f32(ka + off + 4); off += 8; }
    }
    if (wg == 0 || tile_m == 0 || tile_n == 0) return fail(T0_ERR_INVALID, "degenerate kernel configuration");
    if (grid[2] != 1 && grid[2] != 0) return fail(T0_ERR_INVALID, "grid z must be 1");
    uint32_t tiles_m, tiles_n;
    if (k->kind == 1 && k->spec.persistent) {
        // tile_ir.rs:4646-4655: one workgroup loops over every tile
        tiles_m = ceil_div(q.m, tile_m); tiles_n = ceil_div(q.n, tile_n);
    } else {
        if (grid[0] % wg) return fail(T0_ERR_INVALID, "grid x=%u is not a multiple of the workgroup size %u", grid[0], wg);
        if (grid[1] % sk) return fail(T0_ERR_INVALID, "grid y=%u is not a multiple of split_k=%u", grid[1], sk);
        const uint32_t gx = grid[0] / wg, gy = grid[1] / sk;
        tiles_n = swap ? gx : gy;
        tiles_m = swap ? gy : gx;
    }
    if (k->kind == 0) {
        // the 40/48-byte blob has no M: every row of every launched tile is computed
        q.m = tiles_m * tile_m;
        if (sk > 1 && y_split_stride && q.n) q.m = std::min<uint32_t>(q.m, y_split_stride / (4u * q.n));
        q.planes = sk > 1;
        q.plane_stride = y_split_stride / 4;
    } else {
        if ((uint64_t)tiles_m * tile_m < q.m) q.m = tiles_m * tile_m;   // rows no workgroup covers stay untouched
        q.planes = false;   // y_split_stride is always 0 in TileIR blobs (tile_ir.rs:4613): reduce on the device
    }
    if ((uint64_t)tiles_n * tile_n < q.n)
        return fail(T0_ERR_INVALID, "grid covers %u columns but N=%u", tiles_n * tile_n, q.n);
    q.split_k = sk;
    q.tile_n = tile_n;
    q.swap_grid = swap;

    // pointer validation against this runtime's live allocations (stronger than gpu_context.rs:380-395);
    // rows that do not fit the caller's buffers are not computed
    const bool strict = validate && getenv("T0_VALIDATE_KA") != nullptr;
    const size_t ex = extent_from(rt, q.x), eb = extent_from(rt, q.b), ey = extent_from(rt, q.y);
    if (strict && (ex == SIZE_MAX || eb == SIZE_MAX || ey == SIZE_MAX))
        return fail(T0_ERR_INVALID, "kernarg pointer outside every live allocation of this runtime");
    if (validate) {
        if (eb != SIZE_MAX && (uint64_t)q.n * q.k * 2 > eb)
            return fail(T0_ERR_BOUNDS, "weight buffer holds %zu bytes, N*K*2 = %llu", eb, (unsigned long long)q.n * q.k * 2);
        if (ex != SIZE_MAX && q.k) q.m = (uint32_t)std::min<uint64_t>(q.m, ex / ((uint64_t)q.k * 2));
        if (ey != SIZE_MAX && q.n) {
            const uint64_t per_row = (uint64_t)q.n * 4;
            if (q.planes && q.plane_stride) {
                if ((uint64_t)(sk - 1) * q.plane_stride * 4 + (uint64_t)q.m * per_row > ey)
                    return fail(T0_ERR_BOUNDS, "output buffer too small for %u split-K planes", sk);
            } else {
                q.m = (uint32_t)std::min<uint64_t>(q.m, ey / per_row);
            }
        }
        if (q.bias) {
            const size_t ebias = extent_from(rt, q.bias);
            if (ebias != SIZE_MAX && (uint64_t)q.n * 4 > ebias) return fail(T0_ERR_BOUNDS, "bias buffer shorter than N floats");
        }
    }
    *out = q;
    return T0_OK;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ runtime

int t0_rt_new(int device, t0_runtime** out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    *out = nullptr;
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev == 0)
        return fail(T0_ERR_CUDA, "no CUDA device available (%s); this library has no CPU fallback", cudaGetErrorString(e));
    if (device < 0 || device >= n_dev) return fail(T0_ERR_INVALID, "device %d out of range (0..%d)", device, n_dev - 1);
    cudaDeviceProp prop;
    T0_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(T0_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a (B200) only", device, prop.major, prop.minor);
    DeviceGuard guard(device);
    std::unique_ptr<t0_runtime> rt(new t0_runtime());
    rt->device = device;
    rt->sm_count = prop.multiProcessorCount;
    T0_CUDA(cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking));
    T0_CUDA(cudaEventCreate(&rt->ev_start));
    T0_CUDA(cudaEventCreate(&rt->ev_stop));
    T0_CUDA(cudaMalloc(&rt->d_status, sizeof(int)));
    T0_CUDA(cudaMemset(rt->d_status, 0, sizeof(int)));
    T0_CUDA(cudaMalloc(&rt->d_probe, (2 + 64) * sizeof(unsigned long long)));   // clock words + eight launches' trace stamps
    T0_CUDA(cudaMemset(rt->d_probe, 0, (2 + 64) * sizeof(unsigned long long)));
    T0_CUDA(cudaMallocHost(&rt->h_status, sizeof(int)));
    *rt->h_status = 0;
    *out = rt.release();
    return T0_OK;
}

void t0_rt_free(t0_runtime* rt) {
    if (!rt) return;
    DeviceGuard guard(rt->device);
    cudaStreamSynchronize(rt->stream);
    host_pipe_free(rt);
    t0_rt_pool_clear(rt);
    for (Scratch* s : {&rt->scratch_a, &rt->scratch_b, &rt->scratch_planes, &rt->scratch_w4, &rt->scratch_w, &rt->scratch_cvt_a, &rt->scratch_cvt_b, &rt->scratch_cvt_c})
        if (s->ptr) cudaFree(s->ptr);
    if (rt->d_status) cudaFree(rt->d_status);
    if (rt->d_probe) cudaFree(rt->d_probe);
    if (rt->d_peer_maps) cudaFree(rt->d_peer_maps);
    if (rt->h_status) cudaFreeHost(rt->h_status);
    if (rt->ev_start) cudaEventDestroy(rt->ev_start);
    if (rt->ev_stop) cudaEventDestroy(rt->ev_stop);
    if (rt->stream) cudaStreamDestroy(rt->stream);
    delete rt;
}

int t0_rt_is_poisoned(const t0_runtime* rt) { return rt && rt->poisoned.load() ? 1 : 0; }

void t0_rt_mark_poisoned(t0_runtime* rt) {
    if (!rt) return;
    rt->poisoned.store(true);
    fprintf(stderr, "[t0b200] runtime POISONED - all subsequent dispatches will fail fast\n");   // gpu_context.rs:195-198
}

int t0_rt_synchronize(t0_runtime* rt) {
    if (!rt) return fail(T0_ERR_INVALID, "null runtime");
    DeviceGuard guard(rt->device);
    return check_status_after_sync(rt);
}

int t0_rt_wait_idle(t0_runtime* rt) { return t0_rt_synchronize(rt); }

int t0_rt_set_wait_limit_ns(t0_runtime* rt, uint64_t ns) {
    if (!rt) return fail(T0_ERR_INVALID, "null runtime");
    rt->wait_limit_ns.store(ns);
    return T0_OK;
}

int t0_rt_selftest_drop_one_load(t0_runtime* rt) {
    if (!rt) return fail(T0_ERR_INVALID, "null runtime");
    rt->drop_next_load.store(1);
    return T0_OK;
}
int t0_rt_reserve_scratch(t0_runtime* rt, int which, size_t bytes) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    DeviceGuard guard(rt->device);
    Scratch* s = nullptr;
    switch (which) {
        case T0_SCRATCH_OPERAND_A: s = &rt->scratch_a; break;
        case T0_SCRATCH_OPERAND_B: s = &rt->scratch_b; break;
        case T0_SCRATCH_SPLITK_PLANES: s = &rt->scratch_planes; break;
        case T0_SCRATCH_W4_WEIGHTS: s = &rt->scratch_w; break;
        case T0_SCRATCH_F32_A: s = &rt->scratch_cvt_a; break;
        case T0_SCRATCH_F32_B: s = &rt->scratch_cvt_b; break;
        case T0_SCRATCH_F32_C: s = &rt->scratch_cvt_c; break;
        case T0_SCRATCH_W4_FUSED: {
            // arrival counters (must start at zero) followed by two pieces per CTA; the size depends only on the device
            const size_t need = std::max(bytes, t0_rt_w4_fused_scratch_bytes(rt));
            if (need > rt->scratch_w4.size) {
                rc = ensure_scratch(rt, rt->scratch_w4, need);
                if (rc != T0_OK) return rc;
                T0_CUDA(cudaMemsetAsync(rt->scratch_w4.ptr, 0, w4a16_counter_region_bytes(), rt->stream));
            }
            return T0_OK;
        }
        default: return fail(T0_ERR_INVALID, "unknown scratch kind %d", which);
    }
    return ensure_scratch(rt, *s, bytes);
}

size_t t0_rt_w4_fused_scratch_bytes(const t0_runtime* rt) {
    return rt ? w4a16_fixed_scratch_bytes((uint32_t)rt->sm_count) : 0;
}

void* t0_rt_stream(const t0_runtime* rt) { return rt ? (void*)rt->stream : nullptr; }
int t0_rt_device(const t0_runtime* rt) { return rt ? rt->device : -1; }
int t0_rt_sm_count(const t0_runtime* rt) { return rt ? rt->sm_count : 0; }
uint64_t t0_rt_launch_count(const t0_runtime* rt) { return rt ? rt->launches.load() : 0; }

int t0_rt_last_kernel_clock(t0_runtime* rt, double* sm_mhz, double* kernel_us) {
    if (!rt || !sm_mhz) return fail(T0_ERR_INVALID, "null argument");
    DeviceGuard guard(rt->device);
    unsigned long long w[2] = {0, 0};
    T0_CUDA(cudaMemcpyAsync(w, rt->d_probe, sizeof w, cudaMemcpyDeviceToHost, rt->stream));
    T0_CUDA(cudaStreamSynchronize(rt->stream));
    *sm_mhz = w[1] ? (double)w[0] / (double)w[1] * 1e3 : 0.0;
    if (kernel_us) *kernel_us = (double)w[1] * 1e-3;
    if (getenv("T0_GEMM_TRACE")) {
        // the pair kernel's CTA 0, last eight launches: entry, prologue done, dependency wait passed, first operands landed,
        // first tile accumulated, last store issued, exit (microseconds after the entry; then the gap to the next entry)
        unsigned long long t[64];
        T0_CUDA(cudaMemcpy(t, rt->d_probe + 2, sizeof t, cudaMemcpyDeviceToHost));
        std::vector<int> order;
        for (int i = 0; i < 8; ++i) if (t[i * 8]) order.push_back(i);
        std::sort(order.begin(), order.end(), [&](int a, int b) { return t[a * 8] < t[b * 8]; });
        for (size_t k = 0; k < order.size(); ++k) {
            const unsigned long long* s = t + order[k] * 8;
            auto us = [&](int i) { return s[i] ? (double)(s[i] - s[0]) * 1e-3 : -1.0; };
            fprintf(stderr, "[gemm trace] prologue %.2f  dep-wait %.2f  first-load %.2f  first-tile %.2f  last-store %.2f  exit %.2f", us(2), us(1), us(3),
                    us(4), us(5), us(6));
            if (s[7]) fprintf(stderr, "  aux %.2f", us(7));
            if (k + 1 < order.size()) fprintf(stderr, "  | next entry %+.2f after exit", ((double)t[order[k + 1] * 8] - (double)s[6]) * 1e-3);
            fprintf(stderr, "\n");
        }
    }
    return T0_OK;
}

int t0_rt_timer_start(t0_runtime* rt) {
    if (!rt) return fail(T0_ERR_INVALID, "null runtime");
    DeviceGuard guard(rt->device);
    T0_CUDA(cudaEventRecord(rt->ev_start, rt->stream));
    return T0_OK;
}

int t0_rt_timer_stop(t0_runtime* rt, float* ms) {
    if (!rt || !ms) return fail(T0_ERR_INVALID, "null argument");
    DeviceGuard guard(rt->device);
    T0_CUDA(cudaEventRecord(rt->ev_stop, rt->stream));
    T0_CUDA(cudaEventSynchronize(rt->ev_stop));
    T0_CUDA(cudaEventElapsedTime(ms, rt->ev_start, rt->ev_stop));
    return T0_OK;
}

// ------------------------------------------------------------------ buffers

int t0_rt_alloc(t0_runtime* rt, size_t n_bytes, t0_buffer** out) {
    if (!rt || !out) return fail(T0_ERR_INVALID, "null argument");
    *out = nullptr;
    DeviceGuard guard(rt->device);
    const size_t aligned = std::max<size_t>(4096, (n_bytes + 4095) / 4096 * 4096);   // gpu_context.rs:55
    {
        std::unique_lock<std::mutex> g(rt->mu);
        auto it = rt->pool.find(aligned);
        if (it != rt->pool.end() && !it->second.empty()) {
            t0_buffer* b = it->second.back();
            it->second.pop_back();
            rt->cached_bytes -= aligned;
            rt->live[(uintptr_t)b->dptr] = b->size;
            g.unlock();
            // gpu_context.rs:57-62: a reused buffer is zeroed before the new owner sees it
            T0_CUDA(cudaMemsetAsync(b->dptr, 0, b->size, rt->stream));
            *out = b;
            return T0_OK;
        }
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, aligned);
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "cudaMalloc(%zu): %s", aligned, cudaGetErrorString(e));
    t0_buffer* b = new t0_buffer{rt, p, aligned};
    {
        std::lock_guard<std::mutex> g(rt->mu);
        rt->live[(uintptr_t)p] = aligned;
    }
    *out = b;
    return T0_OK;
}

int t0_rt_alloc_zero(t0_runtime* rt, size_t n_bytes, t0_buffer** out) {
    int rc = t0_rt_alloc(rt, n_bytes, out);
    if (rc != T0_OK) return rc;
    return t0_buf_zero(*out);
}

int t0_rt_alloc_f32(t0_runtime* rt, size_t n_elems, t0_buffer** out) {
    const size_t bytes = (std::max<size_t>(n_elems * 4, 512) + 511) & ~(size_t)511;   // gpu_context.rs:521
    return t0_rt_alloc_zero(rt, bytes, out);
}

void t0_rt_recycle(t0_runtime* rt, t0_buffer* buf) {
    if (!rt || !buf) return;
    std::lock_guard<std::mutex> g(rt->mu);
    rt->live.erase((uintptr_t)buf->dptr);
    rt->pool[buf->size].push_back(buf);
    rt->cached_bytes += buf->size;
}

size_t t0_rt_pool_cached_bytes(const t0_runtime* rt) { return rt ? rt->cached_bytes : 0; }

void t0_rt_pool_clear(t0_runtime* rt) {
    if (!rt) return;
    DeviceGuard guard(rt->device);
    cudaStreamSynchronize(rt->stream);
    std::lock_guard<std::mutex> g(rt->mu);
    for (auto& kv : rt->pool)
        for (t0_buffer* b : kv.second) { cudaFree(b->dptr); delete b; }
    rt->pool.clear();
    rt->cached_bytes = 0;
}

void t0_buf_free(t0_buffer* buf) {
    if (!buf) return;
    t0_runtime* rt = buf->rt;
    DeviceGuard guard(rt->device);
    cudaStreamSynchronize(rt->stream);
    {
        std::lock_guard<std::mutex> g(rt->mu);
        rt->live.erase((uintptr_t)buf->dptr);
    }
    cudaFree(buf->dptr);
    delete buf;
}

int t0_buf_write_bytes(t0_buffer* buf, size_t offset, const void* data, size_t len) {
    if (!buf || (!data && len)) return fail(T0_ERR_INVALID, "null argument");
    // src/kfd/buffer.rs:76: assert!(offset + data.len() <= self.size)
    if (offset > buf->size || len > buf->size - offset)
        return fail(T0_ERR_BOUNDS, "write of %zu bytes at offset %zu exceeds buffer size %zu", len, offset, buf->size);
    if (len == 0) return T0_OK;
    DeviceGuard guard(buf->rt->device);
    T0_CUDA(cudaMemcpyAsync((uint8_t*)buf->dptr + offset, data, len, cudaMemcpyHostToDevice, buf->rt->stream));
    T0_CUDA(cudaStreamSynchronize(buf->rt->stream));
    return T0_OK;
}

int t0_buf_read_bytes(const t0_buffer* buf, size_t offset, void* out, size_t len) {
    if (!buf || (!out && len)) return fail(T0_ERR_INVALID, "null argument");
    if (offset > buf->size || len > buf->size - offset)
        return fail(T0_ERR_BOUNDS, "read of %zu bytes at offset %zu exceeds buffer size %zu", len, offset, buf->size);
    if (len == 0) return T0_OK;
    DeviceGuard guard(buf->rt->device);
    T0_CUDA(cudaMemcpyAsync(out, (const uint8_t*)buf->dptr + offset, len, cudaMemcpyDeviceToHost, buf->rt->stream));
    T0_CUDA(cudaStreamSynchronize(buf->rt->stream));
    return T0_OK;
}

int t0_buf_write(t0_buffer* buf, const void* data, size_t len) { return t0_buf_write_bytes(buf, 0, data, len); }
int t0_buf_read(const t0_buffer* buf, void* out, size_t len) { return t0_buf_read_bytes(buf, 0, out, len); }

int t0_buf_zero(t0_buffer* buf) {
    if (!buf) return fail(T0_ERR_INVALID, "null buffer");
    DeviceGuard guard(buf->rt->device);
    T0_CUDA(cudaMemsetAsync(buf->dptr, 0, buf->size, buf->rt->stream));
    return T0_OK;
}

uint64_t t0_buf_gpu_addr(const t0_buffer* buf) { return buf ? (uint64_t)(uintptr_t)buf->dptr : 0; }
size_t t0_buf_size(const t0_buffer* buf) { return buf ? buf->size : 0; }

int t0_rt_read_f32(t0_runtime* rt, const t0_buffer* buf, size_t n, float* out) {
    if (!rt || !buf) return fail(T0_ERR_INVALID, "null argument");
    int rc = t0_rt_wait_idle(rt);   // gpu_context.rs:536
    if (rc != T0_OK) return rc;
    return t0_buf_read(buf, out, n * 4);
}

int t0_rt_write_f32(t0_runtime* rt, t0_buffer* buf, const float* data, size_t n) {
    if (!rt || !buf) return fail(T0_ERR_INVALID, "null argument");
    return t0_buf_write(buf, data, n * 4);
}

int t0_rt_upload_f32(t0_runtime* rt, const float* data, size_t n, t0_buffer** out) {
    int rc = t0_rt_alloc_f32(rt, n, out);
    if (rc != T0_OK) return rc;
    return t0_rt_write_f32(rt, *out, data, n);
}

// ------------------------------------------------------------------ kernels

int t0_rt_ensure_gemm_kernel(t0_runtime* rt, const t0_gemm_config* cfg, t0_kernel** out) {
    if (!rt || !cfg || !out) return fail(T0_ERR_INVALID, "null argument");
    // gemm_gen.rs:270-281 panics on an infeasible config; here that is an error code
    if (!t0_gemm_config_is_feasible(cfg)) return fail(T0_ERR_INVALID, "[gemm_gen] config '%s' is not feasible", gemm_config_name(*cfg).c_str());
    std::string name = gemm_config_name(*cfg);
    std::lock_guard<std::mutex> g(rt->mu);
    auto it = rt->kernels.find(name);
    if (it == rt->kernels.end()) {
        std::unique_ptr<t0_kernel> k(new t0_kernel());
        k->name = name;
        k->kind = 0;
        k->cfg = *cfg;
        memset(&k->spec, 0, sizeof k->spec);
        k->kernarg_size = cfg->epilogue == T0_EPI_STORE_F32 ? 40 : 48;   // gemm_gen.rs:442,466
        it = rt->kernels.emplace(name, std::move(k)).first;
    }
    *out = it->second.get();
    return T0_OK;
}

int t0_rt_ensure_tile_kernel(t0_runtime* rt, const t0_tile_gemm* spec, t0_kernel** out) {
    if (!rt || !spec || !out) return fail(T0_ERR_INVALID, "null argument");
    if (spec->tile_m < 16 || spec->tile_m % 16 || spec->tile_n < 16 || spec->tile_n % 16 || spec->tile_k < 16 ||
        spec->n_epilogue > T0_TILE_MAX_EPILOGUE || spec->wmma_format != 0)
        return fail(T0_ERR_INVALID, "TileGemm spec is not supported (tile %ux%ux%u, format %u)", spec->tile_m, spec->tile_n,
                    spec->tile_k, spec->wmma_format);
    uint32_t sk = spec->split_k ? spec->split_k : 1;
    if (sk & (sk - 1)) return fail(T0_ERR_INVALID, "split_k=%u must be a power of 2", sk);
    std::string name = tile_gemm_name(*spec);
    std::lock_guard<std::mutex> g(rt->mu);
    auto it = rt->kernels.find(name);
    if (it == rt->kernels.end()) {
        std::unique_ptr<t0_kernel> k(new t0_kernel());
        k->name = name;
        k->kind = 1;
        k->spec = *spec;
        memset(&k->cfg, 0, sizeof k->cfg);
        uint8_t tmp[96];
        size_t len = 0;
        t0_tile_build_kernargs_epilogue(0, 0, 0, 0, 0, 0, spec, 0, 1.0f, 0.0f, 0.0f, tmp, sizeof tmp, &len);
        k->kernarg_size = (uint32_t)len;
        it = rt->kernels.emplace(name, std::move(k)).first;
    }
    *out = it->second.get();
    return T0_OK;
}

int t0_rt_ensure_dequant_kernel(t0_runtime* rt, uint32_t group_size_log2, int out_bf16, t0_kernel** out) {
    if (!rt || !out) return fail(T0_ERR_INVALID, "null argument");
    if (group_size_log2 > 31) return fail(T0_ERR_INVALID, "group_size_log2=%u out of range", group_size_log2);
    // the reference names both kernels without the group size (quant_kernels.rs:54,128); the group is part of the key here
    std::string name = std::string(out_bf16 ? "dequant_int4_bf16" : "dequant_int4_f32") + "_g" + std::to_string(group_size_log2);
    std::lock_guard<std::mutex> g(rt->mu);
    auto it = rt->kernels.find(name);
    if (it == rt->kernels.end()) {
        std::unique_ptr<t0_kernel> k(new t0_kernel());
        k->name = name;
        k->kind = 2;
        memset(&k->cfg, 0, sizeof k->cfg);
        memset(&k->spec, 0, sizeof k->spec);
        k->group_log2 = group_size_log2;
        k->out_bf16 = out_bf16 != 0;
        k->kernarg_size = 40;
        it = rt->kernels.emplace(name, std::move(k)).first;
    }
    *out = it->second.get();
    return T0_OK;
}

uint32_t t0_kernel_kernarg_size(const t0_kernel* k) { return k ? k->kernarg_size : 0; }
const char* t0_kernel_name(const t0_kernel* k) { return k ? k->name.c_str() : ""; }
size_t t0_rt_kernel_cache_size(const t0_runtime* rt) {
    if (!rt) return 0;
    std::lock_guard<std::mutex> g(const_cast<t0_runtime*>(rt)->mu);
    return rt->kernels.size();
}

// ------------------------------------------------------------------ dispatch

static int dispatch_impl(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* ka, size_t len, bool validate,
                         bool wait) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!k || !grid || !ka) return fail(T0_ERR_INVALID, "null argument");
    DeviceGuard guard(rt->device);
    if (k->kind == 2) {
        // dequant_int4_{f32,bf16}: [packed, scales, zero_points, output: u64 x 4, rows, cols: u32 x 2] (quant_kernels.rs:45-47);
        // the grid is ceil(rows*cols/256)*256 threads there and is not needed here
        if (len != k->kernarg_size)
            return fail(T0_ERR_INVALID, "kernarg mismatch: builder produced %zuB, kernel declares %uB", len, k->kernarg_size);
        rc = t0_dequant_int4(rt, rd_u64(ka), rd_u64(ka + 8), rd_u64(ka + 16), rd_u64(ka + 24), rd_u32(ka + 32), rd_u32(ka + 36),
                             k->group_log2, k->out_bf16 ? 1 : 0);
        if (rc != T0_OK) return rc;
        rt->slot.fetch_add(1);
        return wait ? check_status_after_sync(rt) : T0_OK;
    }
    GemmRequest q;
    rc = decode_dispatch(rt, k, grid, ka, len, validate, &q);
    if (rc != T0_OK) return rc;
    if (getenv("T0_DEBUG_DISPATCH"))   // gpu_context.rs:335-349
        fprintf(stderr, "[DISPATCH] %s x=0x%llx wt=0x%llx y=0x%llx M=%u N=%u K=%u split_k=%u\n", k->name.c_str(),
                (unsigned long long)q.x, (unsigned long long)q.b, (unsigned long long)q.y, q.m, q.n, q.k, q.split_k);
    rc = run_gemm(rt, q);
    if (rc != T0_OK) return rc;
    rt->slot.fetch_add(1);
    if (wait) return check_status_after_sync(rt);
    return T0_OK;
}

int t0_rt_dispatch(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* kernargs, size_t len) {
    return dispatch_impl(rt, k, grid, kernargs, len, true, true);
}

int t0_rt_dispatch_async(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* kernargs, size_t len, size_t* out_slot) {
    if (rt && out_slot) *out_slot = rt->slot.load() % 256;   // gpu_context.rs:296-298
    return dispatch_impl(rt, k, grid, kernargs, len, true, false);
}

int t0_rt_dispatch_bench(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* kernargs, size_t len) {
    return dispatch_impl(rt, k, grid, kernargs, len, false, true);
}

int t0_rt_submit(t0_runtime* rt, const t0_kernel* k, const uint32_t grid[3], const uint8_t* kernargs, size_t len) {
    return dispatch_impl(rt, k, grid, kernargs, len, false, false);
}

int t0_rt_flush(t0_runtime* rt) { return t0_rt_synchronize(rt); }

int t0_gemm_launch_batch(t0_runtime* rt, const t0_gemm_args* args, size_t count) {
    if (!args && count) return fail(T0_ERR_INVALID, "null arguments");
    for (size_t i = 0; i < count; ++i) {
        int rc = t0_gemm_launch(rt, &args[i]);
        if (rc != T0_OK) return rc;
    }
    return T0_OK;
}

int t0_gemm_launch(t0_runtime* rt, const t0_gemm_args* a) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!a) return fail(T0_ERR_INVALID, "null arguments");
    if (a->transpose > T0_NN || a->epilogue > T0_EPI_BIAS_ADD_RELU_STORE_F32 || a->n_tile_epilogue > T0_TILE_MAX_EPILOGUE)
        return fail(T0_ERR_INVALID, "bad enum value in GEMM arguments");
    uint32_t sk = a->split_k > 1 ? a->split_k : 1;
    if (sk & (sk - 1)) return fail(T0_ERR_INVALID, "split_k=%u must be power of 2", sk);
    DeviceGuard guard(rt->device);
    GemmRequest q;
    memset(&q, 0, sizeof q);
    q.x = a->x; q.b = a->b; q.y = a->y; q.bias = a->bias;
    q.m = a->m; q.n = a->n; q.k = a->k;
    q.tile_n = a->tile_n; q.split_k = sk;
    q.nn = a->transpose == T0_NN; q.out_bf16 = a->out_bf16; q.planes = a->planes && sk > 1; q.swap_grid = a->swap_grid;
    q.plane_stride = (uint64_t)a->m * a->n;
    q.pair = a->pair_cta;
    q.epilogue = a->epilogue; q.n_ops = a->n_tile_epilogue;
    memcpy(q.ops, a->tile_epilogue, sizeof q.ops);
    q.scale = a->scale; q.clamp_min = a->clamp_min; q.clamp_max = a->clamp_max;
    return run_gemm(rt, q);
}

int t0_gemm_launch_grouped(t0_runtime* rt, const t0_gemm_args* args, size_t count) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!args && count) return fail(T0_ERR_INVALID, "null arguments");
    if (count == 0) return T0_OK;
    const t0_gemm_args& a0 = args[0];
    // the problems run at the same time: none may write what another reads or writes
    struct Range { uint64_t lo, hi; };
    auto overlaps = [](Range a, Range b) { return a.lo < b.hi && b.lo < a.hi; };
    std::vector<Range> ins, outs;
    bool same = true;
    for (size_t i = 0; i < count; ++i) {
        const t0_gemm_args& a = args[i];
        if (a.m != a0.m || a.n != a0.n || a.k != a0.k || a.tile_n != a0.tile_n || a.split_k != a0.split_k || a.transpose != a0.transpose ||
            a.epilogue != a0.epilogue || a.out_bf16 != a0.out_bf16 || a.planes != a0.planes || a.swap_grid != a0.swap_grid || a.pair_cta != a0.pair_cta ||
            a.n_tile_epilogue != a0.n_tile_epilogue || memcmp(a.tile_epilogue, a0.tile_epilogue, sizeof a.tile_epilogue) != 0 || a.scale != a0.scale ||
            a.clamp_min != a0.clamp_min || a.clamp_max != a0.clamp_max || a.bias != a0.bias)
            same = false;
        const uint64_t out_bytes = (uint64_t)a.m * a.n * (a.out_bf16 ? 2 : 4) * ((a.planes && a.split_k > 1) ? a.split_k : 1);
        outs.push_back({a.y, a.y + out_bytes});
        ins.push_back({a.x, a.x + (uint64_t)a.m * a.k * 2});
        ins.push_back({a.b, a.b + (uint64_t)a.n * a.k * 2});
    }
    for (size_t i = 0; i < count; ++i) {
        for (size_t j = 0; j < count; ++j) {
            if (i == j) continue;
            if (overlaps(outs[i], outs[j]) || overlaps(outs[i], ins[2 * j]) || overlaps(outs[i], ins[2 * j + 1]))
                return fail(T0_ERR_INVALID, "grouped launch: the output of problem %zu overlaps an operand or the output of problem %zu (the problems run concurrently)", i, j);
        }
    }
    // one launch where the problems share a shape whose configuration is the one-launch split-K; otherwise back to back
    DeviceGuard guard(rt->device);
    uint32_t tile_n = a0.tile_n, split = a0.split_k > 1 ? a0.split_k : 1;
    int pair = a0.pair_cta;
    if (a0.tile_n == 0 && a0.pair_cta == 0 && split == 1 && a0.k >= 64) {
        t0_gemm_config c;
        if (t0_cached_auto_select(a0.m, a0.k, a0.n, &c) == T0_OK) {
            tile_n = c.tile_n; split = c.split_k > 1 ? c.split_k : 1; pair = c.wgp_mode ? 1 : 2;
        }
    }
    static const bool no_cluster = getenv("T0_NO_CLUSTER_SPLITK") != nullptr;
    GemmLaunch g;
    memset(&g, 0, sizeof g);
    g.m = a0.m; g.n = a0.n; g.k = a0.k; g.tile_n = tile_n; g.split_k = split;
    g.nn = a0.transpose == T0_NN; g.out_bf16 = a0.out_bf16 != 0; g.swap_grid = a0.swap_grid != 0;
    g.epilogue = a0.epilogue; g.n_ops = a0.n_tile_epilogue;
    memcpy(g.ops, a0.tile_epilogue, sizeof g.ops);
    g.scale = a0.scale; g.clamp_min = a0.clamp_min; g.clamp_max = a0.clamp_max;
    g.bias = (const float*)a0.bias;
    g.status = rt->d_status; g.probe = rt->d_probe; g.n_sms = (uint32_t)rt->sm_count;
    g.wait_limit_ns = rt->wait_limit_ns.load(std::memory_order_relaxed);
    g.x = (const void*)a0.x; g.b = (const void*)a0.b; g.y = (void*)a0.y;
    const bool needs_bias = g.n_ops ? std::find(g.ops, g.ops + g.n_ops, (uint8_t)T0_TEPI_BIAS_ADD) != g.ops + g.n_ops : g.epilogue != T0_EPI_STORE_F32;
    const bool basics = same && count > 1 && !a0.planes && pair != 1 && a0.k >= 64 && a0.k % 8 == 0 && !g.nn && (!needs_bias || a0.bias);
    // Where the caller fixed neither tile nor split, the split is chosen for the GROUP: a single skinny problem needs split-K to
    // fill the GPU, several of them may not, and every split costs an exchange between the CTAs of a tile.  The smallest split
    // (none, 2, 4, 8) with which the tiles of min(count, 32) problems give every SM at least two work items is taken.
    bool plain = false;                                    // no split-K: the single-CTA kernel, grouped
    if (basics && a0.tile_n == 0 && a0.pair_cta == 0 && (a0.split_k <= 1) && split > 1) {
        const uint32_t bn = a0.n <= 64 ? 64u : 128u;
        const uint64_t tiles = (uint64_t)ceil_div(a0.m, 128) * ceil_div(a0.n, bn) * std::min<size_t>(count, kMaxGroupedGemms);
        uint32_t s = 1;
        while (s < split && tiles * s < 2ull * (uint64_t)rt->sm_count) s *= 2;
        while (s > 1 && (a0.k % s || (a0.k / s) % 8)) s /= 2;
        g.tile_n = bn; g.split_k = split = s;
        plain = s == 1;
    } else if (basics && split == 1 && pair != 1 && (snap_tile_n(tile_n) == 64 || snap_tile_n(tile_n) == 128)) {
        plain = true;                                      // the caller (or the model) asked for no split and a tile this kernel has
    }
    const bool grouped = basics && (plain || (!no_cluster && split > 1 && gemm_splitk_cluster_supported(g)));
    if (!grouped) return t0_gemm_launch_batch(rt, args, count);
    std::vector<GemmLaunch> gs;
    for (size_t i = 0; i < count; i += kMaxGroupedGemms) {
        const size_t n = std::min<size_t>(kMaxGroupedGemms, count - i);
        gs.assign(n, g);
        for (size_t j = 0; j < n; ++j) {
            const t0_gemm_args& a = args[i + j];
            if (!a.x || !a.b || !a.y) return fail(T0_ERR_INVALID, "null device pointer in GEMM arguments");
            if ((a.x & 15) || (a.b & 15)) return t0_gemm_launch_batch(rt, args + i, count - i);     // the staged path takes these one by one
            gs[j].x = (const void*)a.x; gs[j].b = (const void*)a.b; gs[j].y = (void*)a.y;
        }
        rc = plain ? launch_gemm_sm100_grouped(gs.data(), (uint32_t)n, rt->stream) : launch_gemm_sm100_splitk_grouped(gs.data(), (uint32_t)n, rt->stream);
        if (rc != T0_OK) return rc;
        rt->launches.fetch_add(1);
    }
    return T0_OK;
}

int t0_gemm_launch_gather(t0_runtime* rt, const t0_gemm_args* a, const uint64_t* peer_y, uint32_t n_peers) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!a || (n_peers && !peer_y)) return fail(T0_ERR_INVALID, "null arguments");
    if (n_peers > kMaxPeerY) return fail(T0_ERR_INVALID, "at most %u further destinations (got %u)", kMaxPeerY, n_peers);
    if (a->transpose > T0_NN || a->epilogue > T0_EPI_BIAS_ADD_RELU_STORE_F32 || a->n_tile_epilogue > T0_TILE_MAX_EPILOGUE)
        return fail(T0_ERR_INVALID, "bad enum value in GEMM arguments");
    if (a->split_k > 1 || a->planes || a->out_bf16) return fail(T0_ERR_UNSUPPORTED, "a gathered output takes a plain f32 product: no split-K, no bf16 output");
    DeviceGuard guard(rt->device);
    GemmRequest q;
    memset(&q, 0, sizeof q);
    q.x = a->x; q.b = a->b; q.y = a->y; q.bias = a->bias;
    q.m = a->m; q.n = a->n; q.k = a->k;
    q.tile_n = a->tile_n ? a->tile_n : 256; q.split_k = 1;      // a fixed tile: the cost model may not pick split-K here
    q.nn = a->transpose == T0_NN; q.swap_grid = a->swap_grid;
    q.plane_stride = (uint64_t)a->m * a->n;
    q.pair = a->pair_cta;
    q.epilogue = a->epilogue; q.n_ops = a->n_tile_epilogue;
    memcpy(q.ops, a->tile_epilogue, sizeof q.ops);
    q.scale = a->scale; q.clamp_min = a->clamp_min; q.clamp_max = a->clamp_max;
    q.n_peer_y = n_peers;
    for (uint32_t i = 0; i < n_peers; ++i) q.peer_y[i] = peer_y[i];
    return run_gemm(rt, q);
}

int t0_buf_ipc_export(const t0_buffer* buf, uint8_t handle[64]) {
    if (!buf || !handle) return fail(T0_ERR_INVALID, "null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is 64 bytes");
    cudaIpcMemHandle_t h;
    DeviceGuard guard(buf->rt->device);
    cudaError_t e = cudaIpcGetMemHandle(&h, buf->dptr);
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    memcpy(handle, &h, 64);
    return T0_OK;
}

int t0_rt_ipc_open(t0_runtime* rt, const uint8_t handle[64], uint64_t* device_ptr) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!handle || !device_ptr) return fail(T0_ERR_INVALID, "null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    DeviceGuard guard(rt->device);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    *device_ptr = (uint64_t)(uintptr_t)p;
    return T0_OK;
}

int t0_rt_ipc_close(t0_runtime* rt, uint64_t device_ptr) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!device_ptr) return T0_OK;
    DeviceGuard guard(rt->device);
    cudaError_t e = cudaStreamSynchronize(rt->stream);
    if (e == cudaSuccess) e = cudaIpcCloseMemHandle((void*)(uintptr_t)device_ptr);
    if (e != cudaSuccess) return fail(T0_ERR_CUDA, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
    return T0_OK;
}

// ------------------------------------------------------------------ seeded inputs

int t0_fill_uniform_bf16(t0_runtime* rt, uint64_t dst, uint64_t n, uint64_t seed, uint64_t first_index) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    DeviceGuard guard(rt->device);
    rc = launch_fill_uniform_bf16((void*)dst, n, seed, first_index, rt->stream);
    if (rc == T0_OK) rt->launches.fetch_add(1);
    return rc;
}

int t0_fill_u32(t0_runtime* rt, uint64_t dst, uint64_t n, uint64_t seed, uint64_t first_index) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    DeviceGuard guard(rt->device);
    rc = launch_fill_u32((void*)dst, n, seed, first_index, rt->stream);
    if (rc == T0_OK) rt->launches.fetch_add(1);
    return rc;
}

int t0_fill_range_bf16(t0_runtime* rt, uint64_t dst, uint64_t n, uint64_t seed, uint64_t first_index, float lo, float hi) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    DeviceGuard guard(rt->device);
    rc = launch_fill_range_bf16((void*)dst, n, seed, first_index, lo, hi, rt->stream);
    if (rc == T0_OK) rt->launches.fetch_add(1);
    return rc;
}

}  // extern "C"

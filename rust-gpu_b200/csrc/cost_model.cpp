// Config selection for the B200 GEMM: the analytic search behind auto_select
// (reference: src/t0/cost_model.rs:197-534,660-668 — an exhaustive tile search scored by a
// roofline/occupancy model), the legacy hand table (src/t0/gemm_gen.rs:351-404), TileIR's static
// selector (src/t0/tile_ir.rs:740-870) and the process-level memo (src/t0/prefill_spec_cache.rs).
//
// The search space is re-derived for B200: a CTA owns 128 output rows (one UMMA M=128 instruction
// shape, accumulator in tensor memory) or a CTA pair owns 256 x 256 (`wgp_mode`); tile_n is
// 32/64/128/256 columns, tile_k is one 128-byte swizzle atom (64 bf16), split-K is 1..8.  The score
// is predicted time = max(tensor time with wave quantisation over the SMs, HBM time on the
// algorithmic bytes) + launch (+ the split-K reduction pass).
#include "common.h"

namespace t0 {
uint32_t gemm_smem_bytes(uint32_t tile_n);        // gemm_sm100.cu
uint32_t gemm_pair_smem_bytes(uint32_t pair_n);   // gemm_sm100_pair.cu
}

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <string>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

namespace t0 {

struct Candidate {
    t0_gemm_config cfg;
    double pred_us;
    double pred_tflops;
};

// Measured main-loop cost per 64-deep k-block on B200 (SM cycles, from the in-kernel cycle probe at 2048^3..8192^3):
// the tensor pipe needs tn/2 cycles per UMMA and four UMMAs per k-block, but narrow tiles are bound by the
// shared-memory operand feed (A is re-read for every UMMA) and the single-CTA 128x256 tile by L2->SM latency with
// only four stages in flight.  The CTA pair (256x256 over two SMs) comes closest to the pipe's 512 cycles.
static double kblock_cycles(uint32_t tn, bool pair) {
    if (pair) return 590.0;
    switch (tn) {
        case 256: return 740.0;
        case 128: return 540.0;
        case 64: return 400.0;
        default: return 330.0;
    }
}

static double predict_us(const B200Limits& hw, uint32_t m, uint32_t n, uint32_t k, uint32_t tn, uint32_t sk, bool pair) {
    const double tiles = (double)ceil_div(m, pair ? 256 : 128) * ceil_div(n, tn) * sk;
    const double slots = pair ? hw.n_sms / 2 : hw.n_sms;
    const double rounds = std::ceil(tiles / slots);
    const double kb = std::ceil((double)k / sk / 64.0);
    const double tile_clk = kb * kblock_cycles(tn, pair) + 3000.0;   // + pipeline fill and the exposed part of the epilogue
    const double tensor_us = rounds * tile_clk / (hw.sm_clock_ghz * 1e3);
    // memory: count algorithmic bytes, plus the partial planes a split-K reduction writes and re-reads
    double bytes = 2.0 * m * k + 2.0 * (double)n * k + 4.0 * (double)m * n;
    if (sk > 1) bytes += 4.0 * (double)m * n * sk;
    const double mem_us = bytes / (hw.hbm_gbs * 1e3);
    // a partially filled machine cannot pull full bandwidth: scale by the fraction of SMs busy
    const double fill = std::min(1.0, tiles * (pair ? 2.0 : 1.0) / hw.n_sms);
    // split-K runs a second, serialised kernel: it reads sk planes and writes y
    // (a kernel that follows another in the same stream costs about 3 us of launch gap, measured; hw.launch_us is the
    // cost of the first)
    const double reduce_us = sk > 1 ? 3.0 + (sk + 1.0) * 4.0 * (double)m * n / (hw.hbm_gbs * 1e3) : 0.0;
    return std::max(tensor_us, mem_us / std::max(fill, 0.05)) + hw.launch_us + reduce_us;
}

static std::vector<Candidate> schedule(uint32_t m, uint32_t n, uint32_t k) {
    B200Limits hw;
    std::vector<Candidate> out;
    if (m == 0 || n == 0 || k == 0) return out;
    static const uint32_t tns[] = {256, 128, 64, 32};
    static const uint32_t sks[] = {1, 2, 4, 8};
    for (int pair = 1; pair >= 0; --pair) {
        for (uint32_t tn : tns) {
            if (pair && tn != 256) continue;                 // the pair kernel is worth it with 256-wide tiles only
            if (pair && (m <= 128 || n <= 128)) continue;
            if (tn > 32 && tn / 2 >= n && n > 0) continue;   // a tile more than twice as wide as N wastes the pipe
            for (uint32_t sk : sks) {
                if (sk > 1) {
                    if (k % (sk * 64) != 0) continue;        // same rule as cost_model.rs:500-502 with tile_k = 64
                    if (sk > k / 64) continue;
                }
                for (int swap = 1; swap >= 0; --swap) {
                    Candidate c;
                    c.cfg = b200_default_config(tn, sk, swap != 0);
                    if (pair) { c.cfg.tile_m = 256; c.cfg.wgp_mode = 1; }
                    c.pred_us = predict_us(hw, m, n, k, tn, sk, pair != 0);
                    // prefer N-fastest rasterisation when A (the M side) is the larger operand to keep
                    // resident, M-fastest otherwise; a tie-break only
                    const bool want_swap = m >= n;
                    if ((swap != 0) != want_swap) c.pred_us *= 1.001;
                    c.pred_tflops = 2.0 * m * (double)n * k / (c.pred_us * 1e6);
                    out.push_back(c);
                }
            }
        }
    }
    std::stable_sort(out.begin(), out.end(), [](const Candidate& a, const Candidate& b) { return a.pred_us < b.pred_us; });
    return out;
}

static t0_gemm_config legacy(uint32_t m, uint32_t k, uint32_t n) {
    // gemm_gen.rs:351-404, same branches and the same split-K clamp
    auto clamp_sk = [&](uint32_t tile_k, uint32_t desired) -> uint32_t {
        uint32_t max_sk = k / tile_k;
        uint32_t sk = std::min(desired, max_sk);
        while (sk > 1 && k % (tile_k * sk) != 0) sk /= 2;
        return sk > 1 ? sk : 0;
    };
    auto preset = [](const char* name) { t0_gemm_config c; t0_gemm_config_preset(name, &c); return c; };
    const uint64_t mn = (uint64_t)m * n;
    const bool use_128m = m % 128 == 0 && m >= 128;
    const bool use_64m = m % 64 == 0;
    t0_gemm_config c;
    if (m <= 256 && k >= 512 && n >= 1024 && use_128m) {
        c = preset("tile_128x64_k16"); c.swap_grid = 0; c.wgp_mode = 1; c.split_k = clamp_sk(16, 4);
    } else if (m <= 512 && k >= 512 && n >= 1024 && use_128m) {
        c = preset("tile_128x64_k16"); c.swap_grid = 0; c.wgp_mode = 1; c.split_k = clamp_sk(16, 8);
    } else if (mn <= 512ull * 512ull) {
        c = preset("tile_64x64_k16"); c.swap_grid = 0; c.split_k = clamp_sk(16, 8);
    } else if (mn <= 1024ull * 1024ull && use_128m) {
        c = preset("tile_128x64_k16"); c.swap_grid = 0; c.wgp_mode = 1; c.split_k = clamp_sk(16, 2);
    } else if (use_128m && mn >= 2048ull * 2048ull) {
        c = preset("tile_128x64_k32"); c.wgp_mode = 1; c.split_k = clamp_sk(32, 2);
    } else if (use_128m) {
        c = preset("tile_128x64_k16"); c.wgp_mode = 1; c.split_k = clamp_sk(16, 8);
    } else if (use_64m) {
        c = preset("tile_64x64_k16"); c.wgp_mode = 1; c.split_k = clamp_sk(16, 4);
    } else {
        c = preset("tile_32x64_k16"); c.split_k = clamp_sk(16, 4);
    }
    return c;
}

// prefill_spec_cache.rs:42-48
static std::mutex g_cache_mu;
static std::map<std::tuple<uint32_t, uint32_t, uint32_t>, t0_gemm_config> g_cache;

}  // namespace t0

using namespace t0;

extern "C" {

int t0_auto_schedule_gemm(uint32_t m, uint32_t n, uint32_t k, t0_gemm_config* out, double* pred_tflops, int cap) {
    std::vector<Candidate> c = schedule(m, n, k);
    int w = 0;
    for (; w < (int)c.size() && w < cap; ++w) {
        if (out) out[w] = c[w].cfg;
        if (pred_tflops) pred_tflops[w] = c[w].pred_tflops;
    }
    return w;
}

static t0_tile_config tile_config_of(const t0_gemm_config& g) {
    t0_tile_config c;
    memset(&c, 0, sizeof c);
    c.tile_m = g.tile_m; c.tile_n = g.tile_n; c.tile_k = g.tile_k;
    c.waves_per_wg = g.wg_size / 32;
    c.use_lds = 1; c.wgp_mode = g.wgp_mode; c.swap_grid = g.swap_grid;
    c.split_k = g.split_k > 1 ? g.split_k : 1;
    c.lds_pad = 0;
    return c;
}

int t0_auto_schedule_tile_costs(uint32_t m, uint32_t n, uint32_t k, t0_tile_cost* out, int cap) {
    std::vector<Candidate> cands = schedule(m, n, k);
    B200Limits hw;
    int w = 0;
    for (; w < (int)cands.size() && w < cap; ++w) {
        if (!out) continue;
        const t0_gemm_config& g = cands[w].cfg;
        t0_tile_cost& tc = out[w];
        memset(&tc, 0, sizeof tc);
        tc.config = tile_config_of(g);
        const bool pair = g.wgp_mode && g.tile_m == 256;
        const uint32_t sk = tc.config.split_k;
        tc.vgprs = pair ? 101 : 104;                              // registers per thread of the kernel instances (ptxas)
        tc.sgprs = 0;
        tc.lds_bytes = pair ? gemm_pair_smem_bytes(g.tile_n) : gemm_smem_bytes(g.tile_n);
        tc.occupancy = 1;                                         // one persistent CTA per SM
        tc.n_wgs = ceil_div(m, g.tile_m) * ceil_div(n, g.tile_n) * sk;
        tc.feasible = 1;
        tc.score = cands[w].pred_tflops;
        const double tiles = (double)tc.n_wgs, slots = pair ? hw.n_sms / 2 : hw.n_sms;
        const char* why = tiles < slots ? "parallelism" : (2.0 * m * (double)n * k / (2.0 * m * k + 2.0 * (double)n * k + 4.0 * (double)m * n) < 200.0 ? "memory" : "tensor");
        snprintf(tc.bottleneck, sizeof tc.bottleneck, "%s", why);
    }
    return w;
}

int t0_tile_config_name(const t0_tile_config* c, char* buf, size_t buf_len) {
    if (!c || !buf || buf_len == 0) return fail(T0_ERR_INVALID, "null argument");
    // cost_model.rs:157-163
    std::string nm = std::to_string(c->tile_m) + "x" + std::to_string(c->tile_n) + "_k" + std::to_string(c->tile_k);
    if (c->split_k > 1) nm += "_sk" + std::to_string(c->split_k);
    if (!c->swap_grid) nm += "_mg";
    if (c->wgp_mode) nm += "_wgp";
    if (c->lds_pad > 0) nm += "_pad" + std::to_string(c->lds_pad);
    if (nm.size() + 1 > buf_len) return fail(T0_ERR_BOUNDS, "name buffer too small");
    memcpy(buf, nm.c_str(), nm.size() + 1);
    return T0_OK;
}

int t0_tile_config_to_gemm_config(const t0_tile_config* c, t0_gemm_config* out) {
    if (!c || !out) return fail(T0_ERR_INVALID, "null argument");
    memset(out, 0, sizeof *out);
    out->tile_m = c->tile_m; out->tile_n = c->tile_n; out->tile_k = c->tile_k;
    out->wg_size = c->waves_per_wg * 32;
    out->use_lds = c->use_lds; out->double_buffer = c->use_lds;          // cost_model.rs:597: always double-buffer with LDS
    out->split_k = c->split_k > 1 ? c->split_k : 0;
    out->lds_pad = c->lds_pad; out->n_col_passes = 1;
    out->swap_grid = c->swap_grid; out->wgp_mode = c->wgp_mode;
    out->transpose = T0_NT; out->epilogue = T0_EPI_STORE_F32;
    return T0_OK;
}

int t0_tile_config_to_tile_gemm(const t0_tile_config* c, t0_tile_gemm* out) {
    if (!c || !out) return fail(T0_ERR_INVALID, "null argument");
    memset(out, 0, sizeof *out);
    out->tile_m = c->tile_m; out->tile_n = c->tile_n; out->tile_k = c->tile_k;
    out->wgp_mode = c->wgp_mode; out->double_buffer = c->use_lds; out->triple_buffer = 0;
    out->split_k = c->split_k;
    out->swap_grid = 1;                                                   // cost_model.rs:618
    out->transpose = T0_NT;
    return T0_OK;
}

int t0_tile_config_can_use_tile_ir(const t0_tile_config* c) {
    if (!c) return 0;
    // cost_model.rs:639-647
    const uint32_t tile_ir_waves = c->tile_m / 32;
    const bool pow2 = c->tile_k && (c->tile_k & (c->tile_k - 1)) == 0;
    return pow2 && c->tile_m >= 32 && c->tile_n >= 32 && c->waves_per_wg == tile_ir_waves && c->swap_grid && c->split_k <= 1;
}

int t0_auto_select_legacy(uint32_t m, uint32_t k, uint32_t n, t0_gemm_config* out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    if (k == 0) return fail(T0_ERR_INVALID, "k must be positive");
    *out = legacy(m, k, n);
    return T0_OK;
}

// T0_FORCE_CFG=<preset>[:sk<N>]: one config for every shape (read on every call, so a test can set and clear it).
static int forced_config(t0_gemm_config* out) {
    const char* f = getenv("T0_FORCE_CFG");
    if (!f || !*f) return -1;
    std::string name(f);
    uint32_t sk = 0;
    const size_t colon = name.find(":sk");
    if (colon != std::string::npos) {
        sk = (uint32_t)strtoul(name.c_str() + colon + 3, nullptr, 10);
        name.resize(colon);
    }
    int rc = t0_gemm_config_preset(name.c_str(), out);
    if (rc != T0_OK) return fail(T0_ERR_INVALID, "T0_FORCE_CFG=%s does not name a GemmConfig preset", f);
    if (sk > 1) {
        if (sk & (sk - 1)) return fail(T0_ERR_INVALID, "T0_FORCE_CFG=%s: split_k must be a power of 2", f);
        out->split_k = sk;
    }
    return T0_OK;
}

int t0_auto_select(uint32_t m, uint32_t k, uint32_t n, t0_gemm_config* out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    { const int fr = forced_config(out); if (fr >= 0) return fr; }
    std::vector<Candidate> c = schedule(m, n, k);
    if (!c.empty()) { *out = c[0].cfg; return T0_OK; }
    // cost_model.rs:662-667: fall back to the hand table when the search finds nothing
    return t0_auto_select_legacy(m, k ? k : 1, n, out);
}

int t0_auto_select_backward_data(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0_gemm_config* out) {
    return t0_auto_select(m, n_orig, k_orig, out);   // gemm_gen.rs:510-514
}

int t0_auto_select_backward_weight(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0_gemm_config* out) {
    return t0_auto_select(n_orig, m, k_orig, out);   // gemm_gen.rs:545-549
}

int t0_cached_auto_select(uint32_t m, uint32_t k, uint32_t n, t0_gemm_config* out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    { const int fr = forced_config(out); if (fr >= 0) return fr; }   // a forced config is never cached
    auto key = std::make_tuple(m, k, n);
    {
        std::lock_guard<std::mutex> g(g_cache_mu);
        auto it = g_cache.find(key);
        if (it != g_cache.end()) { *out = it->second; return T0_OK; }
    }
    int rc = t0_auto_select(m, k, n, out);
    if (rc != T0_OK) return rc;
    std::lock_guard<std::mutex> g(g_cache_mu);
    g_cache[key] = *out;
    return T0_OK;
}

int t0_cached_auto_select_backward_data(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0_gemm_config* out) {
    return t0_cached_auto_select(m, n_orig, k_orig, out);   // prefill_spec_cache.rs:79-83
}

int t0_cached_auto_select_backward_weight(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0_gemm_config* out) {
    // prefill_spec_cache.rs:88-113: separate key namespace (m + 0x8000_0000)
    if (!out) return fail(T0_ERR_INVALID, "null output");
    auto key = std::make_tuple(m + 0x80000000u, n_orig, k_orig);
    {
        std::lock_guard<std::mutex> g(g_cache_mu);
        auto it = g_cache.find(key);
        if (it != g_cache.end()) { *out = it->second; return T0_OK; }
    }
    int rc = t0_auto_select_backward_weight(m, n_orig, k_orig, out);
    if (rc != T0_OK) return rc;
    std::lock_guard<std::mutex> g(g_cache_mu);
    g_cache[key] = *out;
    return T0_OK;
}

int t0_prewarm_cache(const uint32_t* mkn, size_t n_triples) {
    if (!mkn && n_triples) return fail(T0_ERR_INVALID, "null dims");
    t0_gemm_config c;
    for (size_t i = 0; i < n_triples; ++i) {
        int rc = t0_cached_auto_select(mkn[3 * i], mkn[3 * i + 1], mkn[3 * i + 2], &c);
        if (rc != T0_OK) return rc;
    }
    return T0_OK;
}

void t0_clear_cache(void) { std::lock_guard<std::mutex> g(g_cache_mu); g_cache.clear(); }
size_t t0_cache_size(void) { std::lock_guard<std::mutex> g(g_cache_mu); return g_cache.size(); }

int t0_tile_auto_select(uint32_t m, uint32_t k, uint32_t n, int transpose, t0_tile_gemm* out) {
    // tile_ir.rs:740-870: the static size-class table; auto split-K stays disabled (:852-867).
    // The 64 KiB LDS guard (:812-816) is an RDNA limit and has no counterpart here.
    if (!out) return fail(T0_ERR_INVALID, "null output");
    const uint32_t min_dim = std::min(m, n), max_dim = std::max(m, n);
    const bool k32 = k >= 32 && k % 32 == 0, k64 = k >= 64 && k % 64 == 0;
    const char* name;
    if (min_dim >= 128 && max_dim >= 4096) name = k64 ? "tile_128x128_k64" : k32 ? "tile_128x128_k32" : "tile_128x128_k16";
    else if (min_dim >= 64 && max_dim >= 2048) name = (m >= 256 && k32) ? "tile_256x64_k32_wgp" : k32 ? "tile_64x64_k32" : "tile_64x64_k16";
    else if (min_dim >= 64) name = k32 ? "tile_64x64_k32" : "tile_64x64_k16";
    else if (n >= 256 && k32) name = m >= 128 ? "tile_128x256_k32" : "tile_64x256_k32";
    else if (m >= 256 && n >= 128 && k32) name = "tile_256x128_k32";
    else if (n >= 128 && k32) name = "tile_64x64_k32";
    else if (m >= 128 && n < 32) name = "tile_128x32_k16";
    else if (m < 32 && n >= 128) name = "tile_32x128_k16";
    else if (m < 32 && n < 32) name = "tile_32x32_k16";
    else if (k32) name = "tile_64x64_k32";
    else name = "tile_32x64_k16";
    int rc = t0_tile_gemm_preset(name, out);
    if (rc != T0_OK) return rc;
    out->transpose = transpose == T0_NN ? T0_NN : T0_NT;
    return T0_OK;
}

}  // extern "C"

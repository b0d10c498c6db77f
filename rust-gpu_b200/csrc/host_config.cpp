// Host-side mirror of the reference's GEMM selection records and dispatch helpers:
// GemmConfig (src/t0/gemm_gen.rs:55-236), compute_grid* (:308-329,430-437),
// build_kernargs* (:442-484,523-564), TileGemm (src/t0/tile_ir.rs:109-152,607-727),
// its kernarg/grid helpers (:4570-4665) and bf16 converters (:4677-4683).
// Pure C++: nothing here touches the GPU.
#include "common.h"

#include <algorithm>
#include <vector>

namespace t0 {

static thread_local std::string g_last_error;

void set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
}

int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

uint32_t snap_tile_n(uint32_t requested) {
    if (requested >= 256) return 256;
    if (requested >= 128) return 128;
    if (requested >= 64) return 64;
    return 32;
}

// ---------------------------------------------------------------- GemmConfig

static t0_gemm_config mk(uint32_t tm, uint32_t tn, uint32_t tk, uint32_t wg, bool lds, bool db, uint32_t passes) {
    t0_gemm_config c;
    memset(&c, 0, sizeof c);
    c.tile_m = tm; c.tile_n = tn; c.tile_k = tk; c.wg_size = wg;
    c.use_lds = lds; c.double_buffer = db;
    c.split_k = 0; c.lds_pad = 0; c.n_col_passes = passes;
    c.swap_grid = 1; c.wgp_mode = 1; c.transpose = T0_NT; c.epilogue = T0_EPI_STORE_F32;
    return c;
}

struct Preset { const char* name; t0_gemm_config cfg; };

// gemm_gen.rs:86-145 — the fourteen constructors, as data.
static const std::vector<Preset>& presets() {
    static const std::vector<Preset> p = {
        {"tile_16x64_k16",     mk(16, 64, 16, 32, true, true, 1)},
        {"tile_32x64_direct",  mk(32, 64, 16, 64, false, false, 1)},
        {"tile_32x64_k16",     mk(32, 64, 16, 64, true, true, 1)},
        {"tile_32x64_k32",     mk(32, 64, 32, 64, true, true, 1)},
        {"tile_32x128_k16",    mk(32, 128, 16, 64, true, true, 1)},
        {"tile_64x64_k16",     mk(64, 64, 16, 64, true, true, 1)},
        {"tile_64x64_k32",     mk(64, 64, 32, 64, true, true, 1)},
        {"tile_128x64_k16",    mk(128, 64, 16, 128, true, true, 1)},
        {"tile_64x128_k16",    mk(64, 128, 16, 64, true, true, 1)},
        {"tile_128x64_k32",    mk(128, 64, 32, 128, true, true, 1)},
        {"tile_128x128_k16",   mk(128, 128, 16, 128, true, true, 1)},
        {"tile_64x64_k64",     mk(64, 64, 64, 64, true, true, 1)},
        {"tile_128x128_2pass", mk(128, 64, 16, 128, true, true, 2)},
        {"tile_64x128_2pass",  mk(64, 64, 16, 64, true, true, 2)},
        // B200-native shapes the selector emits (no counterpart constructor in the reference)
        {"b200_128x32_k64",    mk(128, 32, 64, 192, true, true, 1)},
        {"b200_128x64_k64",    mk(128, 64, 64, 192, true, true, 1)},
        {"b200_128x128_k64",   mk(128, 128, 64, 192, true, true, 1)},
        {"b200_128x256_k64",   mk(128, 256, 64, 192, true, true, 1)},
        {"b200_pair_256x256_k64", mk(256, 256, 64, 192, true, true, 1)},
    };
    return p;
}

t0_gemm_config b200_default_config(uint32_t tile_n, uint32_t split_k, bool swap_grid) {
    t0_gemm_config c = mk(128, snap_tile_n(tile_n), 64, 192, true, true, 1);
    c.split_k = split_k > 1 ? split_k : 0;
    c.swap_grid = swap_grid;
    c.wgp_mode = 0;
    return c;
}

std::string gemm_config_name(const t0_gemm_config& c) {
    // gemm_gen.rs:215-235
    std::string s = "t0_gemm_" + std::to_string(c.tile_m) + "x" + std::to_string(c.tile_n) + "_k" + std::to_string(c.tile_k);
    s += c.use_lds ? (c.double_buffer ? "_ldsdb" : "_lds") : "_direct";
    if (c.split_k > 1) s += "_sk" + std::to_string(c.split_k);
    if (c.n_col_passes > 1) s += "_" + std::to_string(c.n_col_passes) + "p";
    if (!c.swap_grid) s += "_mg";
    if (c.wgp_mode) s += "_wgp";
    if (c.transpose == T0_NN) s += "_nn";
    if (c.epilogue == T0_EPI_BIAS_ADD_STORE_F32) s += "_bias";
    else if (c.epilogue == T0_EPI_BIAS_ADD_RELU_STORE_F32) s += "_bias_relu";
    return s;
}

static int copy_out(const std::string& s, char* buf, size_t len) {
    if (!buf || len == 0) return fail(T0_ERR_INVALID, "name buffer is null/empty");
    if (s.size() + 1 > len) return fail(T0_ERR_BOUNDS, "name needs %zu bytes, buffer has %zu", s.size() + 1, len);
    memcpy(buf, s.c_str(), s.size() + 1);
    return T0_OK;
}

static bool config_shape_ok(const t0_gemm_config* c) {
    if (!c) return false;
    if (c->tile_m < 16 || c->tile_m > 256 || c->tile_m % 16) return false;
    if (c->tile_n < 16 || c->tile_n > 256 || c->tile_n % 16) return false;
    if (c->tile_k < 16 || c->tile_k > 256 || c->tile_k % 16) return false;
    if (c->wg_size < 32 || c->wg_size > 1024 || c->wg_size % 32) return false;
    uint32_t sk = c->split_k;
    if (sk > 64 || (sk & (sk - 1))) return false;
    if (c->transpose > T0_NN || c->epilogue > T0_EPI_BIAS_ADD_RELU_STORE_F32) return false;
    return true;
}

// ---------------------------------------------------------------- TileGemm

struct TilePreset { const char* name; uint32_t tm, tn, tk; bool wgp, db; bool swap_grid, acc_swap, persistent; };

// tile_ir.rs:156-604 — the constructors, as data (split_k 1, NT, no epilogue, BF16_F32 in all of them).
static const TilePreset kTilePresets[] = {
    {"tile_128x64_k16", 128, 64, 16, false, true, true, false, false},
    {"tile_64x64_k16", 64, 64, 16, false, true, true, false, false},
    {"tile_64x64_k32", 64, 64, 32, false, true, true, false, false},
    {"tile_64x64_k64", 64, 64, 64, false, true, true, false, false},
    {"tile_32x64_k16", 32, 64, 16, false, true, true, false, false},
    {"tile_128x64_k32", 128, 64, 32, false, true, true, false, false},
    {"tile_64x128_k32", 64, 128, 32, false, true, true, true, false},
    {"tile_64x128_k16", 64, 128, 16, false, true, true, false, false},
    {"tile_128x128_k16", 128, 128, 16, false, true, true, false, false},
    {"tile_128x128_k32", 128, 128, 32, true, false, true, true, false},
    {"tile_128x128_k48", 128, 128, 48, false, true, true, false, false},
    {"tile_128x128_k16_swap", 128, 128, 16, false, true, true, true, false},
    {"tile_128x128_k32_swap", 128, 128, 32, false, true, true, true, false},
    {"tile_256x64_k32_wgp", 256, 64, 32, true, true, true, false, false},
    {"tile_256x64_k64_wgp", 256, 64, 64, true, true, true, false, false},
    {"tile_128x128_k64", 128, 128, 64, false, true, true, true, false},
    {"tile_128x64_k64", 128, 64, 64, false, true, true, false, false},
    {"tile_32x32_k16", 32, 32, 16, false, true, true, false, false},
    {"tile_32x128_k16", 32, 128, 16, false, true, true, false, false},
    {"tile_128x32_k16", 128, 32, 16, false, true, true, false, false},
    {"tile_64x256_k32", 64, 256, 32, false, true, true, false, false},
    {"tile_128x256_k32", 128, 256, 32, false, true, true, false, false},
    {"tile_256x128_k32", 256, 128, 32, false, true, true, false, false},
    {"tile_persistent_decode", 32, 64, 16, false, true, false, false, true},
    {"tile_persistent_128x64_k32", 128, 64, 32, false, true, true, false, true},
    {"tile_persistent_256x128_k32", 256, 128, 32, false, true, true, true, true},
};

static t0_tile_gemm tile_from(const TilePreset& p) {
    t0_tile_gemm s;
    memset(&s, 0, sizeof s);
    s.tile_m = p.tm; s.tile_n = p.tn; s.tile_k = p.tk;
    s.wgp_mode = p.wgp; s.double_buffer = p.db; s.triple_buffer = 0; s.swap_grid = p.swap_grid;
    s.split_k = 1; s.transpose = T0_NT; s.acc_swap = p.acc_swap; s.persistent = p.persistent;
    s.n_epilogue = 0; s.waves_per_wg = 0; s.wmma_format = 0;
    return s;
}

static uint32_t tile_n_waves(const t0_tile_gemm* s) { return s->waves_per_wg ? s->waves_per_wg : s->tile_m / 32; }

static const char* tepi_tag(uint8_t op) {
    switch (op) {
        case T0_TEPI_BIAS_ADD: return "bias";
        case T0_TEPI_SCALE: return "scale";
        case T0_TEPI_RELU: return "relu";
        case T0_TEPI_SILU: return "silu";
        case T0_TEPI_GELU: return "gelu";
        case T0_TEPI_ABS: return "abs";
        case T0_TEPI_NEG: return "neg";
        case T0_TEPI_CLAMP: return "clamp";
        default: return "?";
    }
}

std::string tile_gemm_name(const t0_tile_gemm& s) {
    // tile_ir.rs:677-701
    std::string n = "tile_gemm_" + std::to_string(s.tile_m) + "x" + std::to_string(s.tile_n) + "_k" + std::to_string(s.tile_k);
    if (s.double_buffer) n += "_db";
    if (s.split_k > 1) n += "_sk" + std::to_string(s.split_k);
    if (!s.swap_grid) n += "_mg";
    if (s.wgp_mode) n += "_wgp";
    if (s.transpose == T0_NN) n += "_nn";
    if (s.acc_swap) n += "_swap";
    if (s.persistent) n += "_persistent";
    for (uint32_t i = 0; i < s.n_epilogue && i < T0_TILE_MAX_EPILOGUE; ++i) {
        n += "_";
        n += tepi_tag(s.epilogue[i]);
    }
    return n;
}

static bool tile_has(const t0_tile_gemm* s, uint8_t op) {
    for (uint32_t i = 0; i < s->n_epilogue && i < T0_TILE_MAX_EPILOGUE; ++i)
        if (s->epilogue[i] == op) return true;
    return false;
}

static void put_u32(uint8_t* p, uint32_t v) { for (int i = 0; i < 4; ++i) p[i] = (uint8_t)(v >> (8 * i)); }
static void put_u64(uint8_t* p, uint64_t v) { for (int i = 0; i < 8; ++i) p[i] = (uint8_t)(v >> (8 * i)); }

}  // namespace t0

using namespace t0;

extern "C" {

const char* t0_last_error(void) { return g_last_error.c_str(); }
int t0_version(void) { return 100; }

int t0_gemm_config_preset(const char* preset, t0_gemm_config* out) {
    if (!preset || !out) return fail(T0_ERR_INVALID, "null argument");
    for (const auto& p : presets())
        if (strcmp(p.name, preset) == 0) { *out = p.cfg; return T0_OK; }
    return fail(T0_ERR_INVALID, "unknown GemmConfig preset '%s'", preset);
}

int t0_gemm_config_name(const t0_gemm_config* cfg, char* buf, size_t buf_len) {
    if (!cfg) return fail(T0_ERR_INVALID, "null config");
    return copy_out(gemm_config_name(*cfg), buf, buf_len);
}

uint32_t t0_gemm_config_estimated_vgprs(const t0_gemm_config* c) {
    // gemm_gen.rs:189-201 — the RDNA register estimate; reported for callers that log it.
    if (!c || c->wg_size < 32 || c->tile_m == 0) return 0;
    uint32_t n_waves = c->wg_size / 32;
    uint32_t nrb = (c->tile_m / n_waves) / 16;
    uint32_t nct = c->tile_n / 16;
    uint32_t x_lpt = (c->tile_m * c->tile_k * 2 / c->wg_size) / 16;
    uint32_t wt_lpt = (c->tile_n * c->tile_k * 2 / c->wg_size) / 16;
    return nrb * nct * 8 + nrb * 8 + nct * 8 + x_lpt * 4 + wt_lpt * 4 + 49;
}

int t0_gemm_config_is_feasible(const t0_gemm_config* cfg) { return config_shape_ok(cfg) ? 1 : 0; }

uint32_t t0_gemm_config_lds_total(const t0_gemm_config* cfg) {
    if (!cfg) return 0;
    if (cfg->wgp_mode && cfg->tile_m == 256 && cfg->tile_n == 256) return 6 * (128 * 64 * 2 + 128 * 64 * 2) + 1024;   // per CTA of the pair
    uint32_t bn = snap_tile_n(cfg->tile_n);
    uint32_t stage = 128 * 64 * 2 + bn * 64 * 2;
    uint32_t stages = bn == 256 ? 4 : bn == 128 ? 6 : 8;
    return stages * stage + 1024;
}

static int fill_list(const char* const* names, int n, t0_gemm_config* out, int cap, const uint32_t* sks) {
    for (int i = 0; i < n && i < cap; ++i) {
        t0_gemm_config_preset(names[i], &out[i]);
        if (sks && sks[i] > 1) out[i].split_k = sks[i];
    }
    return n;
}

int t0_sweep_configs(t0_gemm_config* out, int cap) {
    // gemm_gen.rs:239-251
    static const char* names[] = {"tile_16x64_k16", "tile_32x64_k16", "tile_32x64_k32", "tile_32x128_k16", "tile_64x64_k16",
                                  "tile_64x64_k32", "tile_128x64_k16", "tile_64x128_k16", "tile_128x64_k32"};
    return fill_list(names, 9, out, out ? cap : 0, nullptr);
}

int t0_standard_configs(t0_gemm_config* out, int cap) {
    // gemm_gen.rs:407-427
    static const char* names[] = {"tile_16x64_k16", "tile_32x64_k16", "tile_32x64_k32", "tile_32x128_k16", "tile_64x64_k16",
                                  "tile_64x64_k32", "tile_128x64_k16", "tile_128x64_k32",
                                  "tile_32x64_k32", "tile_16x64_k16", "tile_64x64_k32", "tile_64x64_k16", "tile_64x64_k32",
                                  "tile_64x64_k16", "tile_128x64_k16", "tile_128x64_k32"};
    static const uint32_t sks[] = {0, 0, 0, 0, 0, 0, 0, 0, 2, 4, 2, 4, 4, 8, 2, 2};
    return fill_list(names, 16, out, out ? cap : 0, sks);
}

// ---------------------------------------------------------------- grids

int t0_compute_grid(const t0_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t* gx, uint32_t* gy) {
    if (!cfg || !gx || !gy) return fail(T0_ERR_INVALID, "null argument");
    if (cfg->tile_m == 0 || cfg->tile_n == 0) return fail(T0_ERR_INVALID, "zero tile dimension");
    uint32_t tiles_m = ceil_div(m, cfg->tile_m), tiles_n = ceil_div(n, cfg->tile_n);
    if (cfg->swap_grid) { *gx = tiles_n * cfg->wg_size; *gy = tiles_m; }
    else                { *gx = tiles_m * cfg->wg_size; *gy = tiles_n; }
    return T0_OK;
}

int t0_compute_grid_split_k(const t0_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t split_k, uint32_t* gx, uint32_t* gy) {
    if (!cfg || !gx || !gy) return fail(T0_ERR_INVALID, "null argument");
    // gemm_gen.rs:320-321: assert!(split_k > 0 && split_k.is_power_of_two())
    if (split_k == 0 || (split_k & (split_k - 1))) return fail(T0_ERR_INVALID, "split_k=%u must be power of 2", split_k);
    if (cfg->tile_m == 0 || cfg->tile_n == 0) return fail(T0_ERR_INVALID, "zero tile dimension");
    uint32_t tiles_m = ceil_div(m, cfg->tile_m), tiles_n = ceil_div(n, cfg->tile_n);
    if (cfg->swap_grid) { *gx = tiles_n * cfg->wg_size; *gy = tiles_m * split_k; }
    else                { *gx = tiles_m * cfg->wg_size; *gy = tiles_n * split_k; }
    return T0_OK;
}

int t0_compute_grid_auto(const t0_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t* gx, uint32_t* gy) {
    if (!cfg) return fail(T0_ERR_INVALID, "null argument");
    uint32_t sk = split_of(cfg);
    return sk > 1 ? t0_compute_grid_split_k(cfg, m, n, sk, gx, gy) : t0_compute_grid(cfg, m, n, gx, gy);
}

int t0_compute_grid_backward_data(const t0_gemm_config* cfg, uint32_t m, uint32_t k_orig, uint32_t* gx, uint32_t* gy) {
    return t0_compute_grid_auto(cfg, m, k_orig, gx, gy);
}

int t0_compute_grid_backward_weight(const t0_gemm_config* cfg, uint32_t n_orig, uint32_t k_orig, uint32_t* gx, uint32_t* gy) {
    return t0_compute_grid_auto(cfg, n_orig, k_orig, gx, gy);
}

// ---------------------------------------------------------------- kernargs

static void ka40(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m, const t0_gemm_config* cfg, uint8_t* out) {
    uint32_t sk = split_of(cfg);
    uint32_t y_stride = sk > 1 ? m * n * 4u : 0u;   // wraps like the reference's u32 arithmetic
    put_u64(out + 0, x); put_u64(out + 8, wt); put_u64(out + 16, y);
    put_u32(out + 24, k); put_u32(out + 28, n); put_u32(out + 32, 0); put_u32(out + 36, y_stride);
}

int t0_build_kernargs(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                      const t0_gemm_config* cfg, uint8_t out[40]) {
    if (!cfg || !out) return fail(T0_ERR_INVALID, "null argument");
    ka40(x, wt, y, k, n, m, cfg, out);
    return T0_OK;
}

int t0_build_kernargs_with_bias(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                const t0_gemm_config* cfg, uint64_t bias, uint8_t out[48]) {
    if (!cfg || !out) return fail(T0_ERR_INVALID, "null argument");
    ka40(x, wt, y, k, n, m, cfg, out);
    put_u64(out + 40, bias);
    return T0_OK;
}

int t0_build_kernargs_backward_data(uint64_t dy, uint64_t w, uint64_t dx, uint32_t m, uint32_t n_orig, uint32_t k_orig,
                                    const t0_gemm_config* cfg, uint8_t out[40]) {
    return t0_build_kernargs(dy, w, dx, n_orig, k_orig, m, cfg, out);
}

int t0_build_kernargs_backward_weight(uint64_t dy_t, uint64_t x_t, uint64_t dw, uint32_t m, uint32_t n_orig, uint32_t k_orig,
                                      const t0_gemm_config* cfg, uint8_t out[40]) {
    return t0_build_kernargs(dy_t, x_t, dw, m, k_orig, n_orig, cfg, out);
}

// ---------------------------------------------------------------- TileGemm

int t0_tile_gemm_preset(const char* preset, t0_tile_gemm* out) {
    if (!preset || !out) return fail(T0_ERR_INVALID, "null argument");
    for (const auto& p : kTilePresets)
        if (strcmp(p.name, preset) == 0) { *out = tile_from(p); return T0_OK; }
    return fail(T0_ERR_INVALID, "unknown TileGemm preset '%s'", preset);
}

int t0_tile_gemm_name(const t0_tile_gemm* spec, char* buf, size_t buf_len) {
    if (!spec) return fail(T0_ERR_INVALID, "null spec");
    return copy_out(tile_gemm_name(*spec), buf, buf_len);
}

uint32_t t0_tile_gemm_wg_size(const t0_tile_gemm* s) { return s ? tile_n_waves(s) * 32 : 0; }

uint32_t t0_tile_gemm_lds_total(const t0_tile_gemm* s) {
    // tile_ir.rs:629-651,659-664 — the reference's LDS accounting, kept because callers size and compare with it.
    if (!s) return 0;
    uint32_t per_buffer = s->tile_m * s->tile_k * 2 + s->tile_n * s->tile_k * 2;
    uint32_t gemm_lds = s->triple_buffer ? per_buffer * 3 : s->double_buffer ? per_buffer * 2 : per_buffer;
    uint32_t base = gemm_lds;
    if (s->acc_swap) {
        uint32_t n_waves = tile_n_waves(s);
        uint32_t n_row_blocks = n_waves ? (s->tile_m / n_waves) / 16 : 0;
        uint32_t vgprs_per_row_block = (s->tile_n / 16) * 8;
        base += n_row_blocks * vgprs_per_row_block * 32 * 4 * n_waves;
    }
    return s->persistent ? base + 16 : base;
}

static uint32_t sk_shift(uint32_t sk) {
    switch (sk) { case 2: return 1; case 4: return 2; case 8: return 3; case 16: return 4; default: return 0; }
}

int t0_tile_build_kernargs_epilogue(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                    const t0_tile_gemm* spec, uint64_t bias, float scale, float clamp_min, float clamp_max,
                                    uint8_t* out, size_t cap, size_t* out_len) {
    if (!spec || !out || !out_len) return fail(T0_ERR_INVALID, "null argument");
    uint8_t tmp[96];
    size_t len = 0;
    put_u64(tmp + 0, x); put_u64(tmp + 8, wt); put_u64(tmp + 16, y);
    put_u32(tmp + 24, k); put_u32(tmp + 28, n); put_u32(tmp + 32, sk_shift(spec->split_k)); put_u32(tmp + 36, 0);
    put_u32(tmp + 40, m);
    len = 44;
    if (spec->persistent) {
        // tile_ir.rs:4623-4632: counter address, n_tiles_n_shift and tiles_per_wg follow M and the blob is
        // padded to 64 bytes.  build_kernargs_m passes zero for all three (tile_ir.rs:4600), and this
        // library's persistent scheduler needs none of them, so bytes 44..63 are zero.
        memset(tmp + 44, 0, 20);
        len = 64;
    }
    // tile_ir.rs:1015-1026: extra arguments in declaration order
    if (tile_has(spec, T0_TEPI_BIAS_ADD)) { len = (len + 7) & ~(size_t)7; put_u64(tmp + len, bias); len += 8; }
    if (tile_has(spec, T0_TEPI_SCALE)) { uint32_t b; memcpy(&b, &scale, 4); put_u32(tmp + len, b); len += 4; }
    if (tile_has(spec, T0_TEPI_CLAMP)) {
        uint32_t b; memcpy(&b, &clamp_min, 4); put_u32(tmp + len, b); len += 4;
        memcpy(&b, &clamp_max, 4); put_u32(tmp + len, b); len += 4;
    }
    if (len > cap) return fail(T0_ERR_BOUNDS, "kernarg blob needs %zu bytes, buffer has %zu", len, cap);
    memcpy(out, tmp, len);
    *out_len = len;
    return T0_OK;
}

int t0_tile_build_kernargs_m(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                             const t0_tile_gemm* spec, uint8_t* out, size_t cap, size_t* out_len) {
    if (!spec) return fail(T0_ERR_INVALID, "null spec");
    t0_tile_gemm plain = *spec;
    plain.n_epilogue = 0;
    return t0_tile_build_kernargs_epilogue(x, wt, y, k, n, m, &plain, 0, 1.0f, 0.0f, 0.0f, out, cap, out_len);
}

int t0_tile_compute_grid(const t0_tile_gemm* s, uint32_t m, uint32_t n, uint32_t grid[3]) {
    if (!s || !grid) return fail(T0_ERR_INVALID, "null argument");
    if (s->tile_m == 0 || s->tile_n == 0) return fail(T0_ERR_INVALID, "zero tile dimension");
    uint32_t wg = tile_n_waves(s) * 32;
    if (s->persistent) { grid[0] = wg; grid[1] = 1; grid[2] = 1; return T0_OK; }   // tile_ir.rs:4646-4655
    uint32_t n_wgs_n = ceil_div(n, s->tile_n), n_wgs_m = ceil_div(m, s->tile_m);
    uint32_t sk = s->split_k ? s->split_k : 1;
    if (s->swap_grid) { grid[0] = n_wgs_n * wg; grid[1] = n_wgs_m * sk; }
    else              { grid[0] = n_wgs_m * wg; grid[1] = n_wgs_n * sk; }
    grid[2] = 1;
    return T0_OK;
}

uint16_t t0_f32_to_bf16(float v) { uint32_t b; memcpy(&b, &v, 4); return (uint16_t)(b >> 16); }
float t0_bf16_to_f32(uint16_t v) { uint32_t b = (uint32_t)v << 16; float f; memcpy(&f, &b, 4); return f; }


// ------------------------------------------------------------------ warp-layout planners (tile_ir.rs:8365-8545)

int t0_warp_layout_row_dominant(uint32_t n_warps, uint32_t tile_m, uint32_t tile_n, t0_warp_layout* out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    if (n_warps == 0 || n_warps > 8) return fail(T0_ERR_INVALID, "n_warps must be 1-8");
    // small M (decode): fewer warps so that each still has 16 rows
    const uint32_t eff = tile_m < n_warps * 16 ? tile_m / 16 : n_warps;
    if (eff == 0) return fail(T0_ERR_INVALID, "tile_m=%u too small for any warp", tile_m);
    if (tile_m % (eff * 16)) return fail(T0_ERR_INVALID, "tile_m=%u must be divisible by effective_warps*16=%u", tile_m, eff * 16);
    *out = t0_warp_layout{eff, tile_m / eff, tile_n, T0_WARP_ROW_DOMINANT};
    return T0_OK;
}

int t0_warp_layout_col_dominant(uint32_t n_warps, uint32_t tile_m, uint32_t tile_n, t0_warp_layout* out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    if (n_warps == 0 || n_warps > 8) return fail(T0_ERR_INVALID, "n_warps must be 1-8");
    if (tile_n % (n_warps * 16)) return fail(T0_ERR_INVALID, "tile_n=%u must be divisible by n_warps*16=%u", tile_n, n_warps * 16);
    *out = t0_warp_layout{n_warps, tile_m, tile_n / n_warps, T0_WARP_COL_DOMINANT};
    return T0_OK;
}

int t0_warp_layout_square(uint32_t n_warps, uint32_t tile_m, uint32_t tile_n, t0_warp_layout* out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    if (n_warps != 4 && n_warps != 8) return fail(T0_ERR_INVALID, "square layout requires 4 or 8 warps, got %u", n_warps);
    const uint32_t row_warps = n_warps == 4 ? 2 : 4, col_warps = 2;
    if (tile_m % (row_warps * 16)) return fail(T0_ERR_INVALID, "tile_m=%u must be divisible by %u*16", tile_m, row_warps);
    if (tile_n % (col_warps * 16)) return fail(T0_ERR_INVALID, "tile_n=%u must be divisible by %u*16", tile_n, col_warps);
    *out = t0_warp_layout{n_warps, tile_m / row_warps, tile_n / col_warps, T0_WARP_SQUARE};
    return T0_OK;
}

uint32_t t0_warp_layout_wmma_row_blocks(const t0_warp_layout* l) { return l ? l->rows_per_warp / 16 : 0; }
uint32_t t0_warp_layout_wmma_col_tiles(const t0_warp_layout* l) { return l ? l->cols_per_warp / 16 : 0; }
uint32_t t0_warp_layout_wmma_ops_per_warp(const t0_warp_layout* l) { return t0_warp_layout_wmma_row_blocks(l) * t0_warp_layout_wmma_col_tiles(l); }
uint32_t t0_warp_layout_acc_vgprs_per_warp(const t0_warp_layout* l) { return t0_warp_layout_wmma_ops_per_warp(l) * 8; }
uint32_t t0_warp_layout_wg_size(const t0_warp_layout* l) { return l ? l->n_warps * 32 : 0; }
int t0_warp_layout_is_compatible(const t0_warp_layout* l, uint32_t tile_m, uint32_t tile_n) {
    return l && l->rows_per_warp && l->cols_per_warp && tile_m % l->rows_per_warp == 0 && tile_n % l->cols_per_warp == 0;
}

int t0_plan_flash_attention_warps(uint32_t n_warps, uint32_t m, uint32_t n, uint32_t d, t0_warp_layout* qk, t0_warp_layout* av) {
    if (!qk || !av) return fail(T0_ERR_INVALID, "null output");
    // small M (decode): limit the warps so each gets at least 16 rows
    const uint32_t eff = std::max<uint32_t>(1, std::min(n_warps, std::max<uint32_t>(m, 16) / 16));
    int rc;
    if (m <= 32) rc = t0_warp_layout_row_dominant(eff, std::max(m, eff * 16), n, qk);
    else if (m >= 64 && n <= 128) rc = t0_warp_layout_row_dominant(n_warps, m, n, qk);
    else if (n >= 128) rc = t0_warp_layout_row_dominant(n_warps, m, n, qk);
    else rc = t0_warp_layout_square(n_warps, m, n, qk);
    if (rc != T0_OK) return rc;
    const uint32_t av_warps = qk->n_warps;    // the second product keeps the warp count of the first
    if (qk->orientation == T0_WARP_ROW_DOMINANT) {
        if (d % (av_warps * 16) == 0) return t0_warp_layout_col_dominant(av_warps, std::max(m, av_warps * 16), d, av);
        return t0_warp_layout_square(av_warps, std::max(m, av_warps * 16), std::max<uint32_t>(d, 32), av);
    }
    return t0_warp_layout_row_dominant(av_warps, std::max(m, av_warps * 16), d, av);
}

// Int4WmmaConfig::k16 / k32 (quant_kernels.rs:325-335)
int t0_int4_wmma_config_k16(t0_int4_wmma_config* out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    out->tile_m = 16; out->tile_n = 16; out->tile_k = 16;
    return T0_OK;
}

int t0_int4_wmma_config_k32(t0_int4_wmma_config* out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    out->tile_m = 16; out->tile_n = 16; out->tile_k = 32;
    return T0_OK;
}

int t0_plan_single_dot_warps(uint32_t n_warps, uint32_t tile_m, uint32_t tile_n, t0_warp_layout* out) {
    if (tile_n >= tile_m * 2 && tile_m < tile_n * 2) return t0_warp_layout_col_dominant(n_warps, tile_m, tile_n, out);   // wide
    return t0_warp_layout_row_dominant(n_warps, tile_m, tile_n, out);                                                      // tall or square-ish
}

}  // extern "C"

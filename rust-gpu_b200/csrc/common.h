// Internal helpers shared by the host-side translation units of libt0b200.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/t0b200.h"

namespace t0 {

// Thread-local error text behind t0_last_error() (the Rust side's `Err(String)`).
void set_error(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

inline uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
inline uint32_t split_of(const t0_gemm_config* c) { return c->split_k > 1 ? c->split_k : 1; }

// B200 machine constants used by the selector and the launcher.
struct B200Limits {
    uint32_t n_sms = 148;
    uint32_t smem_per_cta = 227 * 1024;
    uint32_t tmem_cols = 512;
    double sm_clock_ghz = 1.6;           // typical clock under a dense tensor load (power management, not the 1.965 max)
    double hbm_gbs = 6500.0;             // measured copy bandwidth of this class of part
    double mma_flops_per_clk = 8192.0;   // dense bf16 per SM per clock
    double smem_bytes_per_clk = 100.0;   // effective operand feed per SM; 128x128 tiles measure ~0.76 of 128x256
    double launch_us = 8.0;              // launch + prologue + drain between dependent kernels, measured
};

// The tile the sm_100a kernel actually runs for a requested (tile_m, tile_n):
// UMMA M is fixed at 128 rows per CTA; tile_n snaps to one of 32/64/128/256.
uint32_t snap_tile_n(uint32_t requested);

std::string gemm_config_name(const t0_gemm_config& c);
std::string tile_gemm_name(const t0_tile_gemm& s);
t0_gemm_config b200_default_config(uint32_t tile_n, uint32_t split_k, bool swap_grid);

}  // namespace t0

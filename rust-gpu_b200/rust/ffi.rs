// Raw bindings to libt0b200, generated from include/t0b200.h by gen_ffi.py: do not edit.
// Never compiled where the library is built (no Rust toolchain there); checked only against the header.
#![allow(non_camel_case_types, non_upper_case_globals, dead_code)]
use std::os::raw::{c_char, c_int, c_long, c_uint, c_void};

pub const T0_TILE_MAX_EPILOGUE: u32 = 8;
pub const T0_OK: u32 = 0;
pub const T0_ERR_INVALID: u32 = 1;
pub const T0_ERR_CUDA: u32 = 2;
pub const T0_ERR_POISONED: u32 = 3;
pub const T0_ERR_TIMEOUT: u32 = 4;
pub const T0_ERR_BOUNDS: u32 = 5;
pub const T0_ERR_UNSUPPORTED: u32 = 6;
pub const T0_ERR_IO: u32 = 7;
pub const T0_NT: u32 = 0;
pub const T0_NN: u32 = 1;
pub const T0_EPI_STORE_F32: u32 = 0;
pub const T0_EPI_BIAS_ADD_STORE_F32: u32 = 1;
pub const T0_EPI_BIAS_ADD_RELU_STORE_F32: u32 = 2;
pub const T0_TEPI_BIAS_ADD: u32 = 0;
pub const T0_TEPI_SCALE: u32 = 1;
pub const T0_TEPI_RELU: u32 = 2;
pub const T0_TEPI_SILU: u32 = 3;
pub const T0_TEPI_GELU: u32 = 4;
pub const T0_TEPI_ABS: u32 = 5;
pub const T0_TEPI_NEG: u32 = 6;
pub const T0_TEPI_CLAMP: u32 = 7;
pub const T0_SCRATCH_OPERAND_A: u32 = 0;
pub const T0_SCRATCH_OPERAND_B: u32 = 1;
pub const T0_SCRATCH_SPLITK_PLANES: u32 = 2;
pub const T0_SCRATCH_W4_WEIGHTS: u32 = 3;
pub const T0_SCRATCH_W4_FUSED: u32 = 4;
pub const T0_SCRATCH_F32_A: u32 = 5;
pub const T0_SCRATCH_F32_B: u32 = 6;
pub const T0_SCRATCH_F32_C: u32 = 7;
pub const T0_WARP_ROW_DOMINANT: u32 = 0;
pub const T0_WARP_COL_DOMINANT: u32 = 1;
pub const T0_WARP_SQUARE: u32 = 2;

#[repr(C)]
pub struct t0_buffer { _private: [u8; 0] }
#[repr(C)]
pub struct t0_kernel { _private: [u8; 0] }
#[repr(C)]
pub struct t0_mg { _private: [u8; 0] }
#[repr(C)]
pub struct t0_runtime { _private: [u8; 0] }
#[repr(C)]
pub struct t0_tuner { _private: [u8; 0] }

#[repr(C)]
#[derive(Clone, Copy)]
pub struct t0_gemm_config {
    pub tile_m: u32,
    pub tile_n: u32,
    pub tile_k: u32,
    pub wg_size: u32,
    pub use_lds: u8,
    pub double_buffer: u8,
    pub _pad0: [u8; 2],
    pub split_k: u32,
    pub lds_pad: u32,
    pub n_col_passes: u32,
    pub swap_grid: u8,
    pub wgp_mode: u8,
    pub transpose: u8,
    pub epilogue: u8,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct t0_tile_gemm {
    pub tile_m: u32,
    pub tile_n: u32,
    pub tile_k: u32,
    pub wgp_mode: u8,
    pub double_buffer: u8,
    pub triple_buffer: u8,
    pub swap_grid: u8,
    pub split_k: u32,
    pub transpose: u8,
    pub acc_swap: u8,
    pub persistent: u8,
    pub n_epilogue: u8,
    pub epilogue: [u8; T0_TILE_MAX_EPILOGUE as usize],
    pub waves_per_wg: u32,
    pub wmma_format: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct t0_gemm_args {
    pub x: u64,
    pub b: u64,
    pub y: u64,
    pub bias: u64,
    pub m: u32,
    pub n: u32,
    pub k: u32,
    pub tile_n: u32,
    pub split_k: u32,
    pub transpose: u8,
    pub epilogue: u8,
    pub out_bf16: u8,
    pub planes: u8,
    pub swap_grid: u8,
    pub pair_cta: u8,
    pub _pad: [u8; 2],
    pub n_tile_epilogue: u8,
    pub tile_epilogue: [u8; T0_TILE_MAX_EPILOGUE as usize],
    pub _pad2: [u8; 3],
    pub scale: f32,
    pub clamp_min: f32,
    pub clamp_max: f32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct t0_tile_config {
    pub tile_m: u32,
    pub tile_n: u32,
    pub tile_k: u32,
    pub waves_per_wg: u32,
    pub use_lds: u8,
    pub wgp_mode: u8,
    pub swap_grid: u8,
    pub _pad: u8,
    pub split_k: u32,
    pub lds_pad: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct t0_tile_cost {
    pub config: t0_tile_config,
    pub vgprs: u32,
    pub sgprs: u32,
    pub lds_bytes: u32,
    pub occupancy: u32,
    pub n_wgs: u32,
    pub feasible: c_int,
    pub score: f64,
    pub bottleneck: [c_char; 24],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct t0_warp_layout {
    pub n_warps: u32,
    pub rows_per_warp: u32,
    pub cols_per_warp: u32,
    pub orientation: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct t0_w4a16_args {
    pub a: u64,
    pub packed: u64,
    pub scales: u64,
    pub zeros: u64,
    pub y: u64,
    pub m: u32,
    pub n: u32,
    pub k: u32,
    pub group: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct t0_int4_wmma_config {
    pub tile_m: u32,
    pub tile_n: u32,
    pub tile_k: u32,
}

extern "C" {
    pub fn t0_last_error() -> *const c_char;
    pub fn t0_version() -> c_int;
    pub fn t0_gemm_config_preset(preset: *const c_char, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_gemm_config_name(cfg: *const t0_gemm_config, buf: *mut c_char, buf_len: usize) -> c_int;
    pub fn t0_gemm_config_estimated_vgprs(cfg: *const t0_gemm_config) -> u32;
    pub fn t0_gemm_config_is_feasible(cfg: *const t0_gemm_config) -> c_int;
    pub fn t0_gemm_config_lds_total(cfg: *const t0_gemm_config) -> u32;
    pub fn t0_sweep_configs(out: *mut t0_gemm_config, cap: c_int) -> c_int;
    pub fn t0_standard_configs(out: *mut t0_gemm_config, cap: c_int) -> c_int;
    pub fn t0_auto_select(m: u32, k: u32, n: u32, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_auto_select_legacy(m: u32, k: u32, n: u32, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_auto_select_backward_data(m: u32, n_orig: u32, k_orig: u32, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_auto_select_backward_weight(m: u32, n_orig: u32, k_orig: u32, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_auto_schedule_gemm(m: u32, n: u32, k: u32, out: *mut t0_gemm_config, pred_tflops: *mut f64, cap: c_int) -> c_int;
    pub fn t0_cached_auto_select(m: u32, k: u32, n: u32, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_cached_auto_select_backward_data(m: u32, n_orig: u32, k_orig: u32, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_cached_auto_select_backward_weight(m: u32, n_orig: u32, k_orig: u32, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_prewarm_cache(mkn_triples: *const u32, n_triples: usize) -> c_int;
    pub fn t0_clear_cache();
    pub fn t0_cache_size() -> usize;
    pub fn t0_compute_grid(cfg: *const t0_gemm_config, m: u32, n: u32, gx: *mut u32, gy: *mut u32) -> c_int;
    pub fn t0_compute_grid_split_k(cfg: *const t0_gemm_config, m: u32, n: u32, split_k: u32, gx: *mut u32, gy: *mut u32) -> c_int;
    pub fn t0_compute_grid_auto(cfg: *const t0_gemm_config, m: u32, n: u32, gx: *mut u32, gy: *mut u32) -> c_int;
    pub fn t0_compute_grid_backward_data(cfg: *const t0_gemm_config, m: u32, k_orig: u32, gx: *mut u32, gy: *mut u32) -> c_int;
    pub fn t0_compute_grid_backward_weight(cfg: *const t0_gemm_config, n_orig: u32, k_orig: u32, gx: *mut u32, gy: *mut u32) -> c_int;
    pub fn t0_build_kernargs(x: u64, wt: u64, y: u64, k: u32, n: u32, m: u32, cfg: *const t0_gemm_config, out: *mut u8) -> c_int;
    pub fn t0_build_kernargs_with_bias(x: u64, wt: u64, y: u64, k: u32, n: u32, m: u32, cfg: *const t0_gemm_config, bias: u64, out: *mut u8) -> c_int;
    pub fn t0_build_kernargs_backward_data(dy: u64, w: u64, dx: u64, m: u32, n_orig: u32, k_orig: u32, cfg: *const t0_gemm_config, out: *mut u8) -> c_int;
    pub fn t0_build_kernargs_backward_weight(dy_t: u64, x_t: u64, dw: u64, m: u32, n_orig: u32, k_orig: u32, cfg: *const t0_gemm_config, out: *mut u8) -> c_int;
    pub fn t0_tile_gemm_preset(preset: *const c_char, out: *mut t0_tile_gemm) -> c_int;
    pub fn t0_tile_gemm_name(spec: *const t0_tile_gemm, buf: *mut c_char, buf_len: usize) -> c_int;
    pub fn t0_tile_gemm_wg_size(spec: *const t0_tile_gemm) -> u32;
    pub fn t0_tile_gemm_lds_total(spec: *const t0_tile_gemm) -> u32;
    pub fn t0_tile_auto_select(m: u32, k: u32, n: u32, transpose: c_int, out: *mut t0_tile_gemm) -> c_int;
    pub fn t0_tile_build_kernargs_m(x: u64, wt: u64, y: u64, k: u32, n: u32, m: u32, spec: *const t0_tile_gemm, out: *mut u8, cap: usize, out_len: *mut usize) -> c_int;
    pub fn t0_tile_build_kernargs_epilogue(x: u64, wt: u64, y: u64, k: u32, n: u32, m: u32, spec: *const t0_tile_gemm, bias: u64, scale: f32, clamp_min: f32, clamp_max: f32, out: *mut u8, cap: usize, out_len: *mut usize) -> c_int;
    pub fn t0_tile_compute_grid(spec: *const t0_tile_gemm, m: u32, n: u32, grid: *mut u32) -> c_int;
    pub fn t0_f32_to_bf16(v: f32) -> u16;
    pub fn t0_bf16_to_f32(v: u16) -> f32;
    pub fn t0_rt_new(device: c_int, out: *mut *mut t0_runtime) -> c_int;
    pub fn t0_rt_free(rt: *mut t0_runtime);
    pub fn t0_rt_is_poisoned(rt: *const t0_runtime) -> c_int;
    pub fn t0_rt_mark_poisoned(rt: *mut t0_runtime);
    pub fn t0_rt_synchronize(rt: *mut t0_runtime) -> c_int;
    pub fn t0_rt_wait_idle(rt: *mut t0_runtime) -> c_int;
    pub fn t0_rt_set_wait_limit_ns(rt: *mut t0_runtime, ns: u64) -> c_int;
    pub fn t0_rt_selftest_drop_one_load(rt: *mut t0_runtime) -> c_int;
    pub fn t0_rt_reserve_scratch(rt: *mut t0_runtime, which: c_int, bytes: usize) -> c_int;
    pub fn t0_rt_w4_fused_scratch_bytes(rt: *const t0_runtime) -> usize;
    pub fn t0_rt_stream(rt: *const t0_runtime) -> *mut c_void;
    pub fn t0_rt_device(rt: *const t0_runtime) -> c_int;
    pub fn t0_rt_sm_count(rt: *const t0_runtime) -> c_int;
    pub fn t0_rt_alloc(rt: *mut t0_runtime, n_bytes: usize, out: *mut *mut t0_buffer) -> c_int;
    pub fn t0_rt_alloc_zero(rt: *mut t0_runtime, n_bytes: usize, out: *mut *mut t0_buffer) -> c_int;
    pub fn t0_rt_alloc_f32(rt: *mut t0_runtime, n_elems: usize, out: *mut *mut t0_buffer) -> c_int;
    pub fn t0_rt_recycle(rt: *mut t0_runtime, buf: *mut t0_buffer);
    pub fn t0_rt_pool_cached_bytes(rt: *const t0_runtime) -> usize;
    pub fn t0_rt_pool_clear(rt: *mut t0_runtime);
    pub fn t0_rt_read_f32(rt: *mut t0_runtime, buf: *const t0_buffer, n: usize, out: *mut f32) -> c_int;
    pub fn t0_rt_write_f32(rt: *mut t0_runtime, buf: *mut t0_buffer, data: *const f32, n: usize) -> c_int;
    pub fn t0_rt_upload_f32(rt: *mut t0_runtime, data: *const f32, n: usize, out: *mut *mut t0_buffer) -> c_int;
    pub fn t0_buf_write(buf: *mut t0_buffer, data: *const c_void, len: usize) -> c_int;
    pub fn t0_buf_read(buf: *const t0_buffer, out: *mut c_void, len: usize) -> c_int;
    pub fn t0_buf_write_bytes(buf: *mut t0_buffer, offset: usize, data: *const c_void, len: usize) -> c_int;
    pub fn t0_buf_read_bytes(buf: *const t0_buffer, offset: usize, out: *mut c_void, len: usize) -> c_int;
    pub fn t0_buf_zero(buf: *mut t0_buffer) -> c_int;
    pub fn t0_buf_gpu_addr(buf: *const t0_buffer) -> u64;
    pub fn t0_buf_size(buf: *const t0_buffer) -> usize;
    pub fn t0_buf_free(buf: *mut t0_buffer);
    pub fn t0_rt_ensure_gemm_kernel(rt: *mut t0_runtime, cfg: *const t0_gemm_config, out: *mut *mut t0_kernel) -> c_int;
    pub fn t0_rt_ensure_tile_kernel(rt: *mut t0_runtime, spec: *const t0_tile_gemm, out: *mut *mut t0_kernel) -> c_int;
    pub fn t0_kernel_kernarg_size(k: *const t0_kernel) -> u32;
    pub fn t0_kernel_name(k: *const t0_kernel) -> *const c_char;
    pub fn t0_rt_kernel_cache_size(rt: *const t0_runtime) -> usize;
    pub fn t0_rt_dispatch(rt: *mut t0_runtime, k: *const t0_kernel, grid: *const u32, kernargs: *const u8, len: usize) -> c_int;
    pub fn t0_rt_dispatch_async(rt: *mut t0_runtime, k: *const t0_kernel, grid: *const u32, kernargs: *const u8, len: usize, out_slot: *mut usize) -> c_int;
    pub fn t0_rt_dispatch_bench(rt: *mut t0_runtime, k: *const t0_kernel, grid: *const u32, kernargs: *const u8, len: usize) -> c_int;
    pub fn t0_rt_submit(rt: *mut t0_runtime, k: *const t0_kernel, grid: *const u32, kernargs: *const u8, len: usize) -> c_int;
    pub fn t0_rt_flush(rt: *mut t0_runtime) -> c_int;
    pub fn t0_rt_launch_count(rt: *const t0_runtime) -> u64;
    pub fn t0_rt_last_kernel_clock(rt: *mut t0_runtime, sm_mhz: *mut f64, kernel_us: *mut f64) -> c_int;
    pub fn t0_rt_timer_start(rt: *mut t0_runtime) -> c_int;
    pub fn t0_rt_timer_stop(rt: *mut t0_runtime, ms: *mut f32) -> c_int;
    pub fn t0_gemm_launch(rt: *mut t0_runtime, args: *const t0_gemm_args) -> c_int;
    pub fn t0_gemm_launch_batch(rt: *mut t0_runtime, args: *const t0_gemm_args, count: usize) -> c_int;
    pub fn t0_gemm_launch_grouped(rt: *mut t0_runtime, args: *const t0_gemm_args, count: usize) -> c_int;
    pub fn t0_gemm_launch_gather(rt: *mut t0_runtime, args: *const t0_gemm_args, peer_y: *const u64, n_peers: u32) -> c_int;
    pub fn t0_buf_ipc_export(buf: *const t0_buffer, handle: *mut u8) -> c_int;
    pub fn t0_rt_ipc_open(rt: *mut t0_runtime, handle: *const u8, device_ptr: *mut u64) -> c_int;
    pub fn t0_rt_ipc_close(rt: *mut t0_runtime, device_ptr: u64) -> c_int;
    pub fn t0_gemm_launch_host_batch(rt: *mut t0_runtime, args: *const t0_gemm_args, count: usize) -> c_int;
    pub fn t0_gemm_launch_host(rt: *mut t0_runtime, args: *const t0_gemm_args) -> c_int;
    pub fn t0_auto_schedule_tile_costs(m: u32, n: u32, k: u32, out: *mut t0_tile_cost, cap: c_int) -> c_int;
    pub fn t0_tile_config_name(c: *const t0_tile_config, buf: *mut c_char, buf_len: usize) -> c_int;
    pub fn t0_tile_config_to_gemm_config(c: *const t0_tile_config, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_tile_config_to_tile_gemm(c: *const t0_tile_config, out: *mut t0_tile_gemm) -> c_int;
    pub fn t0_tile_config_can_use_tile_ir(c: *const t0_tile_config) -> c_int;
    pub fn t0_warp_layout_row_dominant(n_warps: u32, tile_m: u32, tile_n: u32, out: *mut t0_warp_layout) -> c_int;
    pub fn t0_warp_layout_col_dominant(n_warps: u32, tile_m: u32, tile_n: u32, out: *mut t0_warp_layout) -> c_int;
    pub fn t0_warp_layout_square(n_warps: u32, tile_m: u32, tile_n: u32, out: *mut t0_warp_layout) -> c_int;
    pub fn t0_warp_layout_wmma_row_blocks(l: *const t0_warp_layout) -> u32;
    pub fn t0_warp_layout_wmma_col_tiles(l: *const t0_warp_layout) -> u32;
    pub fn t0_warp_layout_wmma_ops_per_warp(l: *const t0_warp_layout) -> u32;
    pub fn t0_warp_layout_acc_vgprs_per_warp(l: *const t0_warp_layout) -> u32;
    pub fn t0_warp_layout_wg_size(l: *const t0_warp_layout) -> u32;
    pub fn t0_warp_layout_is_compatible(l: *const t0_warp_layout, tile_m: u32, tile_n: u32) -> c_int;
    pub fn t0_plan_flash_attention_warps(n_warps: u32, m: u32, n: u32, d: u32, qk: *mut t0_warp_layout, av: *mut t0_warp_layout) -> c_int;
    pub fn t0_plan_single_dot_warps(n_warps: u32, tile_m: u32, tile_n: u32, out: *mut t0_warp_layout) -> c_int;
    pub fn t0_matmul_f32(rt: *mut t0_runtime, x: u64, w: u64, y: u64, m: u32, k: u32, n: u32) -> c_int;
    pub fn t0_matmul_f32_with_wt_bf16(rt: *mut t0_runtime, x: u64, wt_bf16: u64, y: u64, m: u32, k: u32, n: u32) -> c_int;
    pub fn t0_matmul_f32_backward_data(rt: *mut t0_runtime, dy: u64, w: u64, dx: u64, m: u32, k: u32, n: u32) -> c_int;
    pub fn t0_matmul_f32_backward_weight(rt: *mut t0_runtime, x: u64, dy: u64, dw: u64, m: u32, k: u32, n: u32) -> c_int;
    pub fn t0_blas_gemm_f32(rt: *mut t0_runtime, m: u32, n: u32, k: u32, alpha: f32, a: u64, lda: u32, b: u64, ldb: u32, beta: f32, c: u64, ldc: u32) -> c_int;
    pub fn t0_blas_gemv_f32(rt: *mut t0_runtime, m: u32, n: u32, alpha: f32, a: u64, lda: u32, x: u64, incx: u32, beta: f32, y: u64, incy: u32) -> c_int;
    pub fn t0_tuner_new(out: *mut *mut t0_tuner) -> c_int;
    pub fn t0_tuner_with_cache_dir(dir: *const c_char, out: *mut *mut t0_tuner) -> c_int;
    pub fn t0_tuner_free(t: *mut t0_tuner);
    pub fn t0_tuner_configure(t: *mut t0_tuner, max_candidates: usize, n_iters: usize) -> c_int;
    pub fn t0_tuner_max_candidates(t: *const t0_tuner) -> usize;
    pub fn t0_tuner_n_iters(t: *const t0_tuner) -> usize;
    pub fn t0_tuner_cache_len(t: *const t0_tuner) -> usize;
    pub fn t0_tuner_cache_dir(t: *const t0_tuner) -> *const c_char;
    pub fn t0_tuner_tune(t: *mut t0_tuner, rt: *mut t0_runtime, m: u32, n: u32, k: u32, out: *mut t0_gemm_config) -> c_int;
    pub fn t0_tuner_benchmark_tile_ir(t: *mut t0_tuner, rt: *mut t0_runtime, spec: *const t0_tile_gemm, m: u32, n: u32, k: u32, tflops: *mut f64) -> c_int;
    pub fn t0_tuner_result(t: *const t0_tuner, m: u32, n: u32, k: u32, best_tflops: *mut f64, from_cache: *mut c_int, n_measured: *mut c_int) -> c_int;
    pub fn t0_tuner_save_cache(t: *mut t0_tuner, m: u32, n: u32, k: u32, best: *const t0_gemm_config, best_tflops: f64) -> c_int;
    pub fn t0_tuner_load_cache(t: *mut t0_tuner, m: u32, n: u32, k: u32, best: *mut t0_gemm_config, best_tflops: *mut f64) -> c_int;
    pub fn t0_parse_json_number(json: *const c_char, key: *const c_char, out: *mut f64) -> c_int;
    pub fn t0_tuner_invalidate(t: *mut t0_tuner, m: u32, n: u32, k: u32);
    pub fn t0_tuner_clear(t: *mut t0_tuner);
    pub fn t0_tuner_report(t: *const t0_tuner);
    pub fn t0_global_tuner() -> *mut t0_tuner;
    pub fn t0_auto_gemm(rt: *mut t0_runtime, a: *mut t0_buffer, b: *mut t0_buffer, c: *mut t0_buffer, m: u32, n: u32, k: u32, tflops: *mut f64) -> c_int;
    pub fn t0_dequant_int4(rt: *mut t0_runtime, packed: u64, scales: u64, zero_points: u64, out: u64, rows: u32, cols: u32, group_size_log2: u32, out_bf16: c_int) -> c_int;
    pub fn t0_rt_ensure_dequant_kernel(rt: *mut t0_runtime, group_size_log2: u32, out_bf16: c_int, out: *mut *mut t0_kernel) -> c_int;
    pub fn t0_w4_dequant(rt: *mut t0_runtime, packed: u64, scales: u64, zeros: u64, out_bf16: u64, K: u32, N: u32, group: u32) -> c_int;
    pub fn t0_w4a16_gemm(rt: *mut t0_runtime, a: u64, packed: u64, scales: u64, zeros: u64, y: u64, M: u32, N: u32, K: u32, group: u32) -> c_int;
    pub fn t0_w4a16_gemm_batch(rt: *mut t0_runtime, args: *const t0_w4a16_args, count: usize) -> c_int;
    pub fn t0_w4a16_gemm_grouped(rt: *mut t0_runtime, args: *const t0_w4a16_args, count: usize) -> c_int;
    pub fn t0_w4_prepacked_bytes(K: u32, N: u32, group: u32) -> usize;
    pub fn t0_w4_prepack(rt: *mut t0_runtime, packed: u64, scales: u64, zeros: u64, out: u64, K: u32, N: u32, group: u32) -> c_int;
    pub fn t0_w4a16_gemm_prepacked(rt: *mut t0_runtime, a: u64, prepacked: u64, y: u64, M: u32, N: u32, K: u32, group: u32) -> c_int;
    pub fn t0_w4a16_gemm_prepacked_batch(rt: *mut t0_runtime, args: *const t0_w4a16_args, count: usize) -> c_int;
    pub fn t0_w4_tiled_bytes(K: u32, N: u32, group: u32) -> usize;
    pub fn t0_w4_to_tiled(rt: *mut t0_runtime, packed: u64, scales: u64, zeros: u64, out: u64, K: u32, N: u32, group: u32) -> c_int;
    pub fn t0_w4a16_gemm_tiled(rt: *mut t0_runtime, a: u64, tiled: u64, y: u64, M: u32, N: u32, K: u32, group: u32) -> c_int;
    pub fn t0_w4a16_gemm_tiled_grouped(rt: *mut t0_runtime, args: *const t0_w4a16_args, count: usize) -> c_int;
    pub fn t0_w4a16_gemm_static(rt: *mut t0_runtime, a: u64, packed: u64, scales: u64, zeros: u64, y: u64, M: u32, N: u32, K: u32, group: u32) -> c_int;
    pub fn t0_w4a16_gemm_static_scratch_bytes() -> usize;
    pub fn t0_int4_wmma_config_k16(out: *mut t0_int4_wmma_config) -> c_int;
    pub fn t0_int4_wmma_config_k32(out: *mut t0_int4_wmma_config) -> c_int;
    pub fn t0_gptq_parse(raw: *const u8, len: usize, rows: *mut u32, cols: *mut u32, group_size: *mut u32, packed_off: *mut usize, scales_off: *mut usize, zero_points_off: *mut usize) -> c_int;
    pub fn t0_gptq_gpu_buffer_size(rows: u32, cols: u32, group_size: u32) -> usize;
    pub fn t0_gptq_to_b200(packed: *const u8, scales: *const f32, zero_points: *const i32, rows: u32, cols: u32, group_size: u32, packed_out: *mut u32, scales_out: *mut u16, zeros_out: *mut u32) -> c_long;
    pub fn t0_shard_columns(n: u32, n_gpus: u32, rank: u32, first_col: *mut u32, n_cols: *mut u32) -> c_int;
    pub fn t0_mg_new(n_gpus: c_int, out: *mut *mut t0_mg) -> c_int;
    pub fn t0_mg_free(mg: *mut t0_mg);
    pub fn t0_mg_size(mg: *const t0_mg) -> c_int;
    pub fn t0_mg_runtime(mg: *mut t0_mg, rank: c_int) -> *mut t0_runtime;
    pub fn t0_mg_synchronize(mg: *mut t0_mg) -> c_int;
    pub fn t0_mg_gemm_sharded(mg: *mut t0_mg, x: *const u64, b_slice: *const u64, y_slice: *const u64, m: u32, n: u32, k: u32, tile_n: u32, pair_cta: c_int) -> c_int;
    pub fn t0_mg_gemm_sharded_gathered(mg: *mut t0_mg, x: *const u64, b_slice: *const u64, c_gathered: *const u64, m: u32, n: u32, k: u32) -> c_int;
    pub fn t0_mg_gemm_sharded_host(mg: *mut t0_mg, x_host: *const c_void, wt_host: *const c_void, y_host: *mut c_void, m: u32, n: u32, k: u32) -> c_int;
    pub fn t0_mg_all_gather_c(mg: *mut t0_mg, c_gathered: *const u64, m: u32, n: u32) -> c_int;
    pub fn t0_fill_uniform_bf16(rt: *mut t0_runtime, dst: u64, n: u64, seed: u64, first_index: u64) -> c_int;
    pub fn t0_fill_u32(rt: *mut t0_runtime, dst: u64, n: u64, seed: u64, first_index: u64) -> c_int;
    pub fn t0_fill_range_bf16(rt: *mut t0_runtime, dst: u64, n: u64, seed: u64, first_index: u64, lo: f32, hi: f32) -> c_int;
}

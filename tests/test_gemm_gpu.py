"""GPU parity tests for the bf16 GEMM, through the C ABI, against the CPU oracle.

The flows mirror the reference's GPU tests: auto_select/preset -> ensure_kernel -> build_kernargs ->
compute_grid -> dispatch -> read (src/t0/tile_ir.rs:5047-5224, src/t0/test_tile_gemm_suite.rs:179-208,
src/t0/tile_boundary_tests.rs:153-215, examples/test_gemm_correctness.rs, examples/full_matrix_check.rs,
src/t0/precision_vs_torch.rs:80-308).  Tolerances: integer-valued inputs bit-exact; random inputs
relative L2 <= 1e-3 and per-element |err| <= 5e-3*sqrt(K/256).
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SENTINEL = -9999.0   # src/t0/tile_boundary_tests.rs:16


def tol_abs(k):
    return 5e-3 * np.sqrt(max(k, 256) / 256.0)


def assert_gemm_close(got, ref, k):
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    rel = np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref.astype(np.float64)), 1e-30)
    assert err.max() <= tol_abs(k), f"max |err| {err.max():.3e} > {tol_abs(k):.3e}"
    assert rel <= 1e-3, f"relative L2 {rel:.3e} > 1e-3"


def lcg_bf16(oracle, n, seed):
    """The reference suite's inline LCG (src/t0/test_tile_gemm_suite.rs:64-65 uses s*6364136223846793005+1)."""
    out = np.empty(n, np.float32)
    s = np.uint64(seed)
    mul = np.uint64(6364136223846793005)
    with np.errstate(over="ignore"):
        for i in range(n):
            s = s * mul + np.uint64(1)
            out[i] = (float((int(s) >> 33) % 2001) - 1000.0) / 1000.0
    return oracle.f32_to_bf16_trunc(out)


def run_gemm_gen(t0, rt, cfg, a, b, m, n, k, bias=None, y_rows=None):
    """The reference's direct flow (examples/hello_gemm_gen.rs:43-149) with a gemm_gen GemmConfig."""
    kern = rt.ensure_kernel_t0(cfg)
    xa, xb = rt.upload(a), rt.upload(b)
    sk = cfg.split()
    rows = y_rows or m
    y = rt.alloc(rows * n * 4 * sk)
    y.write(np.full(rows * n * sk, SENTINEL, np.float32))
    if bias is not None:
        bb = rt.upload(bias)
        ka = t0.build_kernargs_with_bias(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), k, n, m, cfg, bb.gpu_addr())
    else:
        ka = t0.build_kernargs(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), k, n, m, cfg)
    gx, gy = t0.compute_grid_auto(cfg, m, n)
    rt.dispatch(kern, [gx, gy, 1], ka)
    out = rt.read_f32(y, rows * n * sk).reshape(sk, rows, n) if sk > 1 else rt.read_f32(y, rows * n).reshape(rows, n)
    for buf in (xa, xb, y):
        rt.recycle(buf)
    return out


def run_tile(t0, rt, spec, a, b, m, n, k, pad_rows=0, **epi):
    """The TileIR flow (src/t0/tile_ir.rs:5047-5107) with the 44-byte kernarg blob carrying M."""
    kern = rt.ensure_kernel_t0(spec)
    xa, xb = rt.upload(a), rt.upload(b)
    rows = m + pad_rows
    y = rt.alloc(rows * n * 4)
    y.write(np.full(rows * n, SENTINEL, np.float32))
    bias = epi.get("bias")
    bb = rt.upload(bias) if bias is not None else None
    if spec.n_epilogue:
        ka = t0.tile_build_kernargs_epilogue(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), k, n, m, spec,
                                             bias=bb.gpu_addr() if bb else 0, scale=epi.get("scale", 1.0),
                                             clamp_min=epi.get("clamp_min", 0.0), clamp_max=epi.get("clamp_max", 0.0))
    else:
        ka = t0.tile_build_kernargs_m(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), k, n, m, spec)
    rt.dispatch(kern, t0.tile_compute_grid(spec, m, n), ka)
    out = rt.read_f32(y, rows * n).reshape(rows, n)
    for buf in (xa, xb, y):
        rt.recycle(buf)
    return out


# ----------------------------------------------------------------------------- the 256^3 configuration

def test_config1_256_cubed_through_auto_select(t0, oracle, rt):
    m = n = k = 256
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    cfg = t0.auto_select(m, k, n)
    sk = cfg.split()
    got = run_gemm_gen(t0, rt, cfg, a, b, m, n, k)
    if sk > 1:
        planes, ysum = oracle.gemm_nt_splitk(a, b, m, k, n, sk)
        for s in range(sk):
            assert_gemm_close(got[s], planes[s], k // sk)
        got = got.sum(axis=0, dtype=np.float32)
    assert_gemm_close(got, oracle.gemm_nt(a, b, m, k, n), k)


# ----------------------------------------------------------------------------- golden vectors

def _golden(golden_dir, name, dtype):
    return np.fromfile(os.path.join(golden_dir, "torch_ref", name), dtype=dtype)


@pytest.mark.parametrize("w,ref", [("w_gate.bin", "h_gate_f32ref.bin"), ("w_up.bin", "h_up_f32ref.bin")])
def test_torch_golden_first_gemm(t0, rt, golden_dir, w, ref):
    # src/t0/precision_vs_torch.rs:302-305 accepts 0.05; fp32 accumulation gives ~1e-6 here
    x = _golden(golden_dir, "x.bin", np.uint16)
    wt = _golden(golden_dir, w, np.uint16)
    want = _golden(golden_dir, ref, np.float32).reshape(64, 512)
    got = run_tile(t0, rt, t0.tile_auto_select(64, 256, 512), x, wt, 64, 512, 256)
    assert np.abs(got - want).max() < 1e-5
    assert_gemm_close(got, want, 256)


def test_torch_golden_second_gemm(t0, rt, golden_dir):
    s = _golden(golden_dir, "swiglu_bf16_trunc.bin", np.uint16)
    wd = _golden(golden_dir, "w_down.bin", np.uint16)
    want = _golden(golden_dir, "y_bf16_f32acc.bin", np.float32).reshape(64, 256)
    got = run_tile(t0, rt, t0.tile_auto_select(64, 512, 256), s, wd, 64, 256, 512)
    assert np.abs(got - want).max() < 1e-5


def test_torch_golden_bf16_output(t0, oracle, rt, golden_dir):
    x = _golden(golden_dir, "x.bin", np.uint16)
    wt = _golden(golden_dir, "w_gate.bin", np.uint16)
    want = _golden(golden_dir, "h_gate_bf16acc.bin", np.float32).reshape(64, 512)
    xa, xb = rt.upload(x), rt.upload(wt)
    y = rt.alloc(64 * 512 * 2)
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), 64, 512, 256, out_bf16=True)
    rt.synchronize()
    got = oracle.bf16_to_f32(y.read(64 * 512 * 2, np.uint16)).reshape(64, 512)
    ulp = np.maximum(np.abs(want), 2.0 ** -126) * 2.0 ** -7
    assert np.all(np.abs(got - want) <= ulp)
    assert np.mean(got == want) > 0.99


# ----------------------------------------------------------------------------- bit-exact integer matrices

GEMM_GEN_PRESETS = ["tile_16x64_k16", "tile_32x64_direct", "tile_32x64_k16", "tile_32x64_k32", "tile_32x128_k16",
                    "tile_64x64_k16", "tile_64x64_k32", "tile_128x64_k16", "tile_64x128_k16", "tile_128x64_k32",
                    "tile_128x128_k16", "tile_64x64_k64", "tile_128x128_2pass", "tile_64x128_2pass"]


@pytest.mark.parametrize("preset", GEMM_GEN_PRESETS)
def test_full_matrix_bit_exact_all_presets(t0, oracle, rt, preset):
    # examples/full_matrix_check.rs:96-97,143-157: x = 1 + i%3, wt = 1 + j%2, zero tolerance, K in {1,2,4}*tile_k
    cfg = t0.GemmConfig.preset(preset)
    m, n = 2 * cfg.tile_m, 2 * cfg.tile_n
    for kmul in (1, 2, 4):
        k = kmul * cfg.tile_k
        a = oracle.f32_to_bf16_trunc((1 + np.arange(m * k) % 3).astype(np.float32))
        b = oracle.f32_to_bf16_trunc((1 + np.arange(n * k) % 2).astype(np.float32))
        got = run_gemm_gen(t0, rt, cfg, a, b, m, n, k)
        assert np.array_equal(got, oracle.gemm_nt(a, b, m, k, n)), (preset, k)


@pytest.mark.parametrize("m,k,n", [(128, 256, 64), (128, 64, 64), (64, 64, 64)])
def test_tile_ir_pattern_cases(t0, oracle, rt, m, k, n):
    # src/t0/tile_ir.rs:5056-5059: x = i%17 - 8, wt = i%13 - 6 (exact small integers)
    a = oracle.f32_to_bf16_trunc((np.arange(m * k) % 17 - 8).astype(np.float32))
    b = oracle.f32_to_bf16_trunc((np.arange(n * k) % 13 - 6).astype(np.float32))
    for spec in (t0.TileGemm.tile_128x64_k32(), t0.TileGemm.tile_64x64_k16(), t0.TileGemm.tile_128x64_k16()):
        got = run_tile(t0, rt, spec, a, b, m, n, k)
        assert np.array_equal(got, oracle.gemm_nt(a, b, m, k, n))


def test_all_ones_gives_k(t0, rt):
    # examples/hello_gemm_gen.rs:85-146
    m, n, k = 256, 256, 1024
    ones = np.full(m * k, 0x3F80, np.uint16)
    got = run_gemm_gen(t0, rt, t0.GemmConfig.tile_128x64_k16(), ones, np.full(n * k, 0x3F80, np.uint16), m, n, k)
    assert np.all(got == float(k))


def test_autotuner_smoke_pattern(t0, oracle, rt):
    # src/t0/auto_gemm.rs:223-272: 256^3, a = i%7 - 3, b = j%5 - 2, 72 sampled outputs within 0.05 (exact here)
    S = 256
    a = oracle.f32_to_bf16_trunc((np.arange(S * S) % 7 - 3).astype(np.float32))
    b = oracle.f32_to_bf16_trunc((np.arange(S * S) % 5 - 2).astype(np.float32))
    got = run_gemm_gen(t0, rt, t0.auto_select(S, S, S).copy(split_k=0), a, b, S, S, S)
    ref = oracle.gemm_nt(a, b, S, S, S)
    idx = [i * S + i for i in range(16)] + [i * 331 + 97 for i in range(56)]
    assert np.array_equal(got.ravel()[idx], ref.ravel()[idx])
    assert np.array_equal(got, ref)


# ----------------------------------------------------------------------------- ragged shapes and boundaries

RAGGED = [(64, 64, 64), (128, 256, 64), (33, 100, 50), (129, 65, 17), (1000, 768, 512), (1, 16, 16), (17, 31, 5),
          (255, 129, 257), (16, 4096, 32), (300, 8, 300)]


@pytest.mark.parametrize("m,k,n", RAGGED)
def test_ragged_shapes_with_guard_rows(t0, oracle, rt, m, k, n):
    # src/t0/test_tile_gemm_suite.rs:181-194 (LCG data, padded buffers) and the sentinel rule of
    # src/t0/tile_boundary_tests.rs:130-138: rows >= M must stay untouched
    a = lcg_bf16(oracle, m * k, 42 + m) if m * k <= 40000 else oracle.fill_uniform_bf16(m * k, 42 + m)
    b = lcg_bf16(oracle, n * k, 137 + n) if n * k <= 40000 else oracle.fill_uniform_bf16(n * k, 137 + n)
    ref = oracle.gemm_nt(a, b, m, k, n)
    for spec in (t0.tile_auto_select(m, k, n), t0.TileGemm.tile_128x64_k16(), t0.TileGemm.tile_32x32_k16()):
        got = run_tile(t0, rt, spec, a, b, m, n, k, pad_rows=7)
        assert_gemm_close(got[:m], ref, k)
        assert np.all(got[m:] == SENTINEL), "rows beyond M were written"


@pytest.mark.parametrize("m", [1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 127, 128])
def test_boundary_m_not_above_tile(t0, oracle, rt, m):
    # src/t0/tile_boundary_tests.rs:153-215: M <= tile_m, sentinel rows survive
    k, n = 64, 64
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    got = run_tile(t0, rt, t0.TileGemm.tile_128x64_k16(), a, b, m, n, k, pad_rows=128 - m + 1)
    assert_gemm_close(got[:m], oracle.gemm_nt(a, b, m, k, n), k)
    assert np.all(got[m:] == SENTINEL)


def test_empty_and_degenerate_shapes(t0, oracle, rt):
    buf = rt.alloc(4096)
    buf.write(np.full(1024, SENTINEL, np.float32))
    rt.gemm(buf.gpu_addr(), buf.gpu_addr(), buf.gpu_addr(), 0, 64, 64)      # M = 0: nothing to do
    rt.gemm(buf.gpu_addr(), buf.gpu_addr(), buf.gpu_addr(), 64, 0, 64)      # N = 0
    rt.synchronize()
    assert np.all(buf.read(4096, np.float32) == SENTINEL)
    y = rt.alloc(4096)
    y.write(np.full(1024, SENTINEL, np.float32))
    rt.gemm(buf.gpu_addr(), buf.gpu_addr(), y.gpu_addr(), 8, 16, 0)          # K = 0: an empty sum
    rt.synchronize()
    out = y.read(4096, np.float32)
    assert np.all(out[:128] == 0.0) and np.all(out[128:] == SENTINEL)


# ----------------------------------------------------------------------------- split-K

@pytest.mark.parametrize("sk", [2, 4, 8])
def test_split_k_planes_abi(t0, oracle, rt, sk):
    # gemm_gen.rs:447-448: plane s at Y + s*M*N*4; the host sums planes (examples/test_gemm_correctness.rs:203-207)
    m, n, k = 128, 192, 1024
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    cfg = t0.GemmConfig.tile_128x64_k16().copy(split_k=sk)
    got = run_gemm_gen(t0, rt, cfg, a, b, m, n, k)
    planes, ysum = oracle.gemm_nt_splitk(a, b, m, k, n, sk)
    for s in range(sk):
        assert_gemm_close(got[s], planes[s], k // sk)
    acc = np.zeros((m, n), np.float32)
    for s in range(sk):
        acc = acc + got[s]
    assert_gemm_close(acc, ysum, k)


def test_split_k_reduced_on_device(t0, oracle, rt):
    # the split-K skinny configuration in small: the fp32 sum of per-split fp32 partials, in split order
    m, n, k, sk = 64, 256, 4096, 4
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    xa, xb = rt.upload(a), rt.upload(b)
    y = rt.alloc(m * n * 4)
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, split_k=sk)
    got = rt.read_f32(y, m * n).reshape(m, n)
    _, ysum = oracle.gemm_nt_splitk(a, b, m, k, n, sk)
    assert_gemm_close(got, ysum, k)
    # the TileIR blob has y_split_stride = 0 (tile_ir.rs:4613): split specs reduce on the device too
    spec = t0.TileGemm.tile_64x64_k32().copy(split_k=4)
    got2 = run_tile(t0, rt, spec, a, b, m, n, k)
    assert_gemm_close(got2, ysum, k)


def test_split_k_integer_planes_exact(t0, oracle, rt):
    m, n, k, sk = 128, 128, 512, 4
    a = oracle.f32_to_bf16_trunc((np.arange(m * k) % 5 - 2).astype(np.float32))
    b = oracle.f32_to_bf16_trunc((np.arange(n * k) % 3 - 1).astype(np.float32))
    got = run_gemm_gen(t0, rt, t0.GemmConfig.tile_64x64_k32().copy(split_k=sk), a, b, m, n, k)
    planes, _ = oracle.gemm_nt_splitk(a, b, m, k, n, sk)
    assert np.array_equal(got, planes)


# ----------------------------------------------------------------------------- NN layout

@pytest.mark.parametrize("m,k,n", [(128, 128, 128), (256, 512, 384), (100, 136, 72), (33, 100, 50), (64, 64, 1000)])
def test_nn_layout(t0, oracle, rt, m, k, n):
    # GemmTranspose::NN (gemm_gen.rs:27): b is [K, N] with stride N
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(k * n, 137 + n)
    ref = oracle.gemm_nn(a, b, m, k, n)
    got = run_tile(t0, rt, t0.tile_auto_select(m, k, n, t0.NN), a, b, m, n, k)
    assert_gemm_close(got, ref, k)
    if m % 128 == 0 and n % 64 == 0:
        cfg = t0.GemmConfig.tile_128x64_k16().copy(transpose=t0.NN)
        assert cfg.name().endswith("_nn")
        assert_gemm_close(run_gemm_gen(t0, rt, cfg, a, b, m, n, k), ref, k)


def test_nn_equals_nt_on_transposed_weights(t0, oracle, rt):
    m, k, n = 128, 256, 256
    a = oracle.f32_to_bf16_trunc((np.arange(m * k) % 17 - 8).astype(np.float32))
    wt = oracle.f32_to_bf16_trunc((np.arange(n * k) % 13 - 6).astype(np.float32))
    w = np.ascontiguousarray(wt.reshape(n, k).T)
    nt = run_tile(t0, rt, t0.TileGemm.tile_128x128_k32(), a, wt, m, n, k)
    nn = run_tile(t0, rt, t0.TileGemm.tile_128x128_k32().copy(transpose=t0.NN), a, w, m, n, k)
    assert np.array_equal(nt, nn)


# ----------------------------------------------------------------------------- epilogues

@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_gen_bias_epilogues(t0, oracle, rt, mode):
    # gemm_gen.rs:40-49,1366-1423 with the 48-byte blob (gemm_gen.rs:466-484)
    m, n, k = 128, 192, 256
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    bias = (np.arange(n) % 11 - 5).astype(np.float32) * 0.25
    cfg = t0.GemmConfig.tile_64x64_k16().copy(epilogue=mode)
    kern = rt.ensure_kernel_t0(cfg)
    assert kern.kernarg_size == 48
    got = run_gemm_gen(t0, rt, cfg, a, b, m, n, k, bias=bias)
    want = oracle.epilogue_gemm_gen(oracle.gemm_nt(a, b, m, k, n), bias, mode)
    assert_gemm_close(got, want, k)
    if mode == 2:
        assert got.min() >= 0.0


@pytest.mark.parametrize("ops", [["bias"], ["scale"], ["relu"], ["silu"], ["gelu"], ["abs"], ["neg"], ["clamp"],
                                 ["bias", "scale", "silu", "clamp"], ["gelu", "neg", "abs", "relu"]])
def test_tile_ir_epilogue_chain(t0, oracle, rt, ops):
    # tile_ir.rs:41-62,3406-3533
    m, n, k = 130, 200, 128
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    bias = (np.arange(n) % 7 - 3).astype(np.float32) * 0.5
    spec = t0.TileGemm.tile_128x64_k16().with_epilogue(ops)
    got = run_tile(t0, rt, spec, a, b, m, n, k, bias=bias, scale=0.5, clamp_min=-1.0, clamp_max=2.0)
    want = oracle.epilogue_tile(oracle.gemm_nt(a, b, m, k, n), ops, bias, 0.5, -1.0, 2.0)
    assert np.abs(got - want).max() <= 2e-5 + tol_abs(k) * 1e-2
    if ops in (["relu"], ["abs"], ["neg"], ["clamp"]):
        base = run_tile(t0, rt, t0.TileGemm.tile_128x64_k16(), a, b, m, n, k)
        assert np.array_equal(got, oracle.epilogue_tile(base, ops, bias, 0.5, -1.0, 2.0))   # exact ops stay exact


# ----------------------------------------------------------------------------- runtime behaviour

def test_kernarg_size_assert_and_grid_checks(t0, rt):
    cfg = t0.GemmConfig.tile_128x64_k16()
    kern = rt.ensure_kernel_t0(cfg)
    assert kern.kernarg_size == 40 and kern.name == cfg.name()
    assert rt.ensure_kernel_t0(cfg).name == kern.name
    x = rt.alloc_zero(128 * 64 * 2)
    w = rt.alloc_zero(64 * 64 * 2)
    y = rt.alloc_zero(128 * 64 * 4)
    ka = t0.build_kernargs(x.gpu_addr(), w.gpu_addr(), y.gpu_addr(), 64, 64, 128, cfg)
    with pytest.raises(t0.T0Error) as e:       # gpu_context.rs:319-322
        rt.dispatch(kern, [128, 1, 1], ka + b"\0" * 4)
    assert "kernarg mismatch" in str(e.value)
    with pytest.raises(t0.T0Error):            # grid x must be whole workgroups
        rt.dispatch(kern, [100, 1, 1], ka)
    rt.dispatch(kern, [128, 1, 1], ka)
    assert np.all(rt.read_f32(y, 128 * 64) == 0.0)
    # a weight buffer smaller than N*K is refused before anything is launched
    small = rt.alloc_zero(4096)
    ka2 = t0.build_kernargs(x.gpu_addr(), small.gpu_addr(), y.gpu_addr(), 64, 64, 128, cfg)
    with pytest.raises(t0.T0Error) as e:
        rt.dispatch(kern, [128, 1, 1], ka2)
    assert e.value.code == 5
    assert not rt.is_poisoned()


def test_poisoned_runtime_fails_fast(t0):
    # gpu_context.rs:190-198,311-313; the reference's tests rebuild the runtime afterwards (tile_ir.rs:4987-4998)
    r = t0.GpuRuntime(0)
    cfg = t0.GemmConfig.tile_128x64_k16()
    kern = r.ensure_kernel_t0(cfg)
    x = r.alloc_zero(128 * 64 * 2)
    y = r.alloc_zero(128 * 64 * 4)
    ka = t0.build_kernargs(x.gpu_addr(), x.gpu_addr(), y.gpu_addr(), 64, 64, 128, cfg)
    r.dispatch(kern, [128, 1, 1], ka)
    r.mark_poisoned()
    assert r.is_poisoned()
    with pytest.raises(t0.T0Error) as e:
        r.dispatch(kern, [128, 1, 1], ka)
    assert e.value.code == 3
    r.close()
    r2 = t0.GpuRuntime(0)
    assert not r2.is_poisoned()
    r2.close()


def test_buffer_pool_semantics(t0, rt):
    # gpu_context.rs:31-92,508-530: 4 KiB size classes, zero on reuse, alloc_f32 rounds to 512 B and zeroes
    b = rt.alloc(5000)
    assert b.size == 8192
    addr = b.gpu_addr()
    b.write(np.full(2048, 7.0, np.float32))
    rt.recycle(b)
    assert rt.pool_cached_bytes() >= 8192
    b2 = rt.alloc(8000)
    assert b2.gpu_addr() == addr
    assert np.all(b2.read(8192, np.float32) == 0.0)
    f = rt.alloc_f32(3)
    assert f.size >= 512 and np.all(rt.read_f32(f, 3) == 0.0)
    u = rt.upload_f32(np.arange(10, dtype=np.float32))
    assert rt.read_f32(u, 10).tolist() == list(range(10))
    # bounds-checked partial access (src/kfd/buffer.rs:76,85)
    u.write_bytes(8, np.array([99.0], np.float32))
    assert u.read_bytes(8, 4, np.float32)[0] == 99.0
    with pytest.raises(t0.T0Error):
        u.write_bytes(u.size - 2, np.zeros(1, np.float32))
    with pytest.raises(t0.T0Error):
        u.read_bytes(u.size, 4)
    for x in (b2, f, u):
        rt.recycle(x)


def test_dispatch_async_keeps_queue_order(t0, oracle, rt):
    # dispatch_async = submit only; wait_idle drains (gpu_context.rs:400-410, src/kfd/aql.rs:473)
    m = n = k = 128
    a = oracle.fill_uniform_bf16(m * k, 1)
    b = oracle.fill_uniform_bf16(n * k, 2)
    cfg = t0.GemmConfig.tile_128x64_k16()
    kern = rt.ensure_kernel_t0(cfg)
    xa, xb = rt.upload(a), rt.upload(b)
    ys = [rt.alloc(m * n * 4) for _ in range(4)]
    before = rt.launch_count()
    for y in ys:
        rt.dispatch_async(kern, list(t0.compute_grid_auto(cfg, m, n)) + [1],
                          t0.build_kernargs(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), k, n, m, cfg))
    rt.wait_idle()
    assert rt.launch_count() - before == 4
    ref = oracle.gemm_nt(a, b, m, k, n)
    outs = [rt.read_f32(y, m * n).reshape(m, n) for y in ys]
    for o in outs:
        assert_gemm_close(o, ref, k)
        assert np.array_equal(o, outs[0])      # run-to-run determinism


# ----------------------------------------------------------------------------- full-size properties

def test_square_4096_properties(t0, oracle, rt):
    # 4096^3, size-independent properties on top of the full compares below:
    # (1) integer-valued inputs give exact outputs whose column sums have a closed form,
    # (2) sampled rows of the seeded random case agree with the oracle, (3) bit-identical reruns.
    m = n = k = 4096
    cfg = t0.auto_select(m, k, n)
    a_int = (np.arange(m * k, dtype=np.int64) % 5 - 2).astype(np.float32)
    b_int = ((np.arange(n * k, dtype=np.int64) * 7) % 3 - 1).astype(np.float32)
    xa = rt.upload(oracle.f32_to_bf16_trunc(a_int))
    xb = rt.upload(oracle.f32_to_bf16_trunc(b_int))
    y = rt.alloc(m * n * 4)
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, tile_n=cfg.tile_n, split_k=cfg.split())
    got = rt.read_f32(y, m * n).reshape(m, n)
    colsum = a_int.reshape(m, k).astype(np.float64).sum(axis=0) @ b_int.reshape(n, k).astype(np.float64).T
    assert np.array_equal(got.astype(np.float64).sum(axis=0), colsum)
    rows = [0, 1, 2047, 4095]
    ref = oracle.gemm_nt(oracle.f32_to_bf16_trunc(a_int.reshape(m, k)[rows]), oracle.f32_to_bf16_trunc(b_int), len(rows), k, n)
    assert np.array_equal(got[rows], ref)
    # seeded uniform inputs generated on the device, checked on sampled rows
    rt.fill_uniform_bf16(xa.gpu_addr(), m * k, 42 + m)
    rt.fill_uniform_bf16(xb.gpu_addr(), n * k, 137 + n)
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, tile_n=cfg.tile_n, split_k=cfg.split())
    got = rt.read_f32(y, m * n).reshape(m, n)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    for r in rows:
        a_row = oracle.fill_uniform_bf16(k, 42 + m, r * k)
        assert_gemm_close(got[r:r + 1], oracle.gemm_nt(a_row, b, 1, k, n), k)
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, tile_n=cfg.tile_n, split_k=cfg.split())
    assert np.array_equal(rt.read_f32(y, m * n).reshape(m, n), got)
    for buf in (xa, xb, y):
        buf.free()


@pytest.mark.parametrize("m,n,k,sk", [(128, 4096, 4096, 1), (64, 4096, 16384, 4)])
def test_skinny_configs_full_size(t0, oracle, rt, m, n, k, sk):
    # the skinny configurations at full size (the oracle finishes these in seconds)
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    xa, xb = rt.upload(a), rt.upload(b)
    y = rt.alloc(m * n * 4 * sk)
    if sk > 1:
        # planes ABI, then the device-side reduction
        rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, split_k=sk, planes=True)
        planes = rt.read_f32(y, m * n * sk).reshape(sk, m, n)
        ref_planes, ysum = oracle.gemm_nt_splitk(a, b, m, k, n, sk)
        for s in range(sk):
            assert_gemm_close(planes[s], ref_planes[s], k // sk)
        rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, split_k=sk)
        assert_gemm_close(rt.read_f32(y, m * n).reshape(m, n), ysum, k)
    else:
        cfg = t0.auto_select(m, k, n)
        rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, tile_n=cfg.tile_n, split_k=cfg.split())
        assert_gemm_close(rt.read_f32(y, m * n).reshape(m, n), oracle.gemm_nt(a, b, m, k, n), k)
    for buf in (xa, xb, y):
        buf.free()


@pytest.mark.parametrize("m,n,k,tile_n", [(2304, 2304, 128, 256),    # 81 tiles over 74 pairs: 7 tail tiles cut in halves
                                          (2500, 2400, 200, 256),    # 100 tiles, ragged edges inside tail tiles
                                          (2304, 1152, 192, 128),    # the 256 x 128 instance, 81 tiles
                                          (3072, 2560, 64, 256)])    # 120 tiles: the last wave is too full to be cut
def test_pair_kernel_tail_tiles_full_compare(t0, oracle, rt, m, n, k, tile_n):
    # the CTA-pair kernel cuts the tiles of a thin last wave into two half-width tiles: every element is compared
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    xa, xb = rt.upload(a), rt.upload(b)
    y = rt.alloc(m * n * 4 + 4096)
    y.write(np.full(m * n + 1024, -9999.0, np.float32))
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, tile_n=tile_n, pair_cta=1)
    rt.synchronize()
    got = y.read(m * n * 4, np.float32).reshape(m, n)
    assert_gemm_close(got, oracle.gemm_nt(a, b, m, k, n), k)
    assert np.all(y.read_bytes(m * n * 4, 4096, np.float32) == -9999.0)
    for buf in (xa, xb, y):
        buf.free()


@pytest.mark.parametrize("m,n,k", [(512, 512, 256),        # 4 tiles
                                   (2304, 2304, 128),      # 81 tiles: 7 tail tiles cut in halves
                                   (2500, 2400, 200),      # ragged edges, tail tiles
                                   (3072, 2560, 64)])      # 120 tiles, no tail
def test_pair_kernel_nn_layout_full_compare(t0, oracle, rt, m, n, k):
    # B given as B[K,N]: the CTA-pair kernel reads it through N-major boxes and an MN-major UMMA descriptor
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(k * n, 137 + n)
    xa, xb = rt.upload(a), rt.upload(b)
    y = rt.alloc(m * n * 4 + 4096)
    y.write(np.full(m * n + 1024, -9999.0, np.float32))
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, transpose=t0.NN, pair_cta=1)
    rt.synchronize()
    assert_gemm_close(y.read(m * n * 4, np.float32).reshape(m, n), oracle.gemm_nn(a, b, m, k, n), k)
    assert np.all(y.read_bytes(m * n * 4, 4096, np.float32) == -9999.0)
    for buf in (xa, xb, y):
        buf.free()


# ----------------------------------------------------------------------------- square sweep, every element compared

def assert_bf16_close(oracle, got_bits, ref, k):
    """bf16 output: each element is the f32 accumulator rounded once (nearest even).  The accumulator differs from the
    oracle's within the GEMM tolerance, so an element may land on the neighbouring bf16 value; nearly all are identical."""
    got = oracle.bf16_to_f32(got_bits).reshape(ref.shape)
    want = oracle.bf16_to_f32(oracle.f32_to_bf16_rne(ref.reshape(-1))).reshape(ref.shape)
    ulp = np.maximum(np.abs(want), 2.0 ** -126) * 2.0 ** -7
    assert np.all(np.abs(got - want) <= np.maximum(ulp, tol_abs(k))), "a bf16 output is more than one step from the rounded oracle value"
    assert np.mean(got == want) > 0.97
    assert np.linalg.norm(got.astype(np.float64) - ref) / np.linalg.norm(ref.astype(np.float64)) <= 3e-3   # bf16 rounding alone is 1.1e-3


@pytest.mark.parametrize("size", [2048, 4096])
def test_square_sweep_full_compare(t0, oracle, rt, size):
    # the square sweep, f32 and bf16 output, WT[N,K] and B[K,N]: every element against the oracle
    # (examples/full_matrix_check.rs:118-157 compares whole matrices wherever its CPU check is affordable)
    m = n = k = size
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    wt = oracle.fill_uniform_bf16(n * k, 137 + n)
    ref = oracle.gemm_nt(a, wt, m, k, n)
    xa, xb = rt.upload(a), rt.upload(wt)
    y = rt.alloc(m * n * 4 + 4096)
    for layout in (t0.NT, t0.NN):
        if layout == t0.NN:
            xb.write(np.ascontiguousarray(wt.reshape(n, k).T))       # the same weights as B[K,N]
        y.write_bytes(m * n * 4, np.full(1024, SENTINEL, np.float32))
        rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, transpose=layout)
        rt.synchronize()
        assert_gemm_close(y.read(m * n * 4, np.float32).reshape(m, n), ref, k)
        assert np.all(y.read_bytes(m * n * 4, 4096, np.float32) == SENTINEL)
        y.write_bytes(m * n * 2, np.full(1024, SENTINEL, np.float32))
        rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, transpose=layout, out_bf16=True)
        rt.synchronize()
        assert_bf16_close(oracle, y.read(m * n * 2, np.uint16), ref, k)
        assert np.all(y.read_bytes(m * n * 2, 4096, np.float32) == SENTINEL)
    for buf in (xa, xb, y):
        buf.free()


def test_square_8192_full_compare(t0, oracle, rt):
    # 8192^3: 14 waves of 256 x 256 tiles, both accumulator buffers cycle seven times; inputs generated on the device
    # by the counter-based generator the oracle shares, every element of the f32 result compared
    m = n = k = 8192
    xa, xb, y = rt.alloc(m * k * 2), rt.alloc(n * k * 2), rt.alloc(m * n * 4)
    rt.fill_uniform_bf16(xa.gpu_addr(), m * k, 42 + m)
    rt.fill_uniform_bf16(xb.gpu_addr(), n * k, 137 + n)
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k)
    got = rt.read_f32(y, m * n).reshape(m, n)
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    wt = oracle.fill_uniform_bf16(n * k, 137 + n)
    ref = oracle.gemm_nt(a, wt, m, k, n)
    assert_gemm_close(got, ref, k)
    # bf16 output at the same size: 512 rows spread over every tile row
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, out_bf16=True)
    rt.synchronize()
    rows = np.arange(0, m, 16)
    got16 = y.read(m * n * 2, np.uint16).reshape(m, n)[rows]
    assert_bf16_close(oracle, got16.reshape(-1), ref[rows], k)
    for buf in (xa, xb, y):
        buf.free()


# ----------------------------------------------------------------------------- epilogue store path, tile after tile

@pytest.mark.parametrize("m,n,k,tile_n,pair", [
    (1280, 1280, 64, 32, 2),      # 400 tiles of one 32-column chunk each: every tile of a persistent CTA reuses a staging block
    (1280, 1280, 128, 32, 2),
    (25600, 96, 64, 64, 2),       # N % 64 = 32: the edge tile ends after an odd number of full chunks, 400 tiles
    (1024, 4128, 64, 64, 2),      # 65 x 8 tiles, the last column tile has one full chunk
    (4136, 512, 64, 128, 2),      # M = 4096 + 40: an M-edge tile (three of four warps own no row) follows full tiles
    (4136, 4128, 64, 256, 1),     # the CTA-pair kernel with both edges
    (4136, 4128, 128, 256, 2),    # the single-CTA 256-wide instance
])
def test_tma_store_epilogue_tile_sequences(t0, oracle, rt, m, n, k, tile_n, pair):
    # Short K makes the epilogue the bottleneck, so consecutive tiles' stores are in flight together.  The output leaves
    # through two alternating staging blocks per warp; these shapes make a warp commit an odd number of stores per tile,
    # a single one, or none.  Every element is compared and the guard area behind y must stay untouched.
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    ref = oracle.gemm_nt(a, b, m, k, n)
    xa, xb = rt.upload(a), rt.upload(b)
    y = rt.alloc(m * n * 4 + 4096)
    for _ in range(3):
        y.write(np.full(m * n + 1024, SENTINEL, np.float32))
        rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, tile_n=tile_n, pair_cta=pair)
        rt.synchronize()
        assert_gemm_close(y.read(m * n * 4, np.float32).reshape(m, n), ref, k)
        assert np.all(y.read_bytes(m * n * 4, 4096, np.float32) == SENTINEL)
    for buf in (xa, xb, y):
        buf.free()


# ----------------------------------------------------------------------------- submit / flush, bounded waits

def test_submit_flush_batch(t0, oracle, rt):
    # DispatchQueue::submit x N then flush (src/t0/prefill_dispatch.rs:61-206): fire-and-forget submits, one wait;
    # results equal those of blocking dispatches; a poisoned runtime refuses the submit
    m, n, k = 256, 384, 512
    a = oracle.fill_uniform_bf16(m * k, 11)
    cfg = t0.GemmConfig.tile_128x64_k32()
    kern = rt.ensure_kernel_t0(cfg)
    grid = list(t0.compute_grid_auto(cfg, m, n)) + [1]
    xa = rt.upload(a)
    ws = [rt.upload(oracle.fill_uniform_bf16(n * k, 100 + i)) for i in range(6)]
    ys = [rt.alloc(m * n * 4) for _ in range(6)]
    before = rt.launch_count()
    for w, y in zip(ws, ys):
        rt.submit(kern, grid, t0.build_kernargs(xa.gpu_addr(), w.gpu_addr(), y.gpu_addr(), k, n, m, cfg))
    assert rt.launch_count() - before == 6
    rt.flush()
    y_ref = rt.alloc(m * n * 4)
    for i, (w, y) in enumerate(zip(ws, ys)):
        rt.dispatch(kern, grid, t0.build_kernargs(xa.gpu_addr(), w.gpu_addr(), y_ref.gpu_addr(), k, n, m, cfg))
        got = rt.read_f32(y, m * n)
        assert np.array_equal(got, rt.read_f32(y_ref, m * n))
        assert_gemm_close(got.reshape(m, n), oracle.gemm_nt(a, oracle.fill_uniform_bf16(n * k, 100 + i), m, k, n), k)
    r = t0.GpuRuntime(0)
    kern2 = r.ensure_kernel_t0(cfg)
    x2, y2 = r.alloc_zero(m * k * 2), r.alloc_zero(m * n * 4)
    w2 = r.alloc_zero(n * k * 2)
    ka = t0.build_kernargs(x2.gpu_addr(), w2.gpu_addr(), y2.gpu_addr(), k, n, m, cfg)
    r.submit(kern2, grid, ka)
    r.flush()
    r.mark_poisoned()
    with pytest.raises(t0.T0Error) as e:            # prefill_dispatch.rs: submit checks the poison flag
        r.submit(kern2, grid, ka)
    assert e.value.code == 3
    for buf in (x2, w2, y2):
        buf.free()
    r.close()


@pytest.mark.parametrize("pair", [2, 1])
def test_bounded_wait_reports_timeout_and_poisons(t0, oracle, pair):
    # The reference turns a dispatch that never finishes into Err and poisons the runtime (src/kfd/aql.rs:529-549,
    # src/ignis/gpu_context.rs:352-355).  Here every device-side wait is bounded: with the self-test switch one operand
    # load of the first tile is left out, that tile's wait runs out after the (shortened) limit, the kernel unwinds by
    # itself, releases its tensor memory and leaves a status word.  Nothing faults; the context stays usable.
    m, n, k = 1024, 1024, 512
    a = oracle.fill_uniform_bf16(m * k, 5)
    b = oracle.fill_uniform_bf16(n * k, 6)
    r = t0.GpuRuntime(0)
    xa, xb, y = r.upload(a), r.upload(b), r.alloc_zero(m * n * 4)
    r.set_wait_limit_ns(3_000_000)                  # 3 ms instead of 2 s
    r.selftest_drop_one_load()
    r.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, tile_n=256 if pair == 1 else 128, pair_cta=pair)
    with pytest.raises(t0.T0Error) as e:
        r.synchronize()
    assert e.value.code == 4 and "wait expired" in str(e.value)
    assert r.is_poisoned()
    with pytest.raises(t0.T0Error) as e:            # fail fast from here on (gpu_context.rs:311-313)
        r.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k)
    assert e.value.code == 3
    for buf in (xa, xb, y):
        buf.free()
    r.close()
    # a fresh runtime on the same device works: the kernel released its tensor memory and the context is intact
    r2 = t0.GpuRuntime(0)
    xa, xb, y = r2.upload(a), r2.upload(b), r2.alloc_zero(m * n * 4)
    r2.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, tile_n=256 if pair == 1 else 128, pair_cta=pair)
    assert_gemm_close(r2.read_f32(y, m * n).reshape(m, n), oracle.gemm_nt(a, b, m, k, n), k)
    # the switch is one-shot and the limit is per runtime: the next launch of an armed runtime is normal again
    r2.set_wait_limit_ns(0)
    for buf in (xa, xb, y):
        buf.free()
    r2.close()


# ----------------------------------------------------------------------------- split-K inside one launch (CTA clusters)

@pytest.mark.parametrize("m,n,k,sk,tile_n", [(128, 4096, 4096, 4, 128),      # the skinny configuration
                                              (64, 4096, 16384, 4, 128),      # the split-K skinny configuration
                                              (1000, 4000, 2048, 4, 128),     # 8 x 32 tiles for ~36 clusters: several tiles per cluster, ragged edges
                                              (300, 1000, 1024, 2, 64),
                                              (130, 520, 4096, 8, 64),
                                              (256, 768, 512, 8, 128)])
def test_cluster_split_k_equals_planes_summed_in_split_order(t0, oracle, rt, m, n, k, sk, tile_n):
    # gemm_gen.rs:447-448 leaves split_k planes for the host to add (examples/test_gemm_correctness.rs:203-207).  The
    # one-launch form adds the same partial sums in the same order inside the kernel: bit-identical to the planes added
    # on the host, within tolerance of the oracle, untouched guard area, identical reruns.
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    xa, xb = rt.upload(a), rt.upload(b)
    planes_buf = rt.alloc(m * n * 4 * sk)
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), planes_buf.gpu_addr(), m, n, k, split_k=sk, planes=True, tile_n=tile_n, pair_cta=2)
    planes = rt.read_f32(planes_buf, m * n * sk).reshape(sk, m, n)
    want = np.zeros((m, n), np.float32)
    for s in range(sk):
        want = want + planes[s]
    y = rt.alloc(m * n * 4 + 4096)
    for _ in range(2):
        y.write(np.full(m * n + 1024, SENTINEL, np.float32))
        before = rt.launch_count()
        rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, split_k=sk, tile_n=tile_n, pair_cta=2)
        rt.synchronize()
        assert rt.launch_count() - before == 1                       # one launch: no planes, no reduction pass
        got = y.read(m * n * 4, np.float32).reshape(m, n)
        assert np.array_equal(got, want)
        assert np.all(y.read_bytes(m * n * 4, 4096, np.float32) == SENTINEL)
    _, ysum = oracle.gemm_nt_splitk(a, b, m, k, n, sk)
    assert_gemm_close(want, ysum, k)
    # with a bias + ReLU epilogue and bf16 output: applied once, after the sum
    bias = ((np.arange(n) % 9) - 4).astype(np.float32)
    bb = rt.upload(bias)
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, split_k=sk, tile_n=tile_n, pair_cta=2, bias=bb.gpu_addr(), epilogue=2)
    rt.synchronize()
    assert np.array_equal(y.read(m * n * 4, np.float32).reshape(m, n), np.maximum(want + bias[None, :], 0.0).astype(np.float32))
    rt.gemm(xa.gpu_addr(), xb.gpu_addr(), y.gpu_addr(), m, n, k, split_k=sk, tile_n=tile_n, pair_cta=2, out_bf16=True)
    rt.synchronize()
    got16 = y.read(m * n * 2, np.uint16)
    assert np.array_equal(got16, oracle.f32_to_bf16_rne(want.reshape(-1)))
    for buf in (xa, xb, planes_buf, y, bb):
        buf.free()


def test_reserve_scratch_then_padded_and_planes_paths(t0, oracle):
    # The scratch-growing launch paths (K not a multiple of 8: padded operand copies; the two-launch split-K: fp32 planes)
    # after their buffers were reserved ahead of time; an unknown kind is an error, not a crash.
    rt = t0.GpuRuntime(0)
    try:
        m, k, n = 70, 1001, 136
        rt.reserve_scratch("operand_a", m * 1008 * 2)
        rt.reserve_scratch("operand_b", n * 1008 * 2)
        rt.reserve_scratch("splitk_planes", 128 * 256 * 4 * 4)
        rt.reserve_scratch("w4_fused", 0)
        assert rt.w4_fused_scratch_bytes() > 16384
        with pytest.raises(t0.T0Error):
            t0._check(t0.lib().t0_rt_reserve_scratch(rt._h, 99, 16))
        a, b = oracle.fill_uniform_bf16(m * k, 5), oracle.fill_uniform_bf16(n * k, 6)
        got = run_tile(t0, rt, t0.tile_auto_select(m, k, n), a, b, m, n, k)
        assert_gemm_close(got, oracle.gemm_nt(a, b, m, k, n), k)
    finally:
        rt.close()


@pytest.mark.parametrize("m,n,k,kw,count", [(128, 4096, 4096, {}, 5), (64, 1024, 2048, dict(tile_n=64, split_k=2, pair_cta=2), 40),
                                            (16, 512, 1024, dict(tile_n=128, split_k=8, pair_cta=2), 3), (200, 384, 512, dict(tile_n=128, split_k=4, pair_cta=2), 7),
                                            (300, 512, 256, {}, 4), (16, 4096, 4096, {}, 33), (128, 1024, 512, dict(tile_n=128), 6), (70, 200, 136, dict(tile_n=64, pair_cta=2), 5)])
def test_grouped_launch_equals_one_launch_per_problem(t0, oracle, rt, m, n, k, kw, count):
    # independent problems of one shape in one launch (the clusters walk the tiles of all of them): every y equals the y of
    # its own launch bit for bit, and the oracle within tolerance; more than 32 problems take two launches; a shape whose
    # configuration is not the one-launch split-K (the last case) runs back to back
    xs = [rt.upload(oracle.fill_uniform_bf16(m * k, 10 + i)) for i in range(count)]
    bs = [rt.upload(oracle.fill_uniform_bf16(n * k, 500 + i)) for i in range(count)]
    y_one = [rt.alloc(m * n * 4) for _ in range(count)]
    y_grp = [rt.alloc(m * n * 4) for _ in range(count)]
    for y in y_one + y_grp:
        y.write(np.full(m * n, SENTINEL, np.float32))
    for i in range(count):
        rt.gemm(xs[i].gpu_addr(), bs[i].gpu_addr(), y_one[i].gpu_addr(), m, n, k, **kw)
    rt.gemm_grouped([rt.gemm_args(xs[i].gpu_addr(), bs[i].gpu_addr(), y_grp[i].gpu_addr(), m, n, k, **kw) for i in range(count)])
    rt.synchronize()
    for i in range(count):
        one, grp = rt.read_f32(y_one[i], m * n), rt.read_f32(y_grp[i], m * n)
        if kw:
            assert np.array_equal(one, grp), f"problem {i}"            # the same tile and split: the same sums in the same order
        else:
            assert not np.any(grp == SENTINEL) and np.abs(one - grp).max() <= tol_abs(k), f"problem {i}"   # the split is chosen for the group
        if i in (0, count - 1):
            a, b = oracle.fill_uniform_bf16(m * k, 10 + i), oracle.fill_uniform_bf16(n * k, 500 + i)
            assert_gemm_close(grp.reshape(m, n), oracle.gemm_nt(a, b, m, k, n), k)
    for buf in xs + bs + y_one + y_grp:
        rt.recycle(buf)


def test_grouped_launch_refuses_dependent_problems(t0, rt):
    m, n, k = 128, 4096, 4096
    x, b, y = rt.alloc(m * k * 2), rt.alloc(n * k * 2), rt.alloc(m * n * 4)
    same_y = [rt.gemm_args(x.gpu_addr(), b.gpu_addr(), y.gpu_addr(), m, n, k) for _ in range(2)]
    with pytest.raises(t0.T0Error):
        rt.gemm_grouped(same_y)
    for buf in (x, b, y):
        rt.recycle(buf)


@pytest.mark.parametrize("m,n,k,kw", [(128, 2048, 1024, dict(tile_n=128, split_k=4, pair_cta=2)), (64, 4096, 512, {}), (100, 1000, 256, dict(tile_n=64, pair_cta=2))])
def test_grouped_launch_with_epilogues_and_bf16_output(t0, oracle, rt, m, n, k, kw):
    # the grouped launch carries the same epilogues as the single launch: gemm_gen bias + ReLU, a TileIR chain, bf16 output;
    # through the cluster split-K kernel (first case), the plain kernel chosen for the group (second) and ragged N (third)
    count = 6
    bias = (np.arange(n) % 11 - 5).astype(np.float32) * 0.25
    xb_bias = rt.upload(bias)
    a = [oracle.fill_uniform_bf16(m * k, 20 + i) for i in range(2)]
    b = [oracle.fill_uniform_bf16(n * k, 600 + i) for i in range(2)]
    xa, xb = [rt.upload(v) for v in a], [rt.upload(v) for v in b]
    plain = [oracle.gemm_nt(a[i], b[i], m, k, n) for i in range(2)]
    for what, extra, want_fn, out_bf16 in [("bias+relu", dict(bias=xb_bias.gpu_addr(), epilogue=2), lambda y: oracle.epilogue_gemm_gen(y, bias, 2), False),
                                           ("chain", dict(bias=xb_bias.gpu_addr(), tile_epilogue=["bias", "scale", "silu"], scale=0.5),
                                            lambda y: oracle.epilogue_tile(y, ["bias", "scale", "silu"], bias, 0.5, 0.0, 0.0), False),
                                           ("bf16", dict(out_bf16=True), lambda y: y, True)]:
        ys = [rt.alloc(m * n * 4) for _ in range(count)]
        calls = [rt.gemm_args(xa[i % 2].gpu_addr(), xb[i % 2].gpu_addr(), ys[i].gpu_addr(), m, n, k, **kw, **extra) for i in range(count)]
        rt.gemm_grouped(calls)
        rt.synchronize()
        for i in (0, 1, count - 1):
            want = want_fn(plain[i % 2])
            if out_bf16:
                got = oracle.bf16_to_f32(ys[i].read(m * n * 2, np.uint16)).reshape(m, n)
                assert np.abs(got - want).max() <= tol_abs(k) + np.abs(want).max() * 2.0 ** -8, what
            else:
                assert_gemm_close(rt.read_f32(ys[i], m * n).reshape(m, n), want, k)
        for y in ys:
            rt.recycle(y)
    for buf in xa + xb + [xb_bias]:
        rt.recycle(buf)


def test_grouped_launch_random_shapes(t0, oracle, rt):
    # a seeded sweep over shapes and configurations of the grouped entry (ragged M and N, K that is and is not a multiple of the
    # split, explicit and library-chosen tile and split): every problem against the oracle, rows and bytes beyond untouched
    rng = np.random.default_rng(2026)
    for case in range(14):
        m = int(rng.integers(1, 300))
        n = int(rng.integers(1, 190)) * 8
        k = int(rng.integers(1, 33)) * 64
        count = int(rng.integers(2, 6))
        choice = int(rng.integers(0, 4))
        kw = [{}, dict(tile_n=128, split_k=2, pair_cta=2), dict(tile_n=64, split_k=4, pair_cta=2), dict(tile_n=128, pair_cta=2)][choice]
        if kw.get("split_k", 1) > 1 and (k // 64) % kw["split_k"]:
            kw = {}
        a = [oracle.fill_uniform_bf16(m * k, 1000 + 10 * case + i) for i in range(count)]
        b = [oracle.fill_uniform_bf16(n * k, 5000 + 10 * case + i) for i in range(count)]
        xa, xb = [rt.upload(v) for v in a], [rt.upload(v) for v in b]
        ys = [rt.alloc(m * n * 4 + 4096) for _ in range(count)]
        for y in ys:
            y.write(np.full(m * n + 1024, SENTINEL, np.float32))
        rt.gemm_grouped([rt.gemm_args(xa[i].gpu_addr(), xb[i].gpu_addr(), ys[i].gpu_addr(), m, n, k, **kw) for i in range(count)])
        rt.synchronize()
        for i in range(count):
            got = ys[i].read((m * n + 1024) * 4, np.float32)
            assert_gemm_close(got[:m * n].reshape(m, n), oracle.gemm_nt(a[i], b[i], m, k, n), k), (case, m, n, k, kw)
            assert np.all(got[m * n:] == SENTINEL), ("wrote past the matrix", case, m, n, k, kw)
        for buf in xa + xb + ys:
            buf.free()

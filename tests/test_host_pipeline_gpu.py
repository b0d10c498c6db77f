"""GEMMs on host operands (`t0_gemm_launch_host_batch`): the upload / dispatch / read-back sequence of the reference's
host-facing calls (T0BlasLib::gemm, src/universal/math/blas.rs:18-100; dispatch_gemm_forward,
src/ignis/ops/bf16_matmul.rs:61-190) for an array of problems, checked against the CPU oracle.  The staging sets are
reused every second problem, so a batch of several different shapes also checks the ordering between the three queues:
a result overwritten too early or an operand replaced under a running kernel shows up as a wrong product."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def tol_abs(k):
    return 5e-3 * np.sqrt(max(k, 256) / 256.0)


def close(got, ref, k):
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()
    rel = np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref.astype(np.float64)), 1e-30)
    return err <= tol_abs(k) and rel <= 1e-3


def pinned(arr):
    t = torch.from_numpy(np.ascontiguousarray(arr)).pin_memory()
    return t, t.numpy()


def test_batch_of_mixed_shapes_matches_oracle(t0, oracle, rt):
    shapes = [(128, 256, 192, t0.NT), (256, 128, 64, t0.NN), (100, 136, 72, t0.NT), (64, 512, 384, t0.NT), (33, 100, 50, t0.NN),
              (512, 256, 512, t0.NT), (128, 64, 1000, t0.NT)]
    keep, args, want = [], [], []
    for i, (m, k, n, layout) in enumerate(shapes):
        a = oracle.fill_uniform_bf16(m * k, 42 + m + i)
        b = oracle.fill_uniform_bf16(n * k, 137 + n + i)
        ta, na = pinned(a.view(np.int16))
        tb, nb = pinned(b.view(np.int16))
        ty, ny = pinned(np.full(m * n, np.nan, np.float32))
        keep.append((ta, tb, ty))
        args.append(t0.GpuRuntime.gemm_args(na.ctypes.data, nb.ctypes.data, ny.ctypes.data, m, n, k, transpose=layout))
        want.append((oracle.gemm_nn(a, b, m, k, n) if layout == t0.NN else oracle.gemm_nt(a, b, m, k, n), ny, m, n, k))
    rt.gemm_host_batch(args)
    for i, (ref, ny, m, n, k) in enumerate(want):
        assert close(ny.reshape(m, n), ref, k), f"problem {i} ({m}x{n}x{k})"


def test_integer_operands_are_exact_and_repeatable(t0, oracle, rt):
    # small integers: every product and partial sum is exact in f32, so the result must equal the oracle bit for bit
    m, k, n = 256, 512, 256
    a = oracle.f32_to_bf16_trunc((np.arange(m * k) % 17 - 8).astype(np.float32))
    b = oracle.f32_to_bf16_trunc((np.arange(n * k) % 13 - 6).astype(np.float32))
    ref = oracle.gemm_nt(a, b, m, k, n)
    ta, na = pinned(a.view(np.int16))
    tb, nb = pinned(b.view(np.int16))
    outs = [pinned(np.zeros(m * n, np.float32)) for _ in range(5)]
    args = [t0.GpuRuntime.gemm_args(na.ctypes.data, nb.ctypes.data, ny.ctypes.data, m, n, k) for _, ny in outs]
    rt.gemm_host_batch(args)
    for _, ny in outs:
        assert np.array_equal(ny.reshape(m, n), ref)


def test_bias_epilogue_and_bf16_output_from_host(t0, oracle, rt):
    m, n, k = 128, 192, 256
    a = oracle.fill_uniform_bf16(m * k, 42 + m)
    b = oracle.fill_uniform_bf16(n * k, 137 + n)
    bias = (np.arange(n) % 11 - 5).astype(np.float32) * 0.25
    ta, na = pinned(a.view(np.int16))
    tb, nb = pinned(b.view(np.int16))
    tbias, nbias = pinned(bias)
    ty, ny = pinned(np.zeros(m * n, np.float32))
    ty2, ny2 = pinned(np.zeros(m * n, np.int16))
    plain = oracle.gemm_nt(a, b, m, k, n)
    rt.gemm_host_batch([
        t0.GpuRuntime.gemm_args(na.ctypes.data, nb.ctypes.data, ny.ctypes.data, m, n, k, bias=nbias.ctypes.data, epilogue=2),
        t0.GpuRuntime.gemm_args(na.ctypes.data, nb.ctypes.data, ny2.ctypes.data, m, n, k, out_bf16=True),
    ])
    assert close(ny.reshape(m, n), oracle.epilogue_gemm_gen(plain, bias, 2), k)
    got_bf16 = (ny2.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(m, n)
    assert np.abs(got_bf16 - plain).max() <= tol_abs(k) + np.abs(plain).max() * 2.0 ** -8


def test_single_problem_and_pageable_memory(t0, oracle, rt):
    m, k, n = 64, 128, 96
    a = oracle.fill_uniform_bf16(m * k, 7)
    b = oracle.fill_uniform_bf16(n * k, 8)
    a16, b16 = np.ascontiguousarray(a.view(np.int16)), np.ascontiguousarray(b.view(np.int16))
    y = np.zeros(m * n, np.float32)                      # ordinary (pageable) numpy memory
    arg = t0.GpuRuntime.gemm_args(a16.ctypes.data, b16.ctypes.data, y.ctypes.data, m, n, k)
    t0._check(t0.lib().t0_gemm_launch_host(rt._h, arg))
    assert close(y.reshape(m, n), oracle.gemm_nt(a, b, m, k, n), k)


def test_argument_errors(t0, rt):
    y = np.zeros(16, np.float32)
    x = np.zeros(16, np.int16)
    ok = dict(m=4, n=4, k=4)
    with pytest.raises(t0.T0Error):
        rt.gemm_host_batch([t0.GpuRuntime.gemm_args(0, x.ctypes.data, y.ctypes.data, **ok)])
    with pytest.raises(t0.T0Error):
        rt.gemm_host_batch([t0.GpuRuntime.gemm_args(x.ctypes.data, x.ctypes.data, y.ctypes.data, planes=True, split_k=2, **ok)])
    with pytest.raises(t0.T0Error):
        rt.gemm_host_batch([t0.GpuRuntime.gemm_args(x.ctypes.data, x.ctypes.data, y.ctypes.data, epilogue=1, **ok)])   # bias missing
    with pytest.raises(t0.T0Error):
        rt.gemm_host_batch([t0.GpuRuntime.gemm_args(x.ctypes.data, x.ctypes.data, y.ctypes.data, m=0, n=4, k=4)])
    rt.gemm_host_batch([])                               # nothing to do is not an error
    assert not rt.is_poisoned()

"""GPU test of the allocation-free W4A16 entry (`t0_w4a16_gemm_static`), collected last.

The entry runs the fused INT4 GEMM with its scratch in a fixed array inside the library.  It must give the same bits as
`t0_w4a16_gemm` (same kernel, same order of additions), on two calls in a row (the arrival counters in the shared
array have to be back at zero after the first), whether this file runs alone or after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _inputs(oracle, M, N, K, G, seed):
    a = oracle.fill_normal_bf16(M * K, 11 + seed)
    packed = oracle.fill_u32((K // 8) * N, 4000 + seed)
    scales = oracle.fill_range_bf16((K // G) * N, 5000 + seed, 0.001, 0.02)
    zeros = oracle.fill_u32((K // G) * (N // 8), 6000 + seed)
    return a, packed, scales, zeros


@pytest.mark.parametrize("M,N,K,G", [(16, 11008, 4096, 128), (1, 14336, 4096, 128), (5, 1024, 512, 128), (8, 96, 256, 256)])
def test_static_entry_matches_the_allocating_entry_twice(t0, oracle, rt, M, N, K, G):
    lib = t0.lib()
    assert lib.t0_w4a16_gemm_static_scratch_bytes() >= 16 * 1024 + 148 * 2 * 16 * 256 * 4
    a, packed, scales, zeros = _inputs(oracle, M, N, K, G, M + N)
    ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
    xa, xp, xs, xz = rt.upload(a), rt.upload(packed), rt.upload(scales), rt.upload(zeros)
    y_ref, y = rt.alloc(M * N * 4), rt.alloc(M * N * 4)
    rt.w4a16_gemm(xa.gpu_addr(), xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), y_ref.gpu_addr(), M, N, K, G)
    rt.synchronize()
    want = y_ref.read(M * N * 4, np.float32).reshape(M, N)
    for call in range(2):
        y.write(np.full(M * N, -7777.0, np.float32))
        t0._check(lib.t0_w4a16_gemm_static(rt._h, xa.gpu_addr(), xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), y.gpu_addr(), M, N, K, G))
        rt.synchronize()
        got = y.read(M * N * 4, np.float32).reshape(M, N)
        assert np.array_equal(got, want), f"call {call}: differs from t0_w4a16_gemm"
    err = np.abs(want.astype(np.float64) - ref)
    assert err.max() <= 5e-3 * np.sqrt(max(K, 256) / 256.0)
    for b in (xa, xp, xs, xz, y_ref, y):
        b.free()


def test_static_entry_refuses_what_does_not_fit(t0, oracle, rt):
    lib = t0.lib()
    buf = rt.alloc(1 << 20)
    p = buf.gpu_addr()
    for (M, N, K, G) in [(17, 1024, 512, 128),        # M beyond the fused kernel
                         (4, 1000, 512, 128),         # N not a multiple of 32
                         (4, 1024, 192, 64),          # K and group not multiples of 128
                         (1, 2 ** 21, 128, 128)]:     # more bands than the fixed counter area
        rc = lib.t0_w4a16_gemm_static(rt._h, p, p, p, p, p, M, N, K, G)
        assert rc == 6, (M, N, K, G, rc)                 # T0_ERR_UNSUPPORTED
        assert len(lib.t0_last_error()) > 0
    assert not rt.is_poisoned()
    buf.free()

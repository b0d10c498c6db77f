"""GPU parity tests of the f32 framework entries: Ignis matmul + backward helpers and the BlasLib facade.

Reference: src/ignis/ops/bf16_matmul.rs:33-59,93-133,162-312 (operands rounded to bf16 nearest-even :371-372, fp32
accumulate) and src/universal/math/blas.rs:18-100.  The checker is the oracle GEMM on operands rounded the same way;
tolerances are the GEMM ones (relative L2 <= 1e-3, |err| <= 5e-3*sqrt(K/256)); integer-valued inputs must be exact.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def assert_gemm_close(got, ref, k):
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    rel = np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref.astype(np.float64)), 1e-30)
    assert err.max() <= 5e-3 * np.sqrt(max(k, 256) / 256.0), err.max()
    assert rel <= 1e-3, rel


def f32_case(m, k, n, seed):
    rng = np.random.default_rng(seed)
    return rng.uniform(-1, 1, (m, k)).astype(np.float32), rng.uniform(-1, 1, (k, n)).astype(np.float32)


SHAPES = [(64, 256, 512), (1, 64, 8), (33, 100, 50), (128, 130, 72), (200, 1000, 7), (512, 512, 512), (17, 8, 24)]


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_matmul_forward(t0, oracle, rt, m, k, n):
    x, w = f32_case(m, k, n, m + k + n)
    ref = oracle.gemm_nn(oracle.f32_to_bf16_rne(x), oracle.f32_to_bf16_rne(w), m, k, n)
    xd, wd = rt.upload(x), rt.upload(w)
    y = rt.alloc(m * n * 4 + 4096)
    y.write(np.full(m * n + 1024, -9999.0, np.float32))
    rt.matmul_f32(xd.gpu_addr(), wd.gpu_addr(), y.gpu_addr(), m, k, n)
    rt.synchronize()
    assert_gemm_close(y.read(m * n * 4, np.float32).reshape(m, n), ref, k)
    assert np.all(y.read_bytes(m * n * 4, 4096, np.float32) == -9999.0)
    for b in (xd, wd, y):
        b.free()


def test_matmul_integer_inputs_are_exact_and_rounding_is_nearest_even(t0, oracle, rt):
    m, k, n = 48, 96, 40
    x = (np.arange(m * k) % 17 - 8).astype(np.float32).reshape(m, k)
    w = (np.arange(k * n) % 13 - 6).astype(np.float32).reshape(k, n)
    xd, wd, y = rt.upload(x), rt.upload(w), rt.alloc(m * n * 4)
    rt.matmul_f32(xd.gpu_addr(), wd.gpu_addr(), y.gpu_addr(), m, k, n)
    assert np.array_equal(rt.read_f32(y, m * n).reshape(m, n), x @ w)
    # a tie (1 + 2^-8) must round to even: x = [[1+2^-8]], w = [[1]] -> 1.0; 1 + 3*2^-8 -> 1 + 2^-6
    ties = np.array([[1 + 2.0 ** -8, 1 + 3 * 2.0 ** -8]], np.float32)
    eye = np.eye(2, dtype=np.float32)
    td, ed, o = rt.upload(ties), rt.upload(eye), rt.alloc(8)
    rt.matmul_f32(td.gpu_addr(), ed.gpu_addr(), o.gpu_addr(), 1, 2, 2)
    assert np.array_equal(rt.read_f32(o, 2), np.array([1.0, 1 + 2.0 ** -6], np.float32))
    for b in (xd, wd, y, td, ed, o):
        b.free()


@pytest.mark.parametrize("m,k,n", SHAPES[:6])
def test_matmul_backward_and_pretransposed_weight(t0, oracle, rt, m, k, n):
    x, w = f32_case(m, k, n, 7 * m + n)
    dy = np.random.default_rng(k).uniform(-1, 1, (m, n)).astype(np.float32)
    xb, wb, dyb = oracle.f32_to_bf16_rne(x), oracle.f32_to_bf16_rne(w), oracle.f32_to_bf16_rne(dy)
    xd, wd, dyd = rt.upload(x), rt.upload(w), rt.upload(dy)
    # dX = dY * W^T (contraction over N)
    dx = rt.alloc(m * k * 4)
    rt.matmul_f32_backward_data(dyd.gpu_addr(), wd.gpu_addr(), dx.gpu_addr(), m, k, n)
    assert_gemm_close(rt.read_f32(dx, m * k).reshape(m, k), oracle.gemm_nt(dyb, wb, m, n, k), n)
    # dW = X^T * dY (contraction over M)
    dw = rt.alloc(k * n * 4)
    rt.matmul_f32_backward_weight(xd.gpu_addr(), dyd.gpu_addr(), dw.gpu_addr(), m, k, n)
    xt = np.ascontiguousarray(xb.reshape(m, k).T)
    assert_gemm_close(rt.read_f32(dw, k * n).reshape(k, n), oracle.gemm_nn(xt, dyb, k, m, n), m)
    # forward with the weight already transposed and in bf16
    wt = rt.upload(np.ascontiguousarray(wb.reshape(k, n).T))
    y = rt.alloc(m * n * 4)
    rt.matmul_f32_with_wt_bf16(xd.gpu_addr(), wt.gpu_addr(), y.gpu_addr(), m, k, n)
    assert_gemm_close(rt.read_f32(y, m * n).reshape(m, n), oracle.gemm_nn(xb, wb, m, k, n), k)
    for b in (xd, wd, dyd, dx, dw, wt, y):
        b.free()


@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (0.5, 2.0), (-1.25, 1.0)])
def test_blas_gemm_with_leading_dimensions(t0, oracle, rt, alpha, beta):
    m, n, k, lda, ldb, ldc = 70, 52, 96, 100, 60, 64
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, (m, lda)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, ldb)).astype(np.float32)
    c = rng.uniform(-1, 1, (m, ldc)).astype(np.float32)
    prod = oracle.gemm_nn(oracle.f32_to_bf16_rne(np.ascontiguousarray(a[:, :k])), oracle.f32_to_bf16_rne(np.ascontiguousarray(b[:, :n])), m, k, n)
    want = c.copy()
    want[:, :n] = np.float32(alpha) * prod + (np.float32(beta) * c[:, :n] if beta != 0.0 else 0)
    ad, bd, cd = rt.upload(a), rt.upload(b), rt.upload(c)
    rt.blas_gemm_f32(m, n, k, alpha, ad.gpu_addr(), lda, bd.gpu_addr(), ldb, beta, cd.gpu_addr(), ldc)
    got = rt.read_f32(cd, m * ldc).reshape(m, ldc)
    assert np.array_equal(got[:, n:], c[:, n:])                      # columns past n are not touched
    assert_gemm_close(got[:, :n], want[:, :n], k)
    for buf in (ad, bd, cd):
        buf.free()


def test_blas_gemv(t0, rt):
    m, n, lda, incx, incy = 300, 257, 260, 2, 3
    rng = np.random.default_rng(9)
    a = rng.uniform(-1, 1, (m, lda)).astype(np.float32)
    x = rng.uniform(-1, 1, n * incx).astype(np.float32)
    y = rng.uniform(-1, 1, m * incy).astype(np.float32)
    want = y.copy()
    want[::incy] = 0.75 * (a[:, :n].astype(np.float64) @ x[::incx].astype(np.float64)) + (-0.5) * y[::incy]
    ad, xd, yd = rt.upload(a), rt.upload(x), rt.upload(y)
    rt.blas_gemv_f32(m, n, 0.75, ad.gpu_addr(), lda, xd.gpu_addr(), incx, -0.5, yd.gpu_addr(), incy)
    got = rt.read_f32(yd, m * incy)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)              # f32 sums in a different order than the CPU loop
    mask = np.ones(m * incy, bool)
    mask[::incy] = False
    assert np.array_equal(got[mask], y[mask])
    for buf in (ad, xd, yd):
        buf.free()


def test_f32_entries_reject_bad_arguments(t0, rt):
    buf = rt.alloc(4096)
    p = buf.gpu_addr()
    lib = t0.lib()
    assert lib.t0_matmul_f32(rt._h, 0, p, p, 4, 4, 4) == 1
    assert lib.t0_blas_gemm_f32(rt._h, 4, 4, 4, 1.0, p, 2, p, 4, 0.0, p, 4) == 1     # lda < k
    assert lib.t0_blas_gemv_f32(rt._h, 4, 4, 1.0, p, 4, p, 0, 0.0, p, 1) == 1        # incx == 0
    assert lib.t0_matmul_f32(rt._h, p, p, p, 0, 4, 4) == 0                           # empty M is a no-op
    buf.free()

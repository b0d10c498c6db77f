"""GPU parity tests for the INT4 path: stand-alone dequantisation (bit-exact) and the fused W4A16 GEMM.

Reference items: src/t0/quant_kernels.rs:53-171 (dequant kernels, kernarg ABI :45-47), :188-294 (GptqWeight),
known answers :346-481.  The fused GEMM has no reference counterpart; it is checked against the oracle's
dequant-then-GEMM with the GEMM tolerances (relative L2 <= 1e-3, |err| <= 5e-3*sqrt(K/256)), and its dequantised
weights are extracted bit-exactly with one-hot activations.
"""
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def make_w4(oracle, K, N, G, seed=0):
    packed = oracle.fill_u32((K // 8) * N, 1000 + seed)
    scales = oracle.fill_range_bf16((K // G) * N, 2000 + seed, 0.001, 0.02)
    zeros = oracle.fill_u32((K // G) * ((N + 7) // 8), 3000 + seed)
    return packed, scales, zeros


def run_w4a16(rt, a, packed, scales, zeros, M, N, K, G):
    xa, xp, xs, xz = rt.upload(a), rt.upload(packed), rt.upload(scales), rt.upload(zeros)
    y = rt.alloc(M * N * 4 + 4096)
    y.write(np.full(M * N + 1024, -9999.0, np.float32))
    rt.w4a16_gemm(xa.gpu_addr(), xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), y.gpu_addr(), M, N, K, G)
    rt.synchronize()
    out = y.read(M * N * 4, np.float32).reshape(M, N)
    tail = y.read_bytes(M * N * 4, 4096, np.float32)
    assert np.all(tail == -9999.0), "wrote past the output"
    for b in (xa, xp, xs, xz, y):
        b.free()
    return out


def assert_close(got, ref, k):
    err = np.abs(got.astype(np.float64) - ref)
    rel = np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref.astype(np.float64)), 1e-30)
    assert err.max() <= 5e-3 * np.sqrt(max(k, 256) / 256.0), err.max()
    assert rel <= 1e-3, rel


# ----------------------------------------------------------------------------- K3, reference wire format

@pytest.mark.parametrize("rows,cols,glog2", [(16, 16, 4), (4, 256, 7), (33, 128, 7), (7, 50, 1), (64, 1024, 8)])
@pytest.mark.parametrize("bf16", [False, True])
def test_dequant_reference_format_bit_exact(t0, oracle, rt, rows, cols, glog2, bf16):
    rng = np.random.default_rng(rows * cols + glog2)
    total = rows * cols
    packed = rng.integers(0, 256, size=(total + 1) // 2, dtype=np.uint8)
    n_groups = ((total - 1) >> glog2) + 1
    scales = rng.uniform(-2.0, 2.0, n_groups).astype(np.float32)
    zps = rng.integers(-20, 20, n_groups).astype(np.int32)
    want = oracle.dequant_int4_ref(packed, scales, zps, rows, cols, glog2, bf16=bf16)
    xp, xs, xz = rt.upload(packed), rt.upload(scales), rt.upload(zps)
    out = rt.alloc(total * 4)
    rt.dequant_int4(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), out.gpu_addr(), rows, cols, glog2, out_bf16=bf16)
    rt.synchronize()
    got = out.read(total * (2 if bf16 else 4), np.uint16 if bf16 else np.float32).reshape(rows, cols)
    assert np.array_equal(got.view(np.uint16 if bf16 else np.uint32), want.view(np.uint16 if bf16 else np.uint32))
    # the same kernel through the reference's 40-byte kernarg blob (quant_kernels.rs:45-47) and its grid rule (:49-52)
    kern = rt.ensure_dequant_kernel(glog2, bf16)
    assert kern.kernarg_size == 40
    out.zero()
    ka = struct.pack("<QQQQII", xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), out.gpu_addr(), rows, cols)
    rt.dispatch(kern, [-(-total // 256) * 256, 1, 1], ka)
    got2 = out.read(total * (2 if bf16 else 4), np.uint16 if bf16 else np.float32).reshape(rows, cols)
    assert np.array_equal(got2.view(np.uint16 if bf16 else np.uint32), want.view(np.uint16 if bf16 else np.uint32))


def test_dequant_known_answers(t0, rt):
    # quant_kernels.rs:347-354,365-372,441-448: 0xAB -> 11, 10; 0xD7 -> 7, 13; (12 - 8) * 0.5 = 2.0
    xp = rt.upload(np.array([0xAB, 0xD7, 0x0C, 0x00], np.uint8))
    xs = rt.upload(np.array([1.0, 0.5], np.float32))
    xz = rt.upload(np.array([0, 8], np.int32))
    out = rt.alloc(64)
    rt.dequant_int4(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), out.gpu_addr(), 1, 8, 2)
    rt.synchronize()
    got = out.read(32, np.float32)
    assert got[:4].tolist() == [11.0, 10.0, 7.0, 13.0]
    assert got[4] == 2.0


# ----------------------------------------------------------------------------- K3, B200 layout

@pytest.mark.parametrize("K,N,G", [(128, 8, 128), (512, 264, 128), (256, 100, 64), (64, 1000, 32), (4096, 512, 128)])
def test_dequant_b200_layout_bit_exact(t0, oracle, rt, K, N, G):
    packed, scales, zeros = make_w4(oracle, K, N, G)
    want = oracle.dequant_w4_b200(packed, scales, zeros, K, N, G)
    xp, xs, xz = rt.upload(packed), rt.upload(scales), rt.upload(zeros)
    out = rt.alloc(K * N * 2)
    rt.w4_dequant(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), out.gpu_addr(), K, N, G)
    rt.synchronize()
    assert np.array_equal(out.read(K * N * 2, np.uint16).reshape(K, N), want)


def test_dequant_exhaustive_code_zero_scale(t0, oracle, rt):
    # every (q, z, s): 16 codes down K in each group of 16, one (z, s) pair per (group, column):
    # 65536 bf16 scale patterns x 16 zero points (non-finite scales excluded: NaN payloads are not a parity subject)
    K, G, N = 4096, 16, 4096
    k = np.arange(K)
    codes = (k % 16).astype(np.uint32)
    word_of_group = np.zeros(K // 8, np.uint32)
    for kk in range(8):
        word_of_group |= codes[kk::8] << np.uint32(4 * kk)
    packed = np.repeat(word_of_group[:, None], N, axis=1).astype(np.uint32)
    pair = np.arange((K // G) * N, dtype=np.uint32).reshape(K // G, N)
    sbits = (pair & 0xFFFF).astype(np.uint16)
    sbits = np.where((sbits & 0x7F80) == 0x7F80, np.uint16(0x3C00), sbits)
    z = (pair >> 16).astype(np.uint32) & 0xF
    zeros = np.zeros((K // G, N // 8), np.uint32)
    for j in range(8):
        zeros |= z[:, j::8] << np.uint32(4 * j)
    want = oracle.dequant_w4_b200(packed, sbits, zeros, K, N, G)
    xp, xs, xz = rt.upload(packed), rt.upload(sbits), rt.upload(zeros)
    out = rt.alloc(K * N * 2)
    rt.w4_dequant(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), out.gpu_addr(), K, N, G)
    rt.synchronize()
    assert np.array_equal(out.read(K * N * 2, np.uint16).reshape(K, N), want)
    for b in (xp, xs, xz, out):
        b.free()


def test_gptq_container_to_b200(t0, oracle, rt):
    # a GptqWeight blob (quant_kernels.rs:242-286) -> B200 layout -> same weights as the reference-format kernel, rounded once
    rng = np.random.default_rng(11)
    N, K, G = 48, 256, 128
    q = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8).ravel()
    scales = oracle.bf16_to_f32(oracle.fill_range_bf16(N * (K // G), 1, 0.001, 0.02))
    zps = rng.integers(0, 16, size=N * (K // G)).astype(np.int32)
    raw = np.array([N, K, G], "<u4").tobytes() + packed.tobytes() + scales.astype("<f4").tobytes() + zps.astype("<i4").tobytes()
    g = t0.gptq_parse(raw)
    assert (g["rows"], g["cols"], g["group_size"], g["n_groups"]) == (N, K, G, K // G)
    assert g["gpu_buffer_size"] == packed.size + scales.size * 4 + zps.size * 4
    with pytest.raises(t0.T0Error):
        t0.gptq_parse(raw[:-1])
    p, s, z, inexact = t0.gptq_to_b200(g["packed"], g["scales"], g["zero_points"], N, K, G)
    assert inexact == 0
    po, so, zo, _ = oracle.gptq_to_b200(packed, scales, zps, N, K, G)
    assert np.array_equal(p, po) and np.array_equal(s, so) and np.array_equal(z, zo)
    ref = oracle.dequant_int4_ref(packed, scales, zps, N, K, 7)                       # [N, K] f32, reference formula
    xp, xs, xz = rt.upload(p), rt.upload(s), rt.upload(z)
    out = rt.alloc(K * N * 2)
    rt.w4_dequant(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), out.gpu_addr(), K, N, G)
    rt.synchronize()
    w = oracle.bf16_to_f32(out.read(K * N * 2, np.uint16)).reshape(K, N)
    assert np.array_equal(w, oracle.bf16_to_f32(oracle.f32_to_bf16_rne(ref)).reshape(N, K).T)
    with pytest.raises(t0.T0Error):
        t0.gptq_to_b200(packed, scales, np.full_like(zps, 16), N, K, G)              # a zero point that needs five bits


# ----------------------------------------------------------------------------- K2, fused GEMM

def test_fused_kernel_dequantises_bit_exactly(t0, oracle, rt):
    # one-hot activations make row m of y equal to row k0+m of the dequantised weights, exactly:
    # this reads the fused kernel's in-register dequant back without any rounding of its own
    K, G, M = 128, 128, 16
    N = 65536
    codes = (np.arange(K) % 16).astype(np.uint32)
    words = np.zeros(K // 8, np.uint32)
    for kk in range(8):
        words |= codes[kk::8] << np.uint32(4 * kk)
    packed = np.repeat(words[:, None], N, axis=1).astype(np.uint32)
    col = np.arange(N, dtype=np.uint32)
    # positive and negative normal scales over four octaves around the benchmark's range, all 16 zero points
    sbits = (0x3A00 + (col % 0x400)).astype(np.uint16) | ((col // 0x400 % 2) << 15).astype(np.uint16)
    z = (col // 0x800) % 16
    zeros = np.zeros((1, N // 8), np.uint32)
    for j in range(8):
        zeros[0] |= z[j::8].astype(np.uint32) << np.uint32(4 * j)
    a = np.zeros((M, K), np.uint16)
    for m in range(M):
        a[m, m] = 0x3F80
    want = oracle.bf16_to_f32(oracle.dequant_w4_b200(packed, sbits.reshape(1, N), zeros, K, N, G)).reshape(K, N)[:M]
    got = run_w4a16(rt, a, packed, sbits.reshape(1, N), zeros, M, N, K, G)
    assert np.array_equal(got.view(np.uint32) & 0x7FFFFFFF, want.view(np.uint32) & 0x7FFFFFFF)   # sign of zero aside
    assert np.array_equal(got, want)


@pytest.mark.parametrize("M", [1, 2, 5, 8, 9, 16])
@pytest.mark.parametrize("K,N,G", [(512, 264, 128), (32, 40, 32), (1024, 32, 64), (4096, 96, 128)])
def test_fused_small_shapes(t0, oracle, rt, M, K, N, G):
    a = oracle.fill_normal_bf16(M * K, 7 + M)
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=M)
    ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
    got = run_w4a16(rt, a, packed, scales, zeros, M, N, K, G)
    assert_close(got, ref, K)


@pytest.mark.parametrize("M", [1, 16, 128])
@pytest.mark.parametrize("N", [11008, 14336])
def test_w4a16_full_size(t0, oracle, rt, M, N):
    # the W4A16 configuration at full size: K = 4096, group 128, activations N(0,1), codes uniform, scales U(0.001, 0.02), zero points uniform
    K, G = 4096, 128
    a = oracle.fill_normal_bf16(M * K, 7 + M)
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=N)
    ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
    xa, xp, xs, xz = rt.upload(a), rt.upload(packed), rt.upload(scales), rt.upload(zeros)
    y = rt.alloc(M * N * 4)
    outs = []
    for _ in range(3):   # the scratch area (slab counters, straddling pieces) is reused: repeated calls must agree bit for bit
        y.zero()
        rt.w4a16_gemm(xa.gpu_addr(), xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), y.gpu_addr(), M, N, K, G)
        rt.synchronize()
        outs.append(y.read(M * N * 4, np.float32).reshape(M, N))
    assert_close(outs[0], ref, K)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])
    for b in (xa, xp, xs, xz, y):
        b.free()


def test_general_shapes_take_the_two_step_path(t0, oracle, rt):
    # M > 16, or N / K / group the fused kernel does not take: dequantise into scratch, then the bf16 GEMM
    for (M, K, N, G) in [(33, 256, 100, 64), (17, 512, 264, 128), (4, 64, 12, 8)]:
        a = oracle.fill_normal_bf16(M * K, 3)
        packed, scales, zeros = make_w4(oracle, K, N, G)
        ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
        assert_close(run_w4a16(rt, a, packed, scales, zeros, M, N, K, G), ref, K)


def test_argument_errors(t0, rt):
    b = rt.alloc(4096)
    with pytest.raises(t0.T0Error):
        rt.w4a16_gemm(b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), 1, 8, 12, 4)    # K % 8
    with pytest.raises(t0.T0Error):
        rt.w4a16_gemm(b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), 1, 8, 64, 48)   # group does not divide K
    with pytest.raises(t0.T0Error):
        rt.w4a16_gemm(0, b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), 1, 8, 64, 32)
    rt.w4a16_gemm(b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), b.gpu_addr(), 0, 8, 64, 32)        # M = 0: no-op
    assert not rt.is_poisoned()


# ----------------------------------------------------------------------------- K2 on the streaming (tile-major) layout

def run_w4a16_prepacked(rt, a, packed, scales, zeros, M, N, K, G, repeats=1):
    xa, xp, xs, xz = rt.upload(a), rt.upload(packed), rt.upload(scales), rt.upload(zeros)
    pre = rt.w4_prepack(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), K, N, G)
    y = rt.alloc(M * N * 4 + 4096)
    outs = []
    for _ in range(repeats):
        y.write(np.full(M * N + 1024, -9999.0, np.float32))
        rt.w4a16_gemm_prepacked(xa.gpu_addr(), pre.gpu_addr(), y.gpu_addr(), M, N, K, G)
        rt.synchronize()
        outs.append(y.read(M * N * 4, np.float32).reshape(M, N))
        assert np.all(y.read_bytes(M * N * 4, 4096, np.float32) == -9999.0), "wrote past the output"
    for b in (xa, xp, xs, xz, pre, y):
        b.free()
    return outs if repeats > 1 else outs[0]


@pytest.mark.parametrize("K,N,G", [(128, 8, 128), (256, 264, 128), (512, 1000, 256), (4096, 11008, 128), (1024, 256, 1024)])
def test_prepack_matches_the_oracle_bit_for_bit(t0, oracle, rt, K, N, G):
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=K + N)
    want = oracle.w4_prepack(packed, scales, zeros, K, N, G)
    assert t0.lib().t0_w4_prepacked_bytes(K, N, G) == want.size
    xp, xs, xz = rt.upload(packed), rt.upload(scales), rt.upload(zeros)
    pre = rt.w4_prepack(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), K, N, G)
    rt.synchronize()
    assert np.array_equal(pre.read(want.size, np.uint8), want)
    for b in (xp, xs, xz, pre):
        b.free()


def test_prepacked_kernel_dequantises_bit_exactly(t0, oracle, rt):
    # one-hot activations, sixteen k at a time, read all 128 rows of the dequantised weights of a step back exactly
    K, G, M = 256, 128, 16
    N = 16384
    rng = np.random.default_rng(5)
    packed = rng.integers(0, 2 ** 32, size=(K // 8, N), dtype=np.uint64).astype(np.uint32)
    col = np.arange(N, dtype=np.uint32)
    sbits = np.stack([(0x3A00 + (col % 0x400)).astype(np.uint16) | ((col // 0x400 % 2) << 15).astype(np.uint16),
                      (0x3B80 + (col % 0x300)).astype(np.uint16)])
    zeros = rng.integers(0, 2 ** 32, size=(K // G, N // 8), dtype=np.uint64).astype(np.uint32)
    want = oracle.bf16_to_f32(oracle.dequant_w4_b200(packed, sbits, zeros, K, N, G)).reshape(K, N)
    for base in range(0, K, 16):
        a = np.zeros((M, K), np.uint16)
        for m in range(M):
            a[m, base + m] = 0x3F80
        got = run_w4a16_prepacked(rt, a, packed, sbits, zeros, M, N, K, G)
        assert np.array_equal(got.view(np.uint32) & 0x7FFFFFFF, want[base:base + 16].view(np.uint32) & 0x7FFFFFFF), base


@pytest.mark.parametrize("M", [1, 5, 8, 16])
@pytest.mark.parametrize("K,N,G", [(512, 264, 128), (4096, 96, 128), (1024, 1024, 256), (256, 8, 128), (2048, 3000, 512)])
def test_prepacked_small_shapes(t0, oracle, rt, M, K, N, G):
    a = oracle.fill_normal_bf16(M * K, 7 + M)
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=M)
    ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
    assert_close(run_w4a16_prepacked(rt, a, packed, scales, zeros, M, N, K, G), ref, K)


@pytest.mark.parametrize("M", [1, 16])
@pytest.mark.parametrize("N", [11008, 14336])
def test_prepacked_w4a16_full_size(t0, oracle, rt, M, N):
    K, G = 4096, 128
    a = oracle.fill_normal_bf16(M * K, 7 + M)
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=N)
    ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
    outs = run_w4a16_prepacked(rt, a, packed, scales, zeros, M, N, K, G, repeats=3)   # the first call runs on cold buffers
    assert_close(outs[0], ref, K)
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])


def test_prepacked_argument_errors(t0, rt):
    buf = rt.alloc(1 << 20)
    p = buf.gpu_addr()
    lib = t0.lib()
    assert lib.t0_w4_prepacked_bytes(100, 64, 128) == 0
    assert lib.t0_w4a16_gemm_prepacked(rt._h, p, p, p, 17, 256, 128, 128) == 6        # M beyond the fused kernel
    assert lib.t0_w4a16_gemm_prepacked(rt._h, p, p, p, 4, 256, 192, 64) == 6          # K, group not multiples of 128
    assert lib.t0_w4a16_gemm_prepacked(rt._h, p, 0, p, 1, 256, 128, 128) == 1         # null pointer
    assert not rt.is_poisoned()
    buf.free()


def test_row_layout_more_than_one_wave_of_steps(t0, oracle, rt):
    # K*N large enough that a CTA owns more than 20 steps: the row-layout entry then runs the first fused kernel, which
    # restages its activations in batches of 12 steps
    M, K, N, G = 4, 8192, 16384, 128
    a = oracle.fill_normal_bf16(M * K, 5)
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=3)
    ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
    outs = []
    for _ in range(2):
        outs.append(run_w4a16(rt, a, packed, scales, zeros, M, N, K, G))
    assert_close(outs[0], ref, K)
    assert np.array_equal(outs[0], outs[1])


def test_prepacked_long_ranges(t0, oracle, rt):
    # K*N large enough that a CTA walks dozens of steps and several whole bands: the ring wraps many times
    M, K, N, G = 4, 8192, 16384, 128
    a = oracle.fill_normal_bf16(M * K, 5)
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=3)
    ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
    outs = run_w4a16_prepacked(rt, a, packed, scales, zeros, M, N, K, G, repeats=2)
    assert_close(outs[0], ref, K)
    assert np.array_equal(outs[0], outs[1])


def _batch_problems(oracle, rt, shapes, seed0):
    """Uploads and prepacks one problem per (M, K, N, G); returns (args, per-problem host data, buffers)."""
    probs, bufs = [], []
    for i, (M, K, N, G) in enumerate(shapes):
        a = oracle.fill_normal_bf16(M * K, seed0 + i)
        packed, scales, zeros = make_w4(oracle, K, N, G, seed=seed0 + 100 + i)
        xa, xp, xs, xz = rt.upload(a), rt.upload(packed), rt.upload(scales), rt.upload(zeros)
        pre = rt.w4_prepack(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), K, N, G)
        y = rt.alloc(M * N * 4 + 4096)
        y.write(np.full(M * N + 1024, -9999.0, np.float32))
        rt.synchronize()
        for b in (xp, xs, xz):
            b.free()
        probs.append(dict(M=M, K=K, N=N, G=G, a=a, packed=packed, scales=scales, zeros=zeros, xa=xa, pre=pre, y=y))
        bufs += [xa, pre, y]
    return probs, bufs


def test_prepacked_batch_of_mixed_problems(t0, oracle, rt):
    # one launch walks the steps of every problem of the list: different M (both row-group forms), K, N, group sizes,
    # ranges that start and end inside bands of different problems
    shapes = [(1, 4096, 11008, 128), (16, 512, 264, 128), (5, 1024, 1024, 256), (8, 256, 8, 128), (2, 2048, 3000, 512),
              (16, 4096, 1536, 128), (1, 128, 40, 128), (9, 1024, 4096, 128)]
    probs, bufs = _batch_problems(oracle, rt, shapes, 50)
    calls = [t0.W4A16Args(p["xa"].gpu_addr(), p["pre"].gpu_addr(), 0, 0, p["y"].gpu_addr(), p["M"], p["N"], p["K"], p["G"]) for p in probs]
    before = rt.launch_count()
    rt.w4a16_gemm_prepacked_batch(calls)
    rt.synchronize()
    assert rt.launch_count() - before == 1                    # one launch for the whole list
    batch_out = []
    for p in probs:
        M, N, K, G = p["M"], p["N"], p["K"], p["G"]
        got = p["y"].read(M * N * 4, np.float32).reshape(M, N)
        assert np.all(p["y"].read_bytes(M * N * 4, 4096, np.float32) == -9999.0), "wrote past the output"
        assert_close(got, oracle.w4a16_gemm(p["a"], p["packed"], p["scales"], p["zeros"], M, N, K, G), K)
        batch_out.append(got)
    # the same list again: where a band is cut between CTAs depends on the list, not on timing, so reruns agree bit for bit
    for p in probs:
        p["y"].zero()
    rt.w4a16_gemm_prepacked_batch(calls)
    rt.synchronize()
    for p, got in zip(probs, batch_out):
        assert np.array_equal(p["y"].read(p["M"] * p["N"] * 4, np.float32).reshape(p["M"], p["N"]), got)
    # and one call at a time (bands are cut elsewhere, so the last bits of a sum may differ: tolerance, not equality)
    for p in probs:
        M, N, K, G = p["M"], p["N"], p["K"], p["G"]
        p["y"].zero()
        rt.w4a16_gemm_prepacked(p["xa"].gpu_addr(), p["pre"].gpu_addr(), p["y"].gpu_addr(), M, N, K, G)
        rt.synchronize()
        assert_close(p["y"].read(M * N * 4, np.float32).reshape(M, N), oracle.w4a16_gemm(p["a"], p["packed"], p["scales"], p["zeros"], M, N, K, G), K)
    for b in bufs:
        b.free()


def test_prepacked_batch_longer_than_one_launch(t0, oracle, rt):
    # 70 problems: the list is cut into launches of at most 32; activations differ per problem, two weight sets alternate
    K, N, G = 1024, 2048, 128
    w = [make_w4(oracle, K, N, G, seed=900 + i) for i in range(2)]
    pres = []
    for packed, scales, zeros in w:
        xp, xs, xz = rt.upload(packed), rt.upload(scales), rt.upload(zeros)
        pres.append(rt.w4_prepack(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), K, N, G))
        rt.synchronize()
        for b in (xp, xs, xz):
            b.free()
    n_prob = 70
    ms = [1 + (i * 7) % 16 for i in range(n_prob)]
    a_host = [oracle.fill_normal_bf16(ms[i] * K, 300 + i) for i in range(n_prob)]
    xas = [rt.upload(a) for a in a_host]
    ys = [rt.alloc(ms[i] * N * 4) for i in range(n_prob)]
    calls = [t0.W4A16Args(xas[i].gpu_addr(), pres[i % 2].gpu_addr(), 0, 0, ys[i].gpu_addr(), ms[i], N, K, G) for i in range(n_prob)]
    before = rt.launch_count()
    rt.w4a16_gemm_prepacked_batch(calls)
    rt.synchronize()
    assert rt.launch_count() - before == 3
    for i in range(n_prob):
        packed, scales, zeros = w[i % 2]
        got = ys[i].read(ms[i] * N * 4, np.float32).reshape(ms[i], N)
        assert_close(got, oracle.w4a16_gemm(a_host[i], packed, scales, zeros, ms[i], N, K, G), K)
    for b in pres + xas + ys:
        b.free()


# ----------------------------------------------------------------------------- K2 for 16 < M <= 128 (tcgen05, dequantisation in the main loop)

@pytest.mark.parametrize("M", [17, 64, 100, 128])
@pytest.mark.parametrize("K,N,G", [(64, 32, 64), (512, 288, 128), (1024, 1024, 256), (4096, 1536, 128), (2048, 11008, 128), (192, 8192, 64)])
def test_fused_large_m_shapes(t0, oracle, rt, M, K, N, G):
    # one launch, no K x N scratch: partial column tiles (N = 32, 288), one to four parts of K per tile, three group sizes
    a = oracle.fill_normal_bf16(M * K, 7 + M)
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=M + K)
    ref = oracle.w4a16_gemm(a, packed, scales, zeros, M, N, K, G)
    before = rt.launch_count()
    got = run_w4a16(rt, a, packed, scales, zeros, M, N, K, G)
    assert rt.launch_count() - before == 1
    assert_close(got, ref, K)


def test_fused_large_m_dequantises_bit_exactly(t0, oracle, rt):
    # one-hot activations: row m of y is row base + m of the dequantised weights, exactly
    K, G, M = 256, 128, 128
    N = 8192
    rng = np.random.default_rng(11)
    packed = rng.integers(0, 2 ** 32, size=(K // 8, N), dtype=np.uint64).astype(np.uint32)
    col = np.arange(N, dtype=np.uint32)
    sbits = np.stack([(0x3A00 + (col % 0x400)).astype(np.uint16) | ((col // 0x400 % 2) << 15).astype(np.uint16),
                      (0x3B80 + (col % 0x300)).astype(np.uint16)])
    zeros = rng.integers(0, 2 ** 32, size=(K // G, N // 8), dtype=np.uint64).astype(np.uint32)
    want = oracle.bf16_to_f32(oracle.dequant_w4_b200(packed, sbits, zeros, K, N, G)).reshape(K, N)
    for base in (0, 128):
        a = np.zeros((M, K), np.uint16)
        for m in range(M):
            a[m, base + m] = 0x3F80
        got = run_w4a16(rt, a, packed, sbits, zeros, M, N, K, G)
        assert np.array_equal(got.view(np.uint32) & 0x7FFFFFFF, want[base:base + M].view(np.uint32) & 0x7FFFFFFF), base


@pytest.mark.parametrize("M,K,N,G,count", [(128, 4096, 1536, 128, 5), (17, 512, 288, 128, 3), (100, 1024, 11008, 256, 4), (64, 192, 8192, 64, 40)])
def test_grouped_large_m_problems_in_one_launch(t0, oracle, rt, M, K, N, G, count):
    # independent problems of one shape (their own activations, weights and outputs) in one launch of the fused tcgen05
    # kernel, K not split: each y against the oracle, the guard words behind each y untouched, one launch per 32 problems;
    # with one-hot activations the result is the dequantised weights, bit for bit
    acts = [oracle.fill_normal_bf16(M * K, 70 + i) for i in range(min(count, 3))]
    w = [make_w4(oracle, K, N, G, seed=M + K + i) for i in range(min(count, 3))]
    bufs, calls, ys = [], [], []
    for i in range(count):
        j = i % len(acts)
        xa, xp, xs, xz = rt.upload(acts[j]), rt.upload(w[j][0]), rt.upload(w[j][1]), rt.upload(w[j][2])
        y = rt.alloc(M * N * 4 + 4096)
        y.write(np.full(M * N + 1024, -9999.0, np.float32))
        calls.append(t0.W4A16Args(xa.gpu_addr(), xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), y.gpu_addr(), M, N, K, G))
        bufs += [xa, xp, xs, xz, y]
        ys.append(y)
    before = rt.launch_count()
    rt.w4a16_gemm_grouped(calls)
    rt.synchronize()
    assert rt.launch_count() - before == -(-count // 32)
    refs = [oracle.w4a16_gemm(acts[j], *w[j], M, N, K, G) for j in range(len(acts))]
    for i, y in enumerate(ys):
        assert_close(y.read(M * N * 4, np.float32).reshape(M, N), refs[i % len(acts)], K)
        assert np.all(y.read_bytes(M * N * 4, 4096, np.float32) == -9999.0), "wrote past the output"
    # dependent problems are refused: the output of one as the activations of another
    if count >= 2 and M * K * 2 <= M * N * 4:
        bad = [calls[0], t0.W4A16Args(ys[0].gpu_addr(), calls[1].packed, calls[1].scales, calls[1].zeros, ys[1].gpu_addr(), M, N, K, G)]
        with pytest.raises(t0.T0Error):
            rt.w4a16_gemm_grouped(bad)
    for b in bufs:
        b.free()


@pytest.mark.parametrize("K,N,G", [(64, 32, 64), (512, 288, 128), (256, 1000, 128), (1024, 11008, 256)])
def test_tiled_layout_conversion_is_bit_exact(t0, oracle, rt, K, N, G):
    # the tile-major layout is an index remap of the row layout: the device conversion against the oracle's, byte for byte
    # (partial last tiles and N that is not a multiple of 8 words of zero points included)
    if N % 8:
        pytest.skip("the row layout itself needs N % 8 == 0")
    packed, scales, zeros = make_w4(oracle, K, N, G, seed=K + N)
    xp, xs, xz = rt.upload(packed), rt.upload(scales), rt.upload(zeros)
    tiled = rt.w4_to_tiled(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), K, N, G)
    rt.synchronize()
    want = oracle.w4_to_tiled(packed, scales, zeros, K, N, G)
    got = tiled.read(len(want), np.uint8)
    assert np.array_equal(got, want)
    for b in (xp, xs, xz, tiled):
        b.free()


@pytest.mark.parametrize("M,K,N,G,count", [(128, 4096, 1536, 128, 5), (17, 512, 288, 128, 3), (100, 1024, 11008, 256, 4), (64, 192, 8200, 64, 40),
                                           (1, 256, 1000, 128, 2), (128, 128, 256, 64, 1)])
def test_tiled_weights_single_and_grouped(t0, oracle, rt, M, K, N, G, count):
    # tile-major weights: one problem per launch (K split over a cluster where that fills the GPU) and up to 32 per launch (K
    # not split, weights as the tensor-memory operand), each y against the oracle, guard words untouched; N with a partial last
    # tile and N that the row-layout kernel would refuse (N % 32 != 0) included
    acts = [oracle.fill_normal_bf16(M * K, 170 + i) for i in range(min(count, 3))]
    w = [make_w4(oracle, K, N, G, seed=M + K + 9 * i) for i in range(min(count, 3))]
    refs = [oracle.w4a16_gemm(acts[j], *w[j], M, N, K, G) for j in range(len(acts))]
    tiled = []
    for j in range(len(acts)):
        xp, xs, xz = rt.upload(w[j][0]), rt.upload(w[j][1]), rt.upload(w[j][2])
        tiled.append(rt.w4_to_tiled(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), K, N, G))
        rt.synchronize()
        for b in (xp, xs, xz):
            b.free()
    xas = [rt.upload(a) for a in acts]
    ys, calls = [], []
    for i in range(count):
        y = rt.alloc(M * N * 4 + 4096)
        y.write(np.full(M * N + 1024, -9999.0, np.float32))
        ys.append(y)
        calls.append(t0.W4A16Args(xas[i % len(acts)].gpu_addr(), tiled[i % len(acts)].gpu_addr(), 0, 0, y.gpu_addr(), M, N, K, G))
    rt.w4a16_gemm_tiled(xas[0].gpu_addr(), tiled[0].gpu_addr(), ys[0].gpu_addr(), M, N, K, G)
    rt.synchronize()
    assert_close(ys[0].read(M * N * 4, np.float32).reshape(M, N), refs[0], K)
    ys[0].write(np.full(M * N + 1024, -9999.0, np.float32))
    before = rt.launch_count()
    rt.w4a16_gemm_tiled_grouped(calls)
    rt.synchronize()
    assert rt.launch_count() - before == -(-count // 32)
    for i, y in enumerate(ys):
        assert_close(y.read(M * N * 4, np.float32).reshape(M, N), refs[i % len(acts)], K)
        assert np.all(y.read_bytes(M * N * 4, 4096, np.float32) == -9999.0), "wrote past the output"
    for b in tiled + xas + ys:
        b.free()


def test_tiled_grouped_dequantises_bit_exactly(t0, oracle, rt):
    # one-hot activations through the grouped launch (weights as the tensor-memory operand): row m of y is row base + m of the
    # dequantised weights, exactly
    K, G, M, N = 256, 128, 128, 2048
    rng = np.random.default_rng(12)
    packed = rng.integers(0, 2 ** 32, size=(K // 8, N), dtype=np.uint64).astype(np.uint32)
    col = np.arange(N, dtype=np.uint32)
    sbits = np.stack([(0x3A00 + (col % 0x400)).astype(np.uint16) | ((col // 0x400 % 2) << 15).astype(np.uint16), (0x3B80 + (col % 0x300)).astype(np.uint16)])
    zeros = rng.integers(0, 2 ** 32, size=(K // G, N // 8), dtype=np.uint64).astype(np.uint32)
    want = oracle.bf16_to_f32(oracle.dequant_w4_b200(packed, sbits, zeros, K, N, G)).reshape(K, N)
    xp, xs, xz = rt.upload(packed), rt.upload(sbits), rt.upload(zeros)
    tiled = rt.w4_to_tiled(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), K, N, G)
    bufs, calls, ys = [xp, xs, xz, tiled], [], []
    for base in (0, 128):
        a = np.zeros((M, K), np.uint16)
        for m in range(M):
            a[m, base + m] = 0x3F80
        xa, y = rt.upload(a), rt.alloc(M * N * 4)
        bufs += [xa, y]
        ys.append(y)
        calls.append(t0.W4A16Args(xa.gpu_addr(), tiled.gpu_addr(), 0, 0, y.gpu_addr(), M, N, K, G))
    rt.w4a16_gemm_tiled_grouped(calls)
    rt.synchronize()
    for base, y in zip((0, 128), ys):
        got = y.read(M * N * 4, np.float32).reshape(M, N)
        assert np.array_equal(got.view(np.uint32) & 0x7FFFFFFF, want[base:base + M].view(np.uint32) & 0x7FFFFFFF), base
    for b in bufs:
        b.free()


def test_tiled_grouped_random_shapes(t0, oracle, rt):
    # a seeded sweep over M (1..128), N (multiples of 8, partial last tiles), K (multiples of the group) and both group sizes of
    # the tile-major entries: every problem of a grouped call against the oracle, the words behind each y untouched
    rng = np.random.default_rng(77)
    for case in range(10):
        G = int(rng.choice([64, 128, 256]))
        M = int(rng.integers(1, 129))
        N = int(rng.integers(1, 160)) * 8
        K = int(rng.integers(1, 9)) * G
        count = int(rng.integers(1, 5))
        w = make_w4(oracle, K, N, G, seed=300 + case)
        xp, xs, xz = rt.upload(w[0]), rt.upload(w[1]), rt.upload(w[2])
        tiled = rt.w4_to_tiled(xp.gpu_addr(), xs.gpu_addr(), xz.gpu_addr(), K, N, G)
        acts = [oracle.fill_normal_bf16(M * K, 900 + 7 * case + i) for i in range(count)]
        xas = [rt.upload(a) for a in acts]
        ys = [rt.alloc(M * N * 4 + 4096) for _ in range(count)]
        for y in ys:
            y.write(np.full(M * N + 1024, -9999.0, np.float32))
        rt.w4a16_gemm_tiled_grouped([t0.W4A16Args(xas[i].gpu_addr(), tiled.gpu_addr(), 0, 0, ys[i].gpu_addr(), M, N, K, G) for i in range(count)])
        rt.synchronize()
        for i in range(count):
            got = ys[i].read((M * N + 1024) * 4, np.float32)
            assert_close(got[:M * N].reshape(M, N), oracle.w4a16_gemm(acts[i], *w, M, N, K, G), K)
            assert np.all(got[M * N:] == -9999.0), ("wrote past the output", case, M, N, K, G)
        for b in [xp, xs, xz, tiled] + xas + ys:
            b.free()

"""The CPU oracle against the reference's golden vectors and known-answer tests (no GPU)."""
import os

import numpy as np
import pytest


def _load(golden_dir, name, dtype):
    return np.fromfile(os.path.join(golden_dir, "torch_ref", name), dtype=dtype)


def test_meta_matches_fixture_shapes(golden_dir):
    meta = dict(l.strip().split("=") for l in open(os.path.join(golden_dir, "torch_ref", "meta.txt")) if "=" in l)
    assert (int(meta["M"]), int(meta["K"]), int(meta["N"])) == (64, 256, 512)
    assert _load(golden_dir, "x.bin", np.uint16).size == 64 * 256
    assert _load(golden_dir, "w_gate.bin", np.uint16).size == 512 * 256
    assert _load(golden_dir, "h_gate_f32ref.bin", np.float32).size == 64 * 512


@pytest.mark.parametrize("w,ref", [("w_gate.bin", "h_gate_f32ref.bin"), ("w_up.bin", "h_up_f32ref.bin")])
def test_gemm_matches_torch_fp32_reference(oracle, golden_dir, w, ref):
    # benchmarks/gen_torch_ref.py:98-99: torch.mm(X.float(), W.float().T); thresholds of
    # src/t0/precision_vs_torch.rs:302-305 are 0.05; sequential fp32 summation agrees to ~1e-6
    x = _load(golden_dir, "x.bin", np.uint16)
    wt = _load(golden_dir, w, np.uint16)
    want = _load(golden_dir, ref, np.float32).reshape(64, 512)
    got = oracle.gemm_nt(x, wt, 64, 256, 512)
    assert np.abs(got - want).max() < 2e-6
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-6


def test_second_gemm_matches_torch(oracle, golden_dir):
    s = _load(golden_dir, "swiglu_bf16_trunc.bin", np.uint16)
    wd = _load(golden_dir, "w_down.bin", np.uint16)
    want = _load(golden_dir, "y_bf16_f32acc.bin", np.float32).reshape(64, 256)
    got = oracle.gemm_nt(s, wd, 64, 512, 256)
    assert np.abs(got - want).max() < 2e-6


def test_bf16_output_variant_matches_torch_bf16_matmul(oracle, golden_dir):
    # h_gate_bf16acc = torch.mm(X, W.T) in bf16: RNE of an fp32-accumulated sum up to summation order
    x = _load(golden_dir, "x.bin", np.uint16)
    wt = _load(golden_dir, "w_gate.bin", np.uint16)
    want = _load(golden_dir, "h_gate_bf16acc.bin", np.float32).reshape(64, 512)
    got = oracle.bf16_to_f32(oracle.f32_to_bf16_rne(oracle.gemm_nt(x, wt, 64, 256, 512))).reshape(64, 512)
    ulp = np.maximum(np.abs(want), 2.0 ** -126) * 2.0 ** -7
    assert np.all(np.abs(got - want) <= ulp)          # at most one bf16 ulp apart
    assert np.mean(got == want) > 0.99


def test_gemm_is_bit_exact_against_scalar_loop(oracle):
    # the blocked/vectorised oracle must give the bits of the plain triple loop (tile_ir.rs:5021-5038)
    m, k, n = 7, 53, 37
    a = oracle.fill_uniform_bf16(m * k, 1)
    b = oracle.fill_uniform_bf16(n * k, 2)
    af = oracle.bf16_to_f32(a).reshape(m, k)
    bf = oracle.bf16_to_f32(b).reshape(n, k)
    want = np.zeros((m, n), np.float32)
    for i in range(m):
        for j in range(n):
            s = np.float32(0)
            for kk in range(k):
                s = np.float32(s + np.float32(af[i, kk] * bf[j, kk]))
            want[i, j] = s
    assert np.array_equal(oracle.gemm_nt(a, b, m, k, n), want)
    assert np.array_equal(oracle.gemm_nn(a, np.ascontiguousarray(b.reshape(n, k).T), m, k, n), want)
    assert np.array_equal(oracle.gemm_nt(a, b, m, k, n, threads=1), oracle.gemm_nt(a, b, m, k, n, threads=5))


def test_known_answer_patterns(oracle):
    # all-ones (examples/hello_gemm_gen.rs:85-146): every output equals K
    m, k, n = 32, 96, 48
    ones = np.full(m * k, 0x3F80, np.uint16)
    assert np.all(oracle.gemm_nt(ones, np.full(n * k, 0x3F80, np.uint16), m, k, n) == k)
    # small integers (tile_ir.rs:5056-5059; auto_gemm.rs:235-238; full_matrix_check.rs:96-97): exact in any order
    for (fa, fb) in [(lambda i: i % 17 - 8, lambda i: i % 13 - 6), (lambda i: i % 7 - 3, lambda i: i % 5 - 2),
                     (lambda i: 1 + i % 3, lambda i: 1 + i % 2)]:
        a = fa(np.arange(m * k)).astype(np.float32)
        b = fb(np.arange(n * k)).astype(np.float32)
        want = a.reshape(m, k).astype(np.float64) @ b.reshape(n, k).astype(np.float64).T
        got = oracle.gemm_nt(oracle.f32_to_bf16_trunc(a), oracle.f32_to_bf16_trunc(b), m, k, n)
        assert np.array_equal(got.astype(np.float64), want)


def test_bf16_conversions(oracle):
    L = oracle.lib()
    # tests/tile_gemm_contract.rs:137-154 (truncation semantics)
    assert L.oracle_f32_to_bf16_trunc(1.0) == 0x3F80
    assert L.oracle_f32_to_bf16_trunc(-1.0) == 0xBF80
    assert L.oracle_f32_to_bf16_trunc(0.0) == 0
    assert L.oracle_f32_to_bf16_trunc(float("inf")) == 0x7F80
    over = np.array([0x3F8000FF], np.uint32).view(np.float32)[0]
    assert L.oracle_f32_to_bf16_trunc(float(over)) == 0x3F80
    for bits in (0x3F80, 0xBF80, 0x007F, 0x8000):
        assert L.oracle_f32_to_bf16_trunc(L.oracle_bf16_to_f32(bits)) == bits
    # examples/test_gemm_correctness.rs:15-20 (round to nearest even)
    assert L.oracle_f32_to_bf16_rne(float(over)) == 0x3F80
    tie_even = np.array([0x3F808000], np.uint32).view(np.float32)[0]
    tie_odd = np.array([0x3F818000], np.uint32).view(np.float32)[0]
    assert L.oracle_f32_to_bf16_rne(float(tie_even)) == 0x3F80
    assert L.oracle_f32_to_bf16_rne(float(tie_odd)) == 0x3F82
    import torch
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16_rne(x), want)


def test_split_k_planes_sum(oracle):
    m, k, n, sk = 16, 256, 24, 4
    a = oracle.fill_uniform_bf16(m * k, 3)
    b = oracle.fill_uniform_bf16(n * k, 4)
    planes, ysum = oracle.gemm_nt_splitk(a, b, m, k, n, sk)
    for s in range(sk):
        ak = a.reshape(m, k)[:, s * 64:(s + 1) * 64]
        bk = b.reshape(n, k)[:, s * 64:(s + 1) * 64]
        assert np.array_equal(planes[s], oracle.gemm_nt(ak, bk, m, 64, n))
    acc = np.zeros((m, n), np.float32)
    for s in range(sk):
        acc = acc + planes[s]
    assert np.array_equal(ysum, acc)
    full = oracle.gemm_nt(a, b, m, k, n)
    assert np.abs(ysum - full).max() < 1e-4


def test_int4_known_answers(oracle):
    # quant_kernels.rs:347-354,441-448: 0xAB -> lo 11, hi 10; 0xD7 -> 7, 13
    packed = np.array([0xAB, 0xD7], np.uint8)
    out = oracle.dequant_int4_ref(packed, np.array([1.0], np.float32), np.array([0], np.int32), 1, 4, 7)
    assert out.ravel().tolist() == [11.0, 10.0, 7.0, 13.0]
    # :365-372: (12 - 8) * 0.5 = 2.0
    out = oracle.dequant_int4_ref(np.array([0x0C], np.uint8), np.array([0.5], np.float32), np.array([8], np.int32), 1, 2, 7)
    assert out.ravel()[0] == 2.0
    # :458-469: element 200 with group 128 uses group 1
    packed = np.full(128, 0x11, np.uint8)
    out = oracle.dequant_int4_ref(packed, np.array([1.0, 3.0], np.float32), np.array([0, 0], np.int32), 1, 256, 7)
    assert out.ravel()[127] == 1.0 and out.ravel()[200] == 3.0
    # bf16 variant truncates (quant_kernels.rs:167-168)
    s = np.array([0.3], np.float32)
    o16 = oracle.dequant_int4_ref(np.array([0x07], np.uint8), s, np.array([0], np.int32), 1, 2, 7, bf16=True)
    assert o16.ravel()[0] == (np.array([7.0 * 0.3], np.float32).view(np.uint32)[0] >> 16)


def test_gptq_wire_format(oracle):
    # quant_kernels.rs:385-422,472-481
    rows = cols = group = 16
    raw = (np.array([rows, cols, group], "<u4").tobytes() + bytes([0xAB]) * 128 +
           np.full(16, 1.0, "<f4").tobytes() + np.full(16, 8, "<i4").tobytes())
    g = oracle.gptq_parse(raw)
    assert (g["rows"], g["cols"], g["group_size"], g["n_groups"]) == (16, 16, 16, 1)
    assert g["packed"].size == 128 and np.all(g["scales"] == 1.0) and np.all(g["zero_points"] == 8)
    assert g["packed"].size + g["scales"].size * 4 + g["zero_points"].size * 4 == 256
    with pytest.raises(ValueError):
        oracle.gptq_parse(raw[:100])


def test_b200_layout_dequant_agrees_with_reference_format(oracle):
    # the same weights in the reference container and in the B200 layout dequantise to the same values
    rng = np.random.default_rng(5)
    N, K, G = 24, 256, 128
    q = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8).ravel()
    scales = oracle.bf16_to_f32(oracle.fill_range_bf16(N * (K // G), 1, 0.001, 0.02))
    zps = rng.integers(0, 16, size=N * (K // G)).astype(np.int32)
    ref = oracle.dequant_int4_ref(packed, scales, zps, N, K, 7)              # [N, K] f32
    p, s, z, inexact = oracle.gptq_to_b200(packed, scales, zps, N, K, G)
    assert inexact == 0
    w = oracle.bf16_to_f32(oracle.dequant_w4_b200(p, s, z, K, N, G)).reshape(K, N)
    assert np.array_equal(w, oracle.bf16_to_f32(oracle.f32_to_bf16_rne(ref)).reshape(N, K).T)


def test_w4a16_gemm_is_dequant_then_gemm(oracle):
    M, N, K, G = 3, 40, 256, 128
    a = oracle.fill_normal_bf16(M * K, 7)
    p = oracle.fill_u32((K // 8) * N, 8)
    s = oracle.fill_range_bf16((K // G) * N, 9, 0.001, 0.02)
    z = oracle.fill_u32((K // G) * ((N + 7) // 8), 10)
    w = oracle.dequant_w4_b200(p, s, z, K, N, G)
    assert np.array_equal(oracle.w4a16_gemm(a, p, s, z, M, N, K, G), oracle.gemm_nn(a, w, M, K, N))
    # exhaustive: (q - z) * s in fp32 then RNE equals a bf16 x bf16 product rounded once, for every (q, z)
    sv = oracle.bf16_to_f32(np.arange(0x3A00, 0x3D00, dtype=np.uint16))
    for qz in range(-15, 16):
        exact = (np.float64(qz) * sv.astype(np.float64)).astype(np.float32)
        assert np.array_equal(exact.astype(np.float64), np.float64(qz) * sv.astype(np.float64))


def test_generators_are_counter_based(oracle):
    a = oracle.fill_uniform_bf16(1000, 42)
    assert np.array_equal(a[100:200], oracle.fill_uniform_bf16(100, 42, 100))
    f = oracle.bf16_to_f32(a)
    assert f.min() >= -1.0 and f.max() <= 1.0 and abs(float(f.mean())) < 0.1
    s = oracle.bf16_to_f32(oracle.fill_range_bf16(1000, 3, 0.001, 0.02))
    assert s.min() >= 0.001 * 0.99 and s.max() <= 0.02 * 1.01
    nrm = oracle.bf16_to_f32(oracle.fill_normal_bf16(20000, 5))
    assert abs(float(nrm.mean())) < 0.05 and abs(float(nrm.std()) - 1.0) < 0.05


def test_epilogues(oracle):
    y = np.array([[-2.0, 0.5, 3.0]], np.float32)
    bias = np.array([1.0, -1.0, 0.0], np.float32)
    assert oracle.epilogue_gemm_gen(y, bias, 1).tolist() == [[-1.0, -0.5, 3.0]]
    assert oracle.epilogue_gemm_gen(y, bias, 2).tolist() == [[0.0, 0.0, 3.0]]
    silu = oracle.epilogue_tile(y, ["silu"])
    assert np.allclose(silu, y / (1 + np.exp(-y)), rtol=1e-6)
    gelu = oracle.epilogue_tile(y, ["gelu"])
    assert np.allclose(gelu, y / (1 + np.exp(-1.702 * y)), rtol=1e-6)
    assert oracle.epilogue_tile(y, ["neg", "abs", "scale", "clamp"], scale=2.0, clamp_min=0.5, clamp_max=5.0).tolist() == [[4.0, 1.0, 5.0]]

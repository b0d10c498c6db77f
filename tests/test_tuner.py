"""Autotuner: cache file format and helpers on CPU (src/t0/auto_gemm.rs:627-651,751-780), tuning on the GPU (:662-747)."""
import json
import os

import numpy as np
import pytest


def test_parse_json_helpers(t0):
    # auto_gemm.rs:628-637
    js = '{"tile_m":128,"tile_n":64,"tile_k":32,"wg_size":128,"tflops":79.21,"split_k":1}'
    assert t0.parse_json_number(js, "tile_m") == 128
    assert t0.parse_json_number(js, "tile_n") == 64
    assert t0.parse_json_number(js, "tile_k") == 32
    assert t0.parse_json_number(js, "wg_size") == 128
    assert t0.parse_json_number(js, "split_k") == 1
    assert abs(t0.parse_json_number(js, "tflops") - 79.21) < 0.01
    assert t0.parse_json_number(js, "missing") is None


def test_tuner_new_defaults(t0, monkeypatch):
    # auto_gemm.rs:640-650
    monkeypatch.delenv("T0_TUNE_DIR", raising=False)
    t = t0.GemmTuner()
    assert t.max_candidates == 8 and t.n_iters == 5 and t.cache_len() == 0
    assert "t0_autotune" in t.cache_dir
    t.configure(max_candidates=3)
    assert t.max_candidates == 3 and t.n_iters == 5
    t.free()
    monkeypatch.setenv("T0_TUNE_DIR", "/tmp/t0_env_dir")
    t = t0.GemmTuner()
    assert t.cache_dir == "/tmp/t0_env_dir"
    t.free()


def test_cache_roundtrip(t0, tmp_path):
    # auto_gemm.rs:751-780
    d = str(tmp_path / "t0_autotune_cache_test")
    t = t0.GemmTuner.with_cache_dir(d)
    cfg = t0.GemmConfig.tile_128x64_k32()
    t.save_cache(4096, 4096, 4096, cfg, 79.2)
    path = os.path.join(d, "gemm_4096x4096x4096.json")
    raw = json.loads(open(path).read())     # the file is plain JSON with the reference's keys
    assert raw["tile_m"] == 128 and raw["tile_n"] == 64 and raw["tile_k"] == 32 and raw["wg_size"] == 128
    assert raw["split_k"] == 1 and raw["wgp"] is True and raw["swap"] is True and abs(raw["tflops"] - 79.2) < 0.01
    assert raw["all"][0] == [cfg.name(), 79.2]
    loaded, tf = t.load_cache(4096, 4096, 4096)
    assert (loaded.tile_m, loaded.tile_n, loaded.tile_k) == (128, 64, 32) and abs(tf - 79.2) < 0.1
    assert loaded.name() == cfg.name()
    pair = t0.auto_select(4096, 4096, 4096)
    t.save_cache(8192, 8192, 8192, pair.copy(split_k=2), 1400.0)
    loaded, _ = t.load_cache(8192, 8192, 8192)
    assert loaded.name() == pair.copy(split_k=2).name()
    t.invalidate(4096, 4096, 4096)
    assert not os.path.exists(path)
    with pytest.raises(t0.T0Error):
        t.load_cache(4096, 4096, 4096)
    t.clear()
    assert not os.path.exists(d)
    t.free()


@pytest.mark.gpu
def test_tune_small_problem_and_cache_hit(t0, oracle, rt, tmp_path):
    # auto_gemm.rs:662-747 in small: tune, "kernel alive", full compare, cache hit returns the same config
    d = str(tmp_path / "tune")
    t = t0.GemmTuner.with_cache_dir(d)
    t.configure(max_candidates=4, n_iters=3)
    m, n, k = 512, 1024, 512
    cfg = t.tune(rt, m, n, k)
    res = t.result(m, n, k)
    assert res["best_tflops"] > 1.0 and not res["from_cache"] and 1 <= res["n_measured"] <= 4
    assert os.path.exists(os.path.join(d, f"gemm_{m}x{n}x{k}.json"))
    assert t.tune(rt, m, n, k).name() == cfg.name()            # memory cache
    t2 = t0.GemmTuner.with_cache_dir(d)
    assert t2.tune(rt, m, n, k).name() == cfg.name()           # disk cache
    assert t2.result(m, n, k)["from_cache"]
    t.free(); t2.free()


@pytest.mark.gpu
def test_auto_gemm_one_shot(t0, oracle, rt, tmp_path, monkeypatch):
    # auto_gemm.rs:555-590,699-740: 128x64x128 full compare, max_err < 0.05 there, the GEMM tolerance here
    monkeypatch.setenv("T0_TUNE_DIR", str(tmp_path / "global"))
    m, n, k = 128, 64, 128
    a = oracle.f32_to_bf16_trunc((np.arange(m * k) % 7 - 3).astype(np.float32))
    b = oracle.f32_to_bf16_trunc((np.arange(n * k) % 5 - 2).astype(np.float32))
    xa, xb, y = rt.upload(a), rt.upload(b), rt.alloc_zero(m * n * 4 * 8)
    tf = t0.auto_gemm(rt, xa, xb, y, m, n, k)
    assert tf > 0.0
    assert np.array_equal(rt.read_f32(y, m * n).reshape(m, n), oracle.gemm_nt(a, b, m, k, n))
    assert t0.auto_gemm(rt, xa, xb, y, m, n, k) == tf          # cache hit: same tuned figure
    t0.global_tuner().invalidate(m, n, k)


@pytest.mark.gpu
def test_benchmark_tile_ir(t0, rt, tmp_path):
    # auto_gemm.rs:352-431: one TileGemm spec timed through the TileIR kernargs / grid / dispatch path
    t = t0.GemmTuner.with_cache_dir(str(tmp_path / "tune"))
    spec = t0.tile_auto_select(1024, 1024, 1024)
    tf = t.benchmark_tile_ir(rt, spec, 1024, 1024, 1024)
    assert tf > 1.0
    assert not rt.is_poisoned()
    t.free()

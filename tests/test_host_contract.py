"""CPU-only contract tests for the host helpers, after the reference's tests/tile_gemm_contract.rs,
src/t0/gemm_gen.rs:572-662 and src/t0/prefill_spec_cache.rs:143-218.  They go through the C ABI."""
import struct

import pytest

ALL_TILE_PRESETS = ["tile_32x64_k16", "tile_64x64_k16", "tile_64x64_k32", "tile_64x64_k64", "tile_32x128_k16",
                    "tile_128x64_k16", "tile_128x64_k32", "tile_128x64_k64", "tile_64x128_k16", "tile_64x128_k32",
                    "tile_128x128_k16", "tile_128x128_k32", "tile_128x128_k48", "tile_128x128_k64",
                    "tile_128x128_k16_swap", "tile_128x128_k32_swap", "tile_256x64_k32_wgp", "tile_256x64_k64_wgp",
                    "tile_32x32_k16", "tile_128x32_k16", "tile_64x256_k32", "tile_128x256_k32"]


def test_preset_dimension_identities(t0):
    # tests/tile_gemm_contract.rs:44-58
    for name in ALL_TILE_PRESETS:
        spec = t0.TileGemm.preset(name)
        n_waves = spec.waves_per_wg or spec.tile_m // 32
        rpw = spec.tile_m // n_waves
        assert spec.wg_size() == n_waves * 32, name
        assert spec.n_row_blocks() == rpw // 16
        assert spec.rows_per_wave() == rpw
        assert spec.k_sub_steps() == spec.tile_k // 16
        assert rpw % 16 == 0


def test_tile_lds_total_formulas(t0):
    # tests/tile_gemm_contract.rs:63-69,191-242
    spec = t0.TileGemm.tile_256x64_k32_wgp()
    assert spec.copy(double_buffer=1, triple_buffer=0).lds_total() == 40960
    assert spec.copy(triple_buffer=1).lds_total() == 61440
    assert spec.copy(double_buffer=0, triple_buffer=1).lds_total() == 61440
    forbidden = [n for n in ALL_TILE_PRESETS if t0.TileGemm.preset(n).copy(triple_buffer=1).lds_total() > 65536]
    assert "tile_128x64_k64" in forbidden
    for name in ALL_TILE_PRESETS:
        s = t0.TileGemm.preset(name)
        if not s.acc_swap:
            assert s.lds_total() == s.lds_per_buffer() * (2 if s.double_buffer else 1)


def test_grid_coverage_enumeration(t0):
    # tests/tile_gemm_contract.rs:74-93
    dims = [1, 31, 32, 33, 63, 64, 127, 128, 255, 256, 4095, 4096]
    for cfg in (t0.GemmConfig.tile_128x64_k16(), t0.GemmConfig.tile_128x64_k32(), t0.GemmConfig.tile_64x64_k32(),
                t0.auto_select(4096, 4096, 4096).copy(split_k=0)):
        for m in dims:
            for n in dims:
                gx, gy = t0.compute_grid_auto(cfg, m, n)
                assert gx % cfg.wg_size == 0
                tiles_m = -(-m // cfg.tile_m)
                tiles_n = -(-n // cfg.tile_n)
                assert gy == tiles_m
                assert gx // cfg.wg_size == tiles_n
                assert tiles_n * cfg.tile_n >= n and tiles_m * cfg.tile_m >= m


def test_grid_swap_and_split(t0):
    cfg = t0.GemmConfig.tile_128x64_k16()
    assert t0.compute_grid(cfg, 4096, 4096) == (64 * 128, 32)            # gemm_gen.rs:308-316
    assert t0.compute_grid(cfg.copy(swap_grid=0), 4096, 2048) == (32 * 128, 32)
    assert t0.compute_grid_split_k(cfg, 256, 128, 4) == (2 * 128, 2 * 4)  # gemm_gen.rs:319-329
    assert t0.compute_grid_auto(cfg.copy(split_k=2), 256, 128) == (256, 4)
    with pytest.raises(t0.T0Error):
        t0.compute_grid_split_k(cfg, 256, 128, 3)                         # assert!(is_power_of_two)
    with pytest.raises(t0.T0Error):
        t0.compute_grid_split_k(cfg, 256, 128, 0)


def test_build_kernargs_m_field_layout(t0):
    # tests/tile_gemm_contract.rs:99-115
    spec = t0.TileGemm.tile_64x64_k16().copy(split_k=4)
    ka = t0.tile_build_kernargs_m(0xA000, 0xB000, 0xC000, 64, 128, 32, spec)
    assert len(ka) == 44
    x, wt, y, k, n, shift, stride, m = struct.unpack("<QQQIIIII", ka)
    assert (x, wt, y, k, n, shift, stride, m) == (0xA000, 0xB000, 0xC000, 64, 128, 2, 0, 32)
    for sk, sh in [(1, 0), (2, 1), (8, 3), (16, 4), (3, 0)]:
        assert struct.unpack_from("<I", t0.tile_build_kernargs_m(1, 2, 3, 4, 5, 6, spec.copy(split_k=sk)), 32)[0] == sh
    # persistent specs pad to 64 bytes (tile_ir.rs:4623-4632)
    assert len(t0.tile_build_kernargs_m(1, 2, 3, 4, 5, 6, t0.TileGemm.tile_persistent_decode())) == 64
    # epilogue arguments follow M: bias pointer 8-aligned, then scale, clamp_min, clamp_max (tile_ir.rs:1015-1026)
    spec = t0.TileGemm.tile_128x64_k16().with_epilogue(["bias", "scale", "clamp"])
    ka = t0.tile_build_kernargs_epilogue(1, 2, 3, 4, 5, 6, spec, bias=0xD000, scale=0.5, clamp_min=-1.0, clamp_max=2.0)
    assert len(ka) == 68
    assert struct.unpack_from("<Q", ka, 48)[0] == 0xD000
    assert struct.unpack_from("<fff", ka, 56) == (0.5, -1.0, 2.0)


def test_gemm_build_kernargs_split_stride_semantics(t0):
    # tests/tile_gemm_contract.rs:120-131
    cfg = t0.GemmConfig.tile_128x64_k16().copy(split_k=0)
    ka1 = t0.build_kernargs(1, 2, 3, 64, 64, 64, cfg)
    assert len(ka1) == 40 and struct.unpack_from("<I", ka1, 36)[0] == 0
    ka2 = t0.build_kernargs(1, 2, 3, 64, 64, 256, cfg.copy(split_k=2))
    assert struct.unpack_from("<I", ka2, 36)[0] == 256 * 64 * 4
    assert struct.unpack("<QQQIIII", ka2)[:6] == (1, 2, 3, 64, 64, 0)   # K@24 N@28 split_k_shift always 0


def test_kernargs_with_bias_layout(t0):
    # gemm_gen.rs:651-661
    ka = t0.build_kernargs_with_bias(0x1000, 0x2000, 0x3000, 64, 64, 128, t0.GemmConfig.tile_32x64_k16(), 0x4000)
    assert len(ka) == 48 and struct.unpack_from("<Q", ka, 40)[0] == 0x4000


def test_f32_to_bf16_truncation_semantics(t0):
    # tests/tile_gemm_contract.rs:137-154
    f = t0.f32_to_bf16
    assert f(1.0) == 0x3F80 and f(-1.0) == 0xBF80 and f(0.0) == 0
    assert f(float("inf")) == 0x7F80 and f(float("-inf")) == 0xFF80
    over = struct.unpack("<f", struct.pack("<I", 0x3F8000FF))[0]
    assert f(over) == 0x3F80
    for bits in (0x3F80, 0xBF80, 0x007F, 0x8000):
        assert f(t0.bf16_to_f32(bits)) == bits


def test_auto_select_domain_sample_feasible(t0):
    # tests/tile_gemm_contract.rs:167-180
    n = 0
    for m in (16, 31, 64, 128, 256, 1024, 4096):
        for nn in (32, 64, 128, 256, 4096):
            for k in (16, 32, 64, 256, 4096):
                cfg = t0.auto_select(m, k, nn)
                assert cfg.is_feasible(), (m, k, nn, cfg.name())
                sk = cfg.split()
                assert k % sk == 0
                n += 1
    assert n >= 100


def test_auto_select_sizes(t0):
    # gemm_gen.rs:577-603, with the B200 tile table
    c = t0.auto_select(256, 256, 256)
    assert 16 <= c.tile_m <= 256 and c.wg_size >= 32
    c = t0.auto_select(1024, 1024, 1024)
    assert c.tile_m >= 64
    c = t0.auto_select(8192, 8192, 8192)
    assert c.tile_m >= 64 and c.tile_n >= 128
    c = t0.auto_select(128, 4096, 4096)
    assert 128 % c.tile_m == 0
    # a skinny, bandwidth-bound shape wants many CTAs: narrow tiles or, as measured best on B200 (18.8 us against 23.1),
    # 128-wide tiles with the contraction split four ways
    assert c.tile_n <= 64 or c.split() >= 2
    # every selected tile is one the sm_100a kernel implements
    for (m, k, n) in [(4096, 4096, 4096), (2048, 2048, 2048), (64, 16384, 4096), (1, 4096, 11008)]:
        c = t0.auto_select(m, k, n)
        assert c.tile_k == 64
        if c.tile_m == 256:      # the CTA pair: 256 x 256 over two SMs
            assert c.wgp_mode and c.tile_n == 256
        else:
            assert c.tile_m == 128 and c.tile_n in (32, 64, 128, 256)
    assert t0.auto_select(4096, 4096, 4096).name() == "t0_gemm_256x256_k64_ldsdb_wgp"


def test_auto_select_legacy_preserved(t0):
    # gemm_gen.rs:606-615
    c = t0.auto_select_legacy(256, 256, 256)
    assert c.split() > 1 and c.tile_m == 64
    c = t0.auto_select_legacy(1024, 1024, 1024)
    assert c.tile_m == 128 and c.wgp_mode
    c = t0.auto_select_legacy(4096, 4096, 4096)
    assert (c.tile_m, c.tile_n, c.tile_k, c.split()) == (128, 64, 32, 2)
    c = t0.auto_select_legacy(128, 4096, 4096)
    assert (c.tile_m, c.swap_grid, c.split()) == (128, 0, 4)
    c = t0.auto_select_legacy(100, 64, 100)
    assert c.tile_m == 64 or c.tile_m == 32


def test_config_names(t0):
    # gemm_gen.rs:215-235,622-633
    cfg = t0.GemmConfig.tile_32x64_k16()
    assert cfg.name() == "t0_gemm_32x64_k16_ldsdb_wgp"
    assert cfg.copy(epilogue=t0.EPI_BIAS_ADD_STORE_F32).name().endswith("_bias")
    assert cfg.copy(epilogue=t0.EPI_BIAS_ADD_RELU_STORE_F32).name().endswith("_bias_relu")
    assert t0.GemmConfig.tile_32x64_direct().name() == "t0_gemm_32x64_k16_direct_wgp"
    assert t0.GemmConfig.tile_128x128_2pass().copy(split_k=4, swap_grid=0, wgp_mode=0, transpose=t0.NN).name() == \
        "t0_gemm_128x64_k16_ldsdb_sk4_2p_mg_nn"
    # tile_ir.rs:677-701
    s = t0.TileGemm.tile_128x128_k32()
    assert s.name() == "tile_gemm_128x128_k32_wgp_swap"
    assert t0.TileGemm.tile_64x64_k16().copy(split_k=4).name() == "tile_gemm_64x64_k16_db_sk4"
    assert t0.TileGemm.tile_128x64_k16().with_epilogue(["bias", "silu"]).name() == "tile_gemm_128x64_k16_db_bias_silu"
    assert t0.TileGemm.tile_persistent_decode().name() == "tile_gemm_32x64_k16_db_mg_persistent"
    with pytest.raises(t0.T0Error):
        t0.GemmConfig.preset("tile_7x7_k7")


def test_estimated_vgprs_formula(t0):
    # gemm_gen.rs:189-201 for 128x64 k32, wg 128: acc 2*4*8 + x_frag 16 + wt_frag 32 + gmem 16 + 8 + temps 49
    assert t0.GemmConfig.tile_128x64_k32().estimated_vgprs() == 185
    assert t0.GemmConfig.tile_64x64_k16().is_feasible()
    assert not t0.GemmConfig.tile_64x64_k16().copy(tile_m=0).is_feasible()
    assert not t0.GemmConfig.tile_64x64_k16().copy(split_k=3).is_feasible()


def test_tile_auto_select_table(t0):
    # tile_ir.rs:740-870
    assert t0.tile_auto_select(4096, 4096, 4096).name() == "tile_gemm_128x128_k64_db_swap"
    assert t0.tile_auto_select(2048, 2048, 2048).name() == "tile_gemm_256x64_k32_db_wgp"
    assert t0.tile_auto_select(1024, 1024, 1024).name() == "tile_gemm_64x64_k32_db"
    assert t0.tile_auto_select(16, 64, 512).name() == "tile_gemm_64x256_k32_db"
    assert t0.tile_auto_select(8, 16, 8).name() == "tile_gemm_32x32_k16_db"
    assert t0.tile_auto_select(512, 48, 16).name() == "tile_gemm_128x32_k16_db"
    s = t0.tile_auto_select(4096, 4096, 4096, t0.NN)
    assert s.transpose == t0.NN and s.split_k == 1        # auto split-K stays disabled (tile_ir.rs:852-867)


def test_tile_compute_grid(t0):
    # tile_ir.rs:4645-4665
    s = t0.TileGemm.tile_128x64_k16()
    assert t0.tile_compute_grid(s, 1000, 512) == [8 * 128, 8, 1]
    assert t0.tile_compute_grid(s.copy(swap_grid=0, split_k=2), 1000, 512) == [8 * 128, 16, 1]
    assert t0.tile_compute_grid(t0.TileGemm.tile_persistent_decode(), 1000, 512) == [32, 1, 1]


def test_spec_cache(t0):
    # prefill_spec_cache.rs:143-218
    t0.clear_cache()
    assert t0.cache_size() == 0
    a = t0.cached_auto_select(512, 4096, 11008)
    assert t0.cache_size() == 1
    b = t0.cached_auto_select(512, 4096, 11008)
    assert t0.cache_size() == 1 and a.name() == b.name() == t0.auto_select(512, 4096, 11008).name()
    t0.prewarm_cache([(1, 4096, 4096), (1, 4096, 11008), (512, 4096, 4096), (512, 4096, 11008)])
    assert t0.cache_size() == 4
    t0.clear_cache()
    assert t0.cache_size() == 0


def test_sweep_and_standard_lists(t0):
    import ctypes as C
    arr = (t0.GemmConfig * 32)()
    assert t0.lib().t0_sweep_configs(arr, 32) == 9                    # gemm_gen.rs:239-251
    assert arr[0].tile_m == 16 and arr[8].tile_k == 32
    assert t0.lib().t0_standard_configs(arr, 32) == 16                # gemm_gen.rs:407-427
    assert [arr[i].split_k for i in range(8, 16)] == [2, 4, 2, 4, 4, 8, 2, 2]


def test_backward_helpers(t0):
    # gemm_gen.rs:510-570
    cfg = t0.GemmConfig.tile_64x64_k16()
    out = (__import__("ctypes").c_uint8 * 40)()
    t0.lib().t0_build_kernargs_backward_data(1, 2, 3, 10, 20, 30, cfg, out)
    assert struct.unpack_from("<II", bytes(out), 24) == (20, 30)      # K = n_orig, N = k_orig
    t0.lib().t0_build_kernargs_backward_weight(1, 2, 3, 10, 20, 30, cfg, out)
    assert struct.unpack_from("<II", bytes(out), 24) == (10, 30)      # K = m, N = k_orig


def test_no_gpu_means_loud_failure(t0):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(t0.T0Error) as e:
        t0.GpuRuntime(0)
    assert "no CPU fallback" in str(e.value)


def test_warp_layout_planners(t0):
    # the reference's own known answers: src/t0/tile_ir.rs:8552-8618
    l = t0.WarpLayout.row_dominant(4, 128, 64)
    assert (l.n_warps, l.rows_per_warp, l.cols_per_warp) == (4, 32, 64)
    assert (l.wmma_row_blocks(), l.wmma_col_tiles(), l.wmma_ops_per_warp(), l.acc_vgprs_per_warp()) == (2, 4, 8, 64)
    assert l.wg_size() == 128 and l.is_compatible(128, 64) and not l.is_compatible(48, 64)
    l = t0.WarpLayout.col_dominant(4, 64, 128)
    assert (l.rows_per_warp, l.cols_per_warp, l.wmma_ops_per_warp()) == (64, 32, 8)
    l = t0.WarpLayout.square(4, 128, 128)
    assert (l.rows_per_warp, l.cols_per_warp, l.wmma_ops_per_warp()) == (64, 64, 16)
    qk, av = t0.plan_flash_attention_warps(4, 128, 64, 64)
    assert qk.orientation == t0.WarpLayout.ROW_DOMINANT and av.orientation == t0.WarpLayout.COL_DOMINANT
    qk, av = t0.plan_flash_attention_warps(4, 16, 64, 64)          # decode: one warp of 16 rows
    assert qk.orientation == t0.WarpLayout.ROW_DOMINANT and qk.n_warps == 1 and qk.rows_per_warp == 16
    l = t0.plan_single_dot_warps(4, 128, 64)
    assert (l.rows_per_warp, l.cols_per_warp) == (32, 64)
    l = t0.plan_single_dot_warps(4, 64, 128)
    assert (l.rows_per_warp, l.cols_per_warp) == (64, 32)
    l = t0.WarpLayout.row_dominant(4, 64, 64)
    assert l.rows_per_warp == 16
    l = t0.WarpLayout.row_dominant(4, 32, 64)                       # fewer warps than asked: each keeps 16 rows
    assert (l.n_warps, l.rows_per_warp) == (2, 16)
    # the reference's asserts become errors
    for bad in (lambda: t0.WarpLayout.row_dominant(9, 128, 64), lambda: t0.WarpLayout.row_dominant(4, 8, 64),
                lambda: t0.WarpLayout.col_dominant(4, 64, 100), lambda: t0.WarpLayout.square(3, 128, 128)):
        with pytest.raises(t0.T0Error):
            bad()


def test_cost_model_records(t0):
    # cost_model.rs:130-168,464-534,578-647: TileConfig / TileCost, the ranked schedule and the conversions
    costs = t0.auto_schedule_gemm(4096, 4096, 4096)
    assert len(costs) >= 4 and all(c.feasible for c in costs)
    assert all(costs[i].score >= costs[i + 1].score - 1e-9 for i in range(len(costs) - 1))      # best first
    best = costs[0]
    assert best.config.to_gemm_config().name() == t0.auto_select(4096, 4096, 4096).name()
    assert best.n_wgs == 16 * 16 and best.lds_bytes > 100 * 1024 and best.bottleneck.decode() == "tensor"
    skinny = t0.auto_schedule_gemm(16, 4096, 4096)[0]
    assert skinny.bottleneck.decode() in ("memory", "parallelism")
    c = t0.TileConfig(tile_m=128, tile_n=64, tile_k=32, waves_per_wg=4, use_lds=1, wgp_mode=1, swap_grid=0, split_k=4, lds_pad=8)
    assert c.name() == "128x64_k32_sk4_mg_wgp_pad8"                    # cost_model.rs:157-163
    g = c.to_gemm_config()
    assert (g.tile_m, g.tile_n, g.tile_k, g.wg_size, g.split_k, g.lds_pad, g.swap_grid, g.wgp_mode) == (128, 64, 32, 128, 4, 8, 0, 1)
    assert g.use_lds and g.double_buffer
    tg = c.to_tile_gemm()
    assert (tg.tile_m, tg.tile_n, tg.tile_k, tg.split_k, tg.swap_grid, tg.double_buffer) == (128, 64, 32, 4, 1, 1)
    assert not c.can_use_tile_ir()                                     # split_k > 1 and swap_grid false
    ok = t0.TileConfig(tile_m=128, tile_n=64, tile_k=32, waves_per_wg=4, use_lds=1, wgp_mode=0, swap_grid=1, split_k=1, lds_pad=0)
    assert ok.can_use_tile_ir()
    assert not t0.TileConfig(tile_m=128, tile_n=64, tile_k=48, waves_per_wg=4, use_lds=1, swap_grid=1, split_k=1).can_use_tile_ir()   # tile_k not a power of two
    assert not t0.TileConfig(tile_m=128, tile_n=64, tile_k=32, waves_per_wg=8, use_lds=1, swap_grid=1, split_k=1).can_use_tile_ir()   # waves != tile_m / 32


def test_int4_wmma_config_constructors(t0):
    # quant_kernels.rs:316-336
    c = t0.Int4WmmaConfig.k16()
    assert (c.tile_m, c.tile_n, c.tile_k) == (16, 16, 16)
    c = t0.Int4WmmaConfig.k32()
    assert (c.tile_m, c.tile_n, c.tile_k) == (16, 16, 32)


def test_force_cfg_switch(t0, monkeypatch):
    # T0_FORCE_CFG pins auto_select / cached_auto_select to one preset, is never cached, and bad values are errors
    free = t0.auto_select(4096, 4096, 4096)
    monkeypatch.setenv("T0_FORCE_CFG", "tile_64x64_k32")
    assert t0.auto_select(4096, 4096, 4096).name() == t0.GemmConfig.preset("tile_64x64_k32").name()
    t0.clear_cache()
    assert t0.cached_auto_select(128, 4096, 4096).name() == t0.GemmConfig.preset("tile_64x64_k32").name()
    assert t0.cache_size() == 0
    monkeypatch.setenv("T0_FORCE_CFG", "tile_128x64_k16:sk4")
    forced = t0.auto_select(64, 16384, 4096)
    assert forced.split() == 4 and forced.tile_m == 128 and forced.tile_n == 64
    monkeypatch.setenv("T0_FORCE_CFG", "tile_128x64_k16:sk3")
    with pytest.raises(t0.T0Error):
        t0.auto_select(64, 16384, 4096)
    monkeypatch.setenv("T0_FORCE_CFG", "no_such_preset")
    with pytest.raises(t0.T0Error):
        t0.auto_select(256, 256, 256)
    monkeypatch.delenv("T0_FORCE_CFG")
    assert t0.auto_select(4096, 4096, 4096).name() == free.name()


def test_gptq_parse_rejects_crafted_headers(t0):
    # sizes come from an untrusted header (quant_kernels.rs:251-286): overflowing or inconsistent ones are errors, not offsets
    def raw(rows, cols, group, payload=b""):
        return struct.pack("<III", rows, cols, group) + payload
    with pytest.raises(t0.T0Error):
        t0.gptq_parse(raw(0xFFFFFFFF, 0xFFFFFFFE, 2))              # rows*cols/2 + params*8 wraps a 64-bit size
    with pytest.raises(t0.T0Error):
        t0.gptq_parse(raw(4, 100, 64, b"\0" * 4096))                # cols not a multiple of the group
    with pytest.raises(t0.T0Error):
        t0.gptq_parse(raw(3, 5, 5, b"\0" * 4096))                   # odd element count: two codes share a byte
    with pytest.raises(t0.T0Error):
        t0.gptq_parse(raw(4, 128, 0, b"\0" * 4096))                 # zero group
    ok = t0.gptq_parse(raw(4, 128, 64, b"\0" * (4 * 128 // 2 + 8 * 8)))
    assert (ok["rows"], ok["cols"], ok["group_size"]) == (4, 128, 64)

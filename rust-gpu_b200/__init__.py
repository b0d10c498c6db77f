"""Host-side mirror of the T0-GPU GEMM API over the t0b200 C ABI (ctypes).

The names follow the reference crate (clearnature/rust-gpu): ``GemmConfig``, ``auto_select``,
``compute_grid_auto``, ``build_kernargs``, ``TileGemm``, ``GpuRuntime``, ``GpuBuffer`` ... so that
tests read like the reference's own.  This module is a binding only: every computation happens in
``lib/libt0b200.so`` (hand-written sm_100a kernels).  There is no CPU fallback — if the library is
missing the import of any compute entry point raises.

The package directory name contains a hyphen; import it with
``importlib.import_module("rust-gpu_b200")``.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# T0B200_LIB names another build of the library (e.g. one compiled with tracing flags); the default is the in-tree build
LIB_PATH = os.environ.get("T0B200_LIB") or os.path.join(_HERE, "lib", "libt0b200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "t0b200.h")

NT, NN = 0, 1
EPI_STORE_F32, EPI_BIAS_ADD_STORE_F32, EPI_BIAS_ADD_RELU_STORE_F32 = 0, 1, 2
TEPI = {"bias": 0, "scale": 1, "relu": 2, "silu": 3, "gelu": 4, "abs": 5, "neg": 6, "clamp": 7}
ERR_NAMES = {0: "OK", 1: "INVALID", 2: "CUDA", 3: "POISONED", 4: "TIMEOUT", 5: "BOUNDS", 6: "UNSUPPORTED", 7: "IO"}


class T0Error(RuntimeError):
    """A failing C-ABI call: the Rust side's ``Err(String)`` / panic."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{ERR_NAMES.get(code, code)}] {message}")
        self.code = code
        self.message = message


def build(force: bool = False) -> str:
    """Compile the CUDA library in-tree (nvcc, sm_100a)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_t0b200_build", os.path.join(_HERE, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(force=force)


_lib = None


def lib() -> C.CDLL:
    """The loaded C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise T0Error(2, f"{LIB_PATH} is missing: build it with `python rust-gpu_b200/build.py` "
                             "(there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise T0Error(rc, lib().t0_last_error().decode())


# --------------------------------------------------------------------------- records

class GemmConfig(C.Structure):
    """``GemmConfig`` (src/t0/gemm_gen.rs:55-84)."""
    _fields_ = [("tile_m", C.c_uint32), ("tile_n", C.c_uint32), ("tile_k", C.c_uint32), ("wg_size", C.c_uint32),
                ("use_lds", C.c_uint8), ("double_buffer", C.c_uint8), ("_pad0", C.c_uint8 * 2),
                ("split_k", C.c_uint32), ("lds_pad", C.c_uint32), ("n_col_passes", C.c_uint32),
                ("swap_grid", C.c_uint8), ("wgp_mode", C.c_uint8), ("transpose", C.c_uint8), ("epilogue", C.c_uint8)]

    @classmethod
    def preset(cls, name: str) -> "GemmConfig":
        c = cls()
        _check(lib().t0_gemm_config_preset(name.encode(), C.byref(c)))
        return c

    def copy(self, **kw) -> "GemmConfig":
        c = GemmConfig.from_buffer_copy(self)
        for k, v in kw.items():
            setattr(c, k, v)
        return c

    def name(self) -> str:
        buf = C.create_string_buffer(128)
        _check(lib().t0_gemm_config_name(C.byref(self), buf, 128))
        return buf.value.decode()

    def is_feasible(self) -> bool:
        return bool(lib().t0_gemm_config_is_feasible(C.byref(self)))

    def estimated_vgprs(self) -> int:
        return int(lib().t0_gemm_config_estimated_vgprs(C.byref(self)))

    def lds_total(self) -> int:
        return int(lib().t0_gemm_config_lds_total(C.byref(self)))

    def split(self) -> int:
        return self.split_k if self.split_k > 1 else 1


for _n in ["tile_16x64_k16", "tile_32x64_direct", "tile_32x64_k16", "tile_32x64_k32", "tile_32x128_k16", "tile_64x64_k16",
           "tile_64x64_k32", "tile_128x64_k16", "tile_64x128_k16", "tile_128x64_k32", "tile_128x128_k16", "tile_64x64_k64",
           "tile_128x128_2pass", "tile_64x128_2pass"]:
    setattr(GemmConfig, _n, classmethod(lambda cls, _n=_n: cls.preset(_n)))


class TileGemm(C.Structure):
    """``TileGemm`` (src/t0/tile_ir.rs:109-152)."""
    _fields_ = [("tile_m", C.c_uint32), ("tile_n", C.c_uint32), ("tile_k", C.c_uint32),
                ("wgp_mode", C.c_uint8), ("double_buffer", C.c_uint8), ("triple_buffer", C.c_uint8), ("swap_grid", C.c_uint8),
                ("split_k", C.c_uint32),
                ("transpose", C.c_uint8), ("acc_swap", C.c_uint8), ("persistent", C.c_uint8), ("n_epilogue", C.c_uint8),
                ("epilogue", C.c_uint8 * 8), ("waves_per_wg", C.c_uint32), ("wmma_format", C.c_uint32)]

    @classmethod
    def preset(cls, name: str) -> "TileGemm":
        s = cls()
        _check(lib().t0_tile_gemm_preset(name.encode(), C.byref(s)))
        return s

    def copy(self, **kw) -> "TileGemm":
        s = TileGemm.from_buffer_copy(self)
        for k, v in kw.items():
            setattr(s, k, v)
        return s

    def with_epilogue(self, ops: list[str]) -> "TileGemm":
        s = self.copy()
        s.n_epilogue = len(ops)
        for i, o in enumerate(ops):
            s.epilogue[i] = TEPI[o]
        return s

    def name(self) -> str:
        buf = C.create_string_buffer(160)
        _check(lib().t0_tile_gemm_name(C.byref(self), buf, 160))
        return buf.value.decode()

    def wg_size(self) -> int:
        return int(lib().t0_tile_gemm_wg_size(C.byref(self)))

    def lds_total(self) -> int:
        return int(lib().t0_tile_gemm_lds_total(C.byref(self)))

    def n_waves(self) -> int:
        return self.waves_per_wg or self.tile_m // 32

    def rows_per_wave(self) -> int:
        return self.tile_m // self.n_waves()

    def n_row_blocks(self) -> int:
        return self.rows_per_wave() // 16

    def k_sub_steps(self) -> int:
        return self.tile_k // 16

    def lds_per_buffer(self) -> int:
        return self.tile_m * self.tile_k * 2 + self.tile_n * self.tile_k * 2


TILE_PRESETS = ["tile_128x64_k16", "tile_64x64_k16", "tile_64x64_k32", "tile_64x64_k64", "tile_32x64_k16", "tile_128x64_k32",
                "tile_64x128_k32", "tile_64x128_k16", "tile_128x128_k16", "tile_128x128_k32", "tile_128x128_k48",
                "tile_128x128_k16_swap", "tile_128x128_k32_swap", "tile_256x64_k32_wgp", "tile_256x64_k64_wgp",
                "tile_128x128_k64", "tile_128x64_k64", "tile_32x32_k16", "tile_32x128_k16", "tile_128x32_k16",
                "tile_64x256_k32", "tile_128x256_k32", "tile_256x128_k32", "tile_persistent_decode",
                "tile_persistent_128x64_k32", "tile_persistent_256x128_k32"]
for _n in TILE_PRESETS:
    setattr(TileGemm, _n, classmethod(lambda cls, _n=_n: cls.preset(_n)))


class GemmArgs(C.Structure):
    """``t0_gemm_args``: explicit-argument GEMM launch."""
    _fields_ = [("x", C.c_uint64), ("b", C.c_uint64), ("y", C.c_uint64), ("bias", C.c_uint64),
                ("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32), ("tile_n", C.c_uint32), ("split_k", C.c_uint32),
                ("transpose", C.c_uint8), ("epilogue", C.c_uint8), ("out_bf16", C.c_uint8), ("planes", C.c_uint8),
                ("swap_grid", C.c_uint8), ("pair_cta", C.c_uint8), ("_pad", C.c_uint8 * 2),
                ("n_tile_epilogue", C.c_uint8), ("tile_epilogue", C.c_uint8 * 8), ("_pad2", C.c_uint8 * 3),
                ("scale", C.c_float), ("clamp_min", C.c_float), ("clamp_max", C.c_float)]


class TileConfig(C.Structure):
    """``cost_model::TileConfig`` (src/t0/cost_model.rs:130-168)."""
    _fields_ = [("tile_m", C.c_uint32), ("tile_n", C.c_uint32), ("tile_k", C.c_uint32), ("waves_per_wg", C.c_uint32),
                ("use_lds", C.c_uint8), ("wgp_mode", C.c_uint8), ("swap_grid", C.c_uint8), ("_pad", C.c_uint8),
                ("split_k", C.c_uint32), ("lds_pad", C.c_uint32)]

    def name(self) -> str:
        buf = C.create_string_buffer(96)
        _check(lib().t0_tile_config_name(C.byref(self), buf, 96))
        return buf.value.decode()

    def to_gemm_config(self) -> "GemmConfig":
        out = GemmConfig()
        _check(lib().t0_tile_config_to_gemm_config(C.byref(self), C.byref(out)))
        return out

    def to_tile_gemm(self) -> "TileGemm":
        out = TileGemm()
        _check(lib().t0_tile_config_to_tile_gemm(C.byref(self), C.byref(out)))
        return out

    def can_use_tile_ir(self) -> bool:
        return bool(lib().t0_tile_config_can_use_tile_ir(C.byref(self)))


class TileCost(C.Structure):
    """``cost_model::TileCost`` (src/t0/cost_model.rs:171-190)."""
    _fields_ = [("config", TileConfig), ("vgprs", C.c_uint32), ("sgprs", C.c_uint32), ("lds_bytes", C.c_uint32),
                ("occupancy", C.c_uint32), ("n_wgs", C.c_uint32), ("feasible", C.c_int), ("score", C.c_double),
                ("bottleneck", C.c_char * 24)]


def auto_schedule_gemm(m: int, n: int, k: int, cap: int = 64) -> list:
    """``cost_model::auto_schedule_gemm`` (cost_model.rs:464-534): feasible candidates, best first."""
    arr = (TileCost * cap)()
    got = lib().t0_auto_schedule_tile_costs(m, n, k, arr, cap)
    return [arr[i] for i in range(got)]


class WarpLayout(C.Structure):
    """``WarpLayout`` (src/t0/tile_ir.rs:8365-8475)."""
    _fields_ = [("n_warps", C.c_uint32), ("rows_per_warp", C.c_uint32), ("cols_per_warp", C.c_uint32), ("orientation", C.c_uint32)]
    ROW_DOMINANT, COL_DOMINANT, SQUARE = 0, 1, 2

    @staticmethod
    def _make(fn: str, n_warps: int, tile_m: int, tile_n: int) -> "WarpLayout":
        out = WarpLayout()
        _check(getattr(lib(), fn)(n_warps, tile_m, tile_n, C.byref(out)))
        return out

    @staticmethod
    def row_dominant(n_warps: int, tile_m: int, tile_n: int) -> "WarpLayout":
        return WarpLayout._make("t0_warp_layout_row_dominant", n_warps, tile_m, tile_n)

    @staticmethod
    def col_dominant(n_warps: int, tile_m: int, tile_n: int) -> "WarpLayout":
        return WarpLayout._make("t0_warp_layout_col_dominant", n_warps, tile_m, tile_n)

    @staticmethod
    def square(n_warps: int, tile_m: int, tile_n: int) -> "WarpLayout":
        return WarpLayout._make("t0_warp_layout_square", n_warps, tile_m, tile_n)

    def wmma_row_blocks(self) -> int: return lib().t0_warp_layout_wmma_row_blocks(C.byref(self))
    def wmma_col_tiles(self) -> int: return lib().t0_warp_layout_wmma_col_tiles(C.byref(self))
    def wmma_ops_per_warp(self) -> int: return lib().t0_warp_layout_wmma_ops_per_warp(C.byref(self))
    def acc_vgprs_per_warp(self) -> int: return lib().t0_warp_layout_acc_vgprs_per_warp(C.byref(self))
    def wg_size(self) -> int: return lib().t0_warp_layout_wg_size(C.byref(self))
    def is_compatible(self, tile_m: int, tile_n: int) -> bool: return bool(lib().t0_warp_layout_is_compatible(C.byref(self), tile_m, tile_n))


def plan_flash_attention_warps(n_warps: int, m: int, n: int, d: int):
    """``plan_flash_attention_warps`` (tile_ir.rs:8487-8524) -> (qk_layout, av_layout)."""
    qk, av = WarpLayout(), WarpLayout()
    _check(lib().t0_plan_flash_attention_warps(n_warps, m, n, d, C.byref(qk), C.byref(av)))
    return qk, av


def plan_single_dot_warps(n_warps: int, tile_m: int, tile_n: int) -> WarpLayout:
    """``plan_single_dot_warps`` (tile_ir.rs:8529-8540)."""
    return WarpLayout._make("t0_plan_single_dot_warps", n_warps, tile_m, tile_n)


class W4A16Args(C.Structure):
    """``t0_w4a16_args``."""
    _fields_ = [("a", C.c_uint64), ("packed", C.c_uint64), ("scales", C.c_uint64), ("zeros", C.c_uint64), ("y", C.c_uint64),
                ("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32), ("group", C.c_uint32)]


class Int4WmmaConfig(C.Structure):
    """``Int4WmmaConfig`` (quant_kernels.rs:316-336): the INT4 tile record and its two constructors."""
    _fields_ = [("tile_m", C.c_uint32), ("tile_n", C.c_uint32), ("tile_k", C.c_uint32)]

    @classmethod
    def k16(cls) -> "Int4WmmaConfig":
        out = cls()
        _check(lib().t0_int4_wmma_config_k16(C.byref(out)))
        return out

    @classmethod
    def k32(cls) -> "Int4WmmaConfig":
        out = cls()
        _check(lib().t0_int4_wmma_config_k32(C.byref(out)))
        return out


# --------------------------------------------------------------------------- selection / grids / kernargs

def auto_select(m: int, k: int, n: int) -> GemmConfig:
    """``auto_select(m, k, n)`` (gemm_gen.rs:340) — note the (m, k, n) order."""
    c = GemmConfig()
    _check(lib().t0_auto_select(m, k, n, C.byref(c)))
    return c


def auto_select_legacy(m: int, k: int, n: int) -> GemmConfig:
    c = GemmConfig()
    _check(lib().t0_auto_select_legacy(m, k, n, C.byref(c)))
    return c


def cached_auto_select(m: int, k: int, n: int) -> GemmConfig:
    c = GemmConfig()
    _check(lib().t0_cached_auto_select(m, k, n, C.byref(c)))
    return c


def prewarm_cache(dims: list[tuple[int, int, int]]) -> None:
    arr = (C.c_uint32 * (3 * len(dims)))(*[v for d in dims for v in d])
    _check(lib().t0_prewarm_cache(arr, len(dims)))


def clear_cache() -> None:
    lib().t0_clear_cache()


def cache_size() -> int:
    return int(lib().t0_cache_size())


def auto_schedule_gemm_configs(m: int, n: int, k: int, cap: int = 64) -> list[tuple[GemmConfig, float]]:
    """The same ranking as (GemmConfig, predicted TFLOP/s) pairs."""
    cfgs = (GemmConfig * cap)()
    tf = (C.c_double * cap)()
    cnt = lib().t0_auto_schedule_gemm(m, n, k, cfgs, tf, cap)
    return [(GemmConfig.from_buffer_copy(cfgs[i]), tf[i]) for i in range(cnt)]


def compute_grid(cfg: GemmConfig, m: int, n: int) -> tuple[int, int]:
    gx, gy = C.c_uint32(), C.c_uint32()
    _check(lib().t0_compute_grid(C.byref(cfg), m, n, C.byref(gx), C.byref(gy)))
    return gx.value, gy.value


def compute_grid_split_k(cfg: GemmConfig, m: int, n: int, split_k: int) -> tuple[int, int]:
    gx, gy = C.c_uint32(), C.c_uint32()
    _check(lib().t0_compute_grid_split_k(C.byref(cfg), m, n, split_k, C.byref(gx), C.byref(gy)))
    return gx.value, gy.value


def compute_grid_auto(cfg: GemmConfig, m: int, n: int) -> tuple[int, int]:
    gx, gy = C.c_uint32(), C.c_uint32()
    _check(lib().t0_compute_grid_auto(C.byref(cfg), m, n, C.byref(gx), C.byref(gy)))
    return gx.value, gy.value


def build_kernargs(x: int, wt: int, y: int, k: int, n: int, m: int, cfg: GemmConfig) -> bytes:
    """``build_kernargs(x, wt, y, k, n, m, &cfg) -> [u8; 40]`` (gemm_gen.rs:442-458)."""
    out = (C.c_uint8 * 40)()
    _check(lib().t0_build_kernargs(x, wt, y, k, n, m, C.byref(cfg), out))
    return bytes(out)


def build_kernargs_with_bias(x: int, wt: int, y: int, k: int, n: int, m: int, cfg: GemmConfig, bias: int) -> bytes:
    out = (C.c_uint8 * 48)()
    _check(lib().t0_build_kernargs_with_bias(x, wt, y, k, n, m, C.byref(cfg), bias, out))
    return bytes(out)


def tile_auto_select(m: int, k: int, n: int, transpose: int = NT) -> TileGemm:
    s = TileGemm()
    _check(lib().t0_tile_auto_select(m, k, n, transpose, C.byref(s)))
    return s


def tile_build_kernargs_m(x: int, wt: int, y: int, k: int, n: int, m: int, spec: TileGemm) -> bytes:
    out = (C.c_uint8 * 96)()
    ln = C.c_size_t()
    _check(lib().t0_tile_build_kernargs_m(x, wt, y, k, n, m, C.byref(spec), out, 96, C.byref(ln)))
    return bytes(out[: ln.value])


def tile_build_kernargs_epilogue(x: int, wt: int, y: int, k: int, n: int, m: int, spec: TileGemm, bias: int = 0,
                                 scale: float = 1.0, clamp_min: float = 0.0, clamp_max: float = 0.0) -> bytes:
    out = (C.c_uint8 * 96)()
    ln = C.c_size_t()
    _check(lib().t0_tile_build_kernargs_epilogue(x, wt, y, k, n, m, C.byref(spec), bias, scale, clamp_min, clamp_max,
                                                 out, 96, C.byref(ln)))
    return bytes(out[: ln.value])


def tile_compute_grid(spec: TileGemm, m: int, n: int) -> list[int]:
    g = (C.c_uint32 * 3)()
    _check(lib().t0_tile_compute_grid(C.byref(spec), m, n, g))
    return list(g)


def f32_to_bf16(v: float) -> int:
    return int(lib().t0_f32_to_bf16(v))


def bf16_to_f32(v: int) -> float:
    return float(lib().t0_bf16_to_f32(v))


def gptq_parse(raw: bytes) -> dict:
    """``GptqWeight::from_bytes`` (quant_kernels.rs:242-286)."""
    buf = np.frombuffer(raw, dtype=np.uint8)
    rows, cols, group = C.c_uint32(), C.c_uint32(), C.c_uint32()
    po, so, zo = C.c_size_t(), C.c_size_t(), C.c_size_t()
    _check(lib().t0_gptq_parse(buf.ctypes.data_as(C.c_void_p), len(raw), C.byref(rows), C.byref(cols), C.byref(group),
                               C.byref(po), C.byref(so), C.byref(zo)))
    r, c, g = rows.value, cols.value, group.value
    n_params = (c // g) * r
    return {"rows": r, "cols": c, "group_size": g, "n_groups": c // g,
            "packed": buf[po.value:po.value + r * c // 2].copy(),
            "scales": np.frombuffer(raw, dtype="<f4", count=n_params, offset=so.value).copy(),
            "zero_points": np.frombuffer(raw, dtype="<i4", count=n_params, offset=zo.value).copy(),
            "gpu_buffer_size": int(lib().t0_gptq_gpu_buffer_size(r, c, g))}


def gptq_to_b200(packed, scales, zero_points, rows: int, cols: int, group_size: int):
    """Repack a ``GptqWeight`` (rows = N, cols = K) into the B200 layout; returns (packed, scales, zeros, n_inexact_scales)."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    zero_points = np.ascontiguousarray(zero_points, dtype=np.int32)
    N, K = rows, cols
    p = np.zeros((K // 8, N), dtype=np.uint32)
    s = np.zeros((K // group_size, N), dtype=np.uint16)
    z = np.zeros((K // group_size, (N + 7) // 8), dtype=np.uint32)
    vp = C.c_void_p
    n = lib().t0_gptq_to_b200(packed.ctypes.data_as(vp), scales.ctypes.data_as(vp), zero_points.ctypes.data_as(vp), rows, cols,
                              group_size, p.ctypes.data_as(vp), s.ctypes.data_as(vp), z.ctypes.data_as(vp))
    if n < 0:
        raise T0Error(1, lib().t0_last_error().decode())
    return p, s, z, int(n)


# --------------------------------------------------------------------------- runtime

class GpuBuffer:
    """``GpuBuffer`` (src/kfd/buffer.rs:9-123)."""

    def __init__(self, handle, rt: "GpuRuntime"):
        self._h = handle
        self._rt = rt

    def gpu_addr(self) -> int:
        return int(lib().t0_buf_gpu_addr(self._h))

    @property
    def size(self) -> int:
        return int(lib().t0_buf_size(self._h))

    def write(self, data) -> None:
        a = np.ascontiguousarray(data)
        _check(lib().t0_buf_write(self._h, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def write_bytes(self, offset: int, data) -> None:
        a = np.ascontiguousarray(data)
        _check(lib().t0_buf_write_bytes(self._h, offset, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def read(self, nbytes: int, dtype=np.uint8) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        _check(lib().t0_buf_read(self._h, out.ctypes.data_as(C.c_void_p), nbytes))
        return out.view(dtype)

    def read_bytes(self, offset: int, nbytes: int, dtype=np.uint8) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        _check(lib().t0_buf_read_bytes(self._h, offset, out.ctypes.data_as(C.c_void_p), nbytes))
        return out.view(dtype)

    def zero(self) -> None:
        _check(lib().t0_buf_zero(self._h))

    def ipc_export(self) -> bytes:
        """The 64-byte handle another process on this machine passes to ``GpuRuntime.ipc_open``."""
        h = (C.c_uint8 * 64)()
        _check(lib().t0_buf_ipc_export(self._h, h))
        return bytes(h)

    def free(self) -> None:
        if self._h:
            lib().t0_buf_free(self._h)
            self._h = None


class GpuKernel:
    def __init__(self, handle):
        self._h = handle

    @property
    def kernarg_size(self) -> int:
        return int(lib().t0_kernel_kernarg_size(self._h))

    @property
    def name(self) -> str:
        return lib().t0_kernel_name(self._h).decode()


class GpuRuntime:
    """``GpuRuntime`` (src/ignis/gpu_context.rs:99-597): stream, buffer pool, kernel cache, poison flag."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        _check(lib().t0_rt_new(device, C.byref(h)))
        self._h = h

    @classmethod
    def new(cls, device: int = 0) -> "GpuRuntime":
        return cls(device)

    def close(self) -> None:
        if self._h:
            lib().t0_rt_free(self._h)
            self._h = None

    def is_poisoned(self) -> bool:
        return bool(lib().t0_rt_is_poisoned(self._h))

    def mark_poisoned(self) -> None:
        lib().t0_rt_mark_poisoned(self._h)

    def synchronize(self) -> None:
        _check(lib().t0_rt_synchronize(self._h))

    wait_idle = synchronize

    def set_wait_limit_ns(self, ns: int) -> None:
        """Limit of every single device-side barrier wait of the GEMM kernels (0 = default, 2 s)."""
        _check(lib().t0_rt_set_wait_limit_ns(self._h, ns))

    def selftest_drop_one_load(self) -> None:
        """Arms the failure-path self-test: the next GEMM launch leaves out one operand load (see the header)."""
        _check(lib().t0_rt_selftest_drop_one_load(self._h))

    SCRATCH_KINDS = {"operand_a": 0, "operand_b": 1, "splitk_planes": 2, "w4_weights": 3, "w4_fused": 4,
                     "f32_a": 5, "f32_b": 6, "f32_c": 7}

    def reserve_scratch(self, kind: str, n_bytes: int) -> None:
        """Grows one of the runtime's scratch buffers ahead of time so that later launches up to that size neither
        allocate nor synchronise (the header lists which paths use which buffer)."""
        _check(lib().t0_rt_reserve_scratch(self._h, self.SCRATCH_KINDS[kind], n_bytes))

    def w4_fused_scratch_bytes(self) -> int:
        return int(lib().t0_rt_w4_fused_scratch_bytes(self._h))

    def stream(self) -> int:
        return int(lib().t0_rt_stream(self._h) or 0)

    def sm_count(self) -> int:
        return int(lib().t0_rt_sm_count(self._h))

    def launch_count(self) -> int:
        return int(lib().t0_rt_launch_count(self._h))

    def alloc(self, n_bytes: int) -> GpuBuffer:
        h = C.c_void_p()
        _check(lib().t0_rt_alloc(self._h, n_bytes, C.byref(h)))
        return GpuBuffer(h, self)

    def alloc_zero(self, n_bytes: int) -> GpuBuffer:
        h = C.c_void_p()
        _check(lib().t0_rt_alloc_zero(self._h, n_bytes, C.byref(h)))
        return GpuBuffer(h, self)

    def alloc_f32(self, n: int) -> GpuBuffer:
        h = C.c_void_p()
        _check(lib().t0_rt_alloc_f32(self._h, n, C.byref(h)))
        return GpuBuffer(h, self)

    def recycle(self, buf: GpuBuffer) -> None:
        lib().t0_rt_recycle(self._h, buf._h)
        buf._h = None

    def pool_cached_bytes(self) -> int:
        return int(lib().t0_rt_pool_cached_bytes(self._h))

    def upload(self, data) -> GpuBuffer:
        a = np.ascontiguousarray(data)
        b = self.alloc(max(a.nbytes, 1))
        if a.nbytes:
            b.write(a)
        return b

    def read_f32(self, buf: GpuBuffer, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        _check(lib().t0_rt_read_f32(self._h, buf._h, n, out.ctypes.data_as(C.c_void_p)))
        return out

    def write_f32(self, buf: GpuBuffer, data) -> None:
        a = np.ascontiguousarray(data, dtype=np.float32)
        _check(lib().t0_rt_write_f32(self._h, buf._h, a.ctypes.data_as(C.c_void_p), a.size))

    def upload_f32(self, data) -> GpuBuffer:
        a = np.ascontiguousarray(data, dtype=np.float32)
        h = C.c_void_p()
        _check(lib().t0_rt_upload_f32(self._h, a.ctypes.data_as(C.c_void_p), a.size, C.byref(h)))
        return GpuBuffer(h, self)

    def ensure_kernel_t0(self, spec) -> GpuKernel:
        """``ensure_kernel_t0(name, || generate(&cfg) / lower_gemm(&spec), ..)`` (gpu_context.rs:212-259)."""
        h = C.c_void_p()
        if isinstance(spec, GemmConfig):
            _check(lib().t0_rt_ensure_gemm_kernel(self._h, C.byref(spec), C.byref(h)))
        else:
            _check(lib().t0_rt_ensure_tile_kernel(self._h, C.byref(spec), C.byref(h)))
        return GpuKernel(h)

    def kernel_cache_size(self) -> int:
        return int(lib().t0_rt_kernel_cache_size(self._h))

    def dispatch(self, kernel: GpuKernel, grid, kernargs: bytes) -> None:
        g = (C.c_uint32 * 3)(*grid)
        ka = (C.c_uint8 * len(kernargs)).from_buffer_copy(kernargs)
        _check(lib().t0_rt_dispatch(self._h, kernel._h, g, ka, len(kernargs)))

    def dispatch_async(self, kernel: GpuKernel, grid, kernargs: bytes) -> int:
        g = (C.c_uint32 * 3)(*grid)
        ka = (C.c_uint8 * len(kernargs)).from_buffer_copy(kernargs)
        slot = C.c_size_t()
        _check(lib().t0_rt_dispatch_async(self._h, kernel._h, g, ka, len(kernargs), C.byref(slot)))
        return slot.value

    def dispatch_bench(self, kernel: GpuKernel, grid, kernargs: bytes) -> None:
        g = (C.c_uint32 * 3)(*grid)
        ka = (C.c_uint8 * len(kernargs)).from_buffer_copy(kernargs)
        _check(lib().t0_rt_dispatch_bench(self._h, kernel._h, g, ka, len(kernargs)))

    def last_kernel_clock(self) -> tuple[float, float]:
        """(SM MHz, microseconds) measured inside the last GEMM kernel by its CTA 0."""
        mhz, us = C.c_double(), C.c_double()
        _check(lib().t0_rt_last_kernel_clock(self._h, C.byref(mhz), C.byref(us)))
        return mhz.value, us.value

    def timer_start(self) -> None:
        _check(lib().t0_rt_timer_start(self._h))

    def timer_stop(self) -> float:
        ms = C.c_float()
        _check(lib().t0_rt_timer_stop(self._h, C.byref(ms)))
        return ms.value

    def submit(self, kernel: GpuKernel, grid, kernargs: bytes) -> None:
        """``DispatchQueue::submit`` (prefill_dispatch.rs:61-100): no wait, no pointer validation."""
        g = (C.c_uint32 * 3)(*grid)
        ka = (C.c_uint8 * len(kernargs)).from_buffer_copy(kernargs)
        _check(lib().t0_rt_submit(self._h, kernel._h, g, ka, len(kernargs)))

    def flush(self) -> None:
        _check(lib().t0_rt_flush(self._h))

    @staticmethod
    def gemm_args(x: int, b: int, y: int, m: int, n: int, k: int, *, bias: int = 0, tile_n: int = 0, split_k: int = 1,
                  transpose: int = NT, epilogue: int = 0, out_bf16: bool = False, planes: bool = False,
                  swap_grid: bool = True, pair_cta: int = 0, tile_epilogue: list[str] | None = None, scale: float = 1.0,
                  clamp_min: float = 0.0, clamp_max: float = 0.0) -> GemmArgs:
        a = GemmArgs()
        a.x, a.b, a.y, a.bias = x, b, y, bias
        a.m, a.n, a.k, a.tile_n, a.split_k = m, n, k, tile_n, split_k
        a.transpose, a.epilogue, a.out_bf16, a.planes, a.swap_grid = transpose, epilogue, int(out_bf16), int(planes), int(swap_grid)
        a.pair_cta = pair_cta
        ops = tile_epilogue or []
        a.n_tile_epilogue = len(ops)
        for i, o in enumerate(ops):
            a.tile_epilogue[i] = TEPI[o]
        a.scale, a.clamp_min, a.clamp_max = scale, clamp_min, clamp_max
        return a

    def gemm_batch(self, args_list: list[GemmArgs]) -> None:
        """``t0_gemm_launch_batch``: the launches are submitted back to back from native code."""
        arr = (GemmArgs * len(args_list))(*args_list)
        _check(lib().t0_gemm_launch_batch(self._h, arr, len(args_list)))

    def gemm_grouped(self, args_list: list[GemmArgs]) -> None:
        """``t0_gemm_launch_grouped``: independent problems of one shape in one launch where the shape's configuration is the
        one-launch split-K; otherwise the same as ``gemm_batch``."""
        arr = (GemmArgs * len(args_list))(*args_list)
        _check(lib().t0_gemm_launch_grouped(self._h, arr, len(args_list)))

    def gemm_gather(self, args: GemmArgs, peer_y: list[int]) -> None:
        """``t0_gemm_launch_gather``: the product goes to ``args.y`` and, in the same epilogue, to every address of
        ``peer_y`` (other GPUs' memory mapped into this process)."""
        arr = (C.c_uint64 * max(1, len(peer_y)))(*peer_y)
        _check(lib().t0_gemm_launch_gather(self._h, C.byref(args), arr, len(peer_y)))

    def ipc_open(self, handle: bytes) -> int:
        """Maps a buffer exported by another process (``GpuBuffer.ipc_export``) and returns its device address here."""
        if len(handle) != 64:
            raise ValueError("an IPC handle is 64 bytes")
        ptr = C.c_uint64()
        _check(lib().t0_rt_ipc_open(self._h, (C.c_uint8 * 64)(*handle), C.byref(ptr)))
        return int(ptr.value)

    def ipc_close(self, device_ptr: int) -> None:
        _check(lib().t0_rt_ipc_close(self._h, device_ptr))

    def gemm_host_batch(self, args_list: list[GemmArgs]) -> None:
        """``t0_gemm_launch_host_batch``: x, b, y (and bias) of every problem are HOST addresses; uploads, kernels and
        downloads of consecutive problems overlap.  Returns when every result is in host memory."""
        arr = (GemmArgs * len(args_list))(*args_list)
        _check(lib().t0_gemm_launch_host_batch(self._h, arr, len(args_list)))

    def gemm(self, x: int, b: int, y: int, m: int, n: int, k: int, *, bias: int = 0, tile_n: int = 0, split_k: int = 1,
             transpose: int = NT, epilogue: int = 0, out_bf16: bool = False, planes: bool = False, swap_grid: bool = True,
             pair_cta: int = 0, tile_epilogue: list[str] | None = None, scale: float = 1.0, clamp_min: float = 0.0,
             clamp_max: float = 0.0) -> None:
        """Explicit-argument launch (``t0_gemm_launch``); device addresses as integers."""
        a = self.gemm_args(x, b, y, m, n, k, bias=bias, tile_n=tile_n, split_k=split_k, transpose=transpose, epilogue=epilogue,
                           out_bf16=out_bf16, planes=planes, swap_grid=swap_grid, pair_cta=pair_cta, tile_epilogue=tile_epilogue,
                           scale=scale, clamp_min=clamp_min, clamp_max=clamp_max)
        _check(lib().t0_gemm_launch(self._h, C.byref(a)))

    def ensure_dequant_kernel(self, group_size_log2: int, out_bf16: bool) -> GpuKernel:
        """``build_dequant_int4_f32/bf16(group_size_log2)`` (quant_kernels.rs:53,127) as a dispatchable kernel."""
        h = C.c_void_p()
        _check(lib().t0_rt_ensure_dequant_kernel(self._h, group_size_log2, int(out_bf16), C.byref(h)))
        return GpuKernel(h)

    def dequant_int4(self, packed: int, scales: int, zero_points: int, out: int, rows: int, cols: int, group_size_log2: int,
                     out_bf16: bool = False) -> None:
        _check(lib().t0_dequant_int4(self._h, packed, scales, zero_points, out, rows, cols, group_size_log2, int(out_bf16)))

    def w4_dequant(self, packed: int, scales: int, zeros: int, out_bf16: int, K: int, N: int, group: int = 128) -> None:
        _check(lib().t0_w4_dequant(self._h, packed, scales, zeros, out_bf16, K, N, group))

    def w4a16_gemm(self, a: int, packed: int, scales: int, zeros: int, y: int, M: int, N: int, K: int, group: int = 128) -> None:
        _check(lib().t0_w4a16_gemm(self._h, a, packed, scales, zeros, y, M, N, K, group))

    def w4a16_gemm_static(self, a: int, packed: int, scales: int, zeros: int, y: int, M: int, N: int, K: int, group: int = 128) -> None:
        """``t0_w4a16_gemm_static``: the fused kernel on the library's fixed scratch array; never allocates."""
        _check(lib().t0_w4a16_gemm_static(self._h, a, packed, scales, zeros, y, M, N, K, group))

    def matmul_f32(self, x: int, w: int, y: int, m: int, k: int, n: int) -> None:
        """Ignis ``matmul`` (src/ignis/ops/bf16_matmul.rs:33-59): y[M,N] = bf16(x[M,K]) * bf16(w[K,N]), f32 in and out."""
        _check(lib().t0_matmul_f32(self._h, x, w, y, m, k, n))

    def matmul_f32_with_wt_bf16(self, x: int, wt_bf16: int, y: int, m: int, k: int, n: int) -> None:
        _check(lib().t0_matmul_f32_with_wt_bf16(self._h, x, wt_bf16, y, m, k, n))

    def matmul_f32_backward_data(self, dy: int, w: int, dx: int, m: int, k: int, n: int) -> None:
        _check(lib().t0_matmul_f32_backward_data(self._h, dy, w, dx, m, k, n))

    def matmul_f32_backward_weight(self, x: int, dy: int, dw: int, m: int, k: int, n: int) -> None:
        _check(lib().t0_matmul_f32_backward_weight(self._h, x, dy, dw, m, k, n))

    def blas_gemm_f32(self, m: int, n: int, k: int, alpha: float, a: int, lda: int, b: int, ldb: int, beta: float, c: int, ldc: int) -> None:
        """``BlasLib::gemm`` (src/universal/math/mod.rs:24-35) for f32 operands."""
        _check(lib().t0_blas_gemm_f32(self._h, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc))

    def blas_gemv_f32(self, m: int, n: int, alpha: float, a: int, lda: int, x: int, incx: int, beta: float, y: int, incy: int) -> None:
        _check(lib().t0_blas_gemv_f32(self._h, m, n, alpha, a, lda, x, incx, beta, y, incy))

    def w4_prepack(self, packed: int, scales: int, zeros: int, K: int, N: int, group: int = 128) -> "GpuBuffer":
        """``t0_w4_prepack``: row layout -> streaming layout, into a new buffer."""
        n = lib().t0_w4_prepacked_bytes(K, N, group)
        if n == 0:
            raise T0Error(6, f"no streaming layout for K={K} N={N} group={group}")
        out = self.alloc(n)
        _check(lib().t0_w4_prepack(self._h, packed, scales, zeros, out.gpu_addr(), K, N, group))
        return out

    def w4a16_gemm_prepacked(self, a: int, prepacked: int, y: int, M: int, N: int, K: int, group: int = 128) -> None:
        _check(lib().t0_w4a16_gemm_prepacked(self._h, a, prepacked, y, M, N, K, group))

    def w4a16_gemm_prepacked_batch(self, calls: list[W4A16Args]) -> None:
        arr = (W4A16Args * len(calls))(*calls)
        _check(lib().t0_w4a16_gemm_prepacked_batch(self._h, arr, len(calls)))

    def w4a16_gemm_batch(self, calls: list[W4A16Args]) -> None:
        arr = (W4A16Args * len(calls))(*calls)
        _check(lib().t0_w4a16_gemm_batch(self._h, arr, len(calls)))

    def w4_to_tiled(self, packed: int, scales: int, zeros: int, K: int, N: int, group: int = 128) -> "GpuBuffer":
        """``t0_w4_to_tiled``: the weights rewritten into the tile-major layout (a new buffer)."""
        n = int(lib().t0_w4_tiled_bytes(K, N, group))
        if n == 0:
            raise T0Error(f"the tile-major layout does not take K={K} group={group}")
        out = self.alloc(n)
        _check(lib().t0_w4_to_tiled(self._h, packed, scales, zeros, out.gpu_addr(), K, N, group))
        return out

    def w4a16_gemm_tiled(self, a: int, tiled: int, y: int, M: int, N: int, K: int, group: int = 128) -> None:
        _check(lib().t0_w4a16_gemm_tiled(self._h, a, tiled, y, M, N, K, group))

    def w4a16_gemm_tiled_grouped(self, calls: list[W4A16Args]) -> None:
        """``t0_w4a16_gemm_tiled_grouped``: independent problems on tile-major weights, up to 32 of one shape per launch."""
        arr = (W4A16Args * len(calls))(*calls)
        _check(lib().t0_w4a16_gemm_tiled_grouped(self._h, arr, len(calls)))

    def w4a16_gemm_grouped(self, calls: list[W4A16Args]) -> None:
        """``t0_w4a16_gemm_grouped``: independent problems; one shape with 16 < M <= 128 runs up to 32 per launch."""
        arr = (W4A16Args * len(calls))(*calls)
        _check(lib().t0_w4a16_gemm_grouped(self._h, arr, len(calls)))

    def fill_uniform_bf16(self, dst: int, n: int, seed: int, first_index: int = 0) -> None:
        _check(lib().t0_fill_uniform_bf16(self._h, dst, n, seed, first_index))

    def fill_u32(self, dst: int, n: int, seed: int, first_index: int = 0) -> None:
        _check(lib().t0_fill_u32(self._h, dst, n, seed, first_index))

    def fill_range_bf16(self, dst: int, n: int, seed: int, lo: float, hi: float, first_index: int = 0) -> None:
        _check(lib().t0_fill_range_bf16(self._h, dst, n, seed, first_index, lo, hi))


def shard_columns(n: int, n_gpus: int, rank: int) -> tuple[int, int]:
    """(first column, number of columns) of rank's block of C: ``t0_shard_columns``."""
    a, b = C.c_uint32(), C.c_uint32()
    _check(lib().t0_shard_columns(n, n_gpus, rank, C.byref(a), C.byref(b)))
    return a.value, b.value


class MultiGpu:
    """One process driving several GPUs (``t0_mg``): N-column sharded GEMM, optional gathered C."""

    def __init__(self, n_gpus: int):
        h = C.c_void_p()
        _check(lib().t0_mg_new(n_gpus, C.byref(h)))
        self._h = h
        self.n = n_gpus

    def runtime(self, rank: int) -> "GpuRuntime":
        rt = GpuRuntime.__new__(GpuRuntime)
        rt._h = C.c_void_p(lib().t0_mg_runtime(self._h, rank))
        return rt

    def gemm_sharded(self, x: list[int], b_slice: list[int], y_slice: list[int], m: int, n: int, k: int, tile_n: int = 0,
                     pair_cta: int = 0) -> None:
        arr = lambda v: (C.c_uint64 * len(v))(*v)
        _check(lib().t0_mg_gemm_sharded(self._h, arr(x), arr(b_slice), arr(y_slice), m, n, k, tile_n, pair_cta))

    def gemm_sharded_host(self, x_host: np.ndarray, wt_host: np.ndarray, y_host: np.ndarray, m: int, n: int, k: int) -> None:
        """Host operands: A uploaded once in total (1/g per GPU, completed over NVLink), C written into ``y_host``."""
        _check(lib().t0_mg_gemm_sharded_host(self._h, x_host.ctypes.data_as(C.c_void_p), wt_host.ctypes.data_as(C.c_void_p),
                                             y_host.ctypes.data_as(C.c_void_p), m, n, k))

    def gemm_sharded_gathered(self, x: list[int], b_slice: list[int], c_gathered: list[int], m: int, n: int, k: int) -> None:
        """GEMM and all-gather in one kernel per GPU: every GPU's epilogue stores its block into slot r of all ``c_gathered``."""
        arr = lambda v: (C.c_uint64 * len(v))(*v)
        _check(lib().t0_mg_gemm_sharded_gathered(self._h, arr(x), arr(b_slice), arr(c_gathered), m, n, k))

    def all_gather_c(self, c_gathered: list[int], m: int, n: int) -> None:
        _check(lib().t0_mg_all_gather_c(self._h, (C.c_uint64 * len(c_gathered))(*c_gathered), m, n))

    def synchronize(self) -> None:
        _check(lib().t0_mg_synchronize(self._h))

    def free(self) -> None:
        if self._h:
            lib().t0_mg_free(self._h)
            self._h = None


class GemmTuner:
    """``GemmTuner`` (src/t0/auto_gemm.rs:46-216)."""

    def __init__(self, cache_dir: str | None = None, _handle=None):
        if _handle is not None:
            self._h, self._owned = _handle, False
            return
        h = C.c_void_p()
        if cache_dir is None:
            _check(lib().t0_tuner_new(C.byref(h)))
        else:
            _check(lib().t0_tuner_with_cache_dir(cache_dir.encode(), C.byref(h)))
        self._h, self._owned = h, True

    @classmethod
    def with_cache_dir(cls, d: str) -> "GemmTuner":
        return cls(d)

    @property
    def max_candidates(self) -> int:
        return int(lib().t0_tuner_max_candidates(self._h))

    @property
    def n_iters(self) -> int:
        return int(lib().t0_tuner_n_iters(self._h))

    def configure(self, max_candidates: int = 0, n_iters: int = 0) -> None:
        _check(lib().t0_tuner_configure(self._h, max_candidates, n_iters))

    @property
    def cache_dir(self) -> str:
        return lib().t0_tuner_cache_dir(self._h).decode()

    def cache_len(self) -> int:
        return int(lib().t0_tuner_cache_len(self._h))

    def tune(self, rt: "GpuRuntime", m: int, n: int, k: int) -> GemmConfig:
        c = GemmConfig()
        _check(lib().t0_tuner_tune(self._h, rt._h, m, n, k, C.byref(c)))
        return c

    def benchmark_tile_ir(self, rt: "GpuRuntime", spec: "TileGemm", m: int, n: int, k: int) -> float:
        """``GemmTuner::benchmark_tile_ir`` (auto_gemm.rs:352-431): median TFLOP/s of one TileGemm spec."""
        tf = C.c_double()
        _check(lib().t0_tuner_benchmark_tile_ir(self._h, rt._h, C.byref(spec), m, n, k, C.byref(tf)))
        return tf.value

    def result(self, m: int, n: int, k: int) -> dict:
        tf, fc, nm = C.c_double(), C.c_int(), C.c_int()
        _check(lib().t0_tuner_result(self._h, m, n, k, C.byref(tf), C.byref(fc), C.byref(nm)))
        return {"best_tflops": tf.value, "from_cache": bool(fc.value), "n_measured": nm.value}

    def save_cache(self, m: int, n: int, k: int, best: GemmConfig, tflops: float) -> None:
        _check(lib().t0_tuner_save_cache(self._h, m, n, k, C.byref(best), tflops))

    def load_cache(self, m: int, n: int, k: int) -> tuple[GemmConfig, float]:
        c, tf = GemmConfig(), C.c_double()
        _check(lib().t0_tuner_load_cache(self._h, m, n, k, C.byref(c), C.byref(tf)))
        return c, tf.value

    def invalidate(self, m: int, n: int, k: int) -> None:
        lib().t0_tuner_invalidate(self._h, m, n, k)

    def clear(self) -> None:
        lib().t0_tuner_clear(self._h)

    def report(self) -> None:
        lib().t0_tuner_report(self._h)

    def free(self) -> None:
        if self._owned and self._h:
            lib().t0_tuner_free(self._h)
            self._h = None


def global_tuner() -> GemmTuner:
    return GemmTuner(_handle=C.c_void_p(lib().t0_global_tuner()))


def auto_gemm(rt: "GpuRuntime", a: "GpuBuffer", b: "GpuBuffer", c: "GpuBuffer", m: int, n: int, k: int) -> float:
    """``auto_gemm(rt, a, b, c, m, n, k) -> Result<f64>`` (auto_gemm.rs:555-590); note the (m, n, k) order."""
    tf = C.c_double()
    _check(lib().t0_auto_gemm(rt._h, a._h, b._h, c._h, m, n, k, C.byref(tf)))
    return tf.value


def parse_json_number(json: str, key: str) -> float | None:
    out = C.c_double()
    return out.value if lib().t0_parse_json_number(json.encode(), key.encode(), C.byref(out)) == 0 else None


# --------------------------------------------------------------------------- ctypes signatures

def _declare(L: C.CDLL) -> None:
    u8p, u32, u64, sz, vp, i32 = C.POINTER(C.c_uint8), C.c_uint32, C.c_uint64, C.c_size_t, C.c_void_p, C.c_int
    cfgp, tilep, u32p = C.POINTER(GemmConfig), C.POINTER(TileGemm), C.POINTER(C.c_uint32)

    def sig(name, restype, *argtypes):
        fn = getattr(L, name)
        fn.restype = restype
        fn.argtypes = list(argtypes)

    sig("t0_last_error", C.c_char_p)
    sig("t0_version", i32)
    sig("t0_gemm_config_preset", i32, C.c_char_p, cfgp)
    sig("t0_gemm_config_name", i32, cfgp, C.c_char_p, sz)
    sig("t0_gemm_config_estimated_vgprs", u32, cfgp)
    sig("t0_gemm_config_is_feasible", i32, cfgp)
    sig("t0_gemm_config_lds_total", u32, cfgp)
    sig("t0_sweep_configs", i32, cfgp, i32)
    sig("t0_standard_configs", i32, cfgp, i32)
    for n in ("t0_auto_select", "t0_auto_select_legacy", "t0_auto_select_backward_data", "t0_auto_select_backward_weight",
              "t0_cached_auto_select", "t0_cached_auto_select_backward_data", "t0_cached_auto_select_backward_weight"):
        sig(n, i32, u32, u32, u32, cfgp)
    sig("t0_auto_schedule_gemm", i32, u32, u32, u32, cfgp, C.POINTER(C.c_double), i32)
    sig("t0_prewarm_cache", i32, u32p, sz)
    sig("t0_clear_cache", None)
    sig("t0_cache_size", sz)
    sig("t0_compute_grid", i32, cfgp, u32, u32, u32p, u32p)
    sig("t0_compute_grid_split_k", i32, cfgp, u32, u32, u32, u32p, u32p)
    sig("t0_compute_grid_auto", i32, cfgp, u32, u32, u32p, u32p)
    sig("t0_compute_grid_backward_data", i32, cfgp, u32, u32, u32p, u32p)
    sig("t0_compute_grid_backward_weight", i32, cfgp, u32, u32, u32p, u32p)
    sig("t0_build_kernargs", i32, u64, u64, u64, u32, u32, u32, cfgp, u8p)
    sig("t0_build_kernargs_with_bias", i32, u64, u64, u64, u32, u32, u32, cfgp, u64, u8p)
    sig("t0_build_kernargs_backward_data", i32, u64, u64, u64, u32, u32, u32, cfgp, u8p)
    sig("t0_build_kernargs_backward_weight", i32, u64, u64, u64, u32, u32, u32, cfgp, u8p)
    sig("t0_tile_gemm_preset", i32, C.c_char_p, tilep)
    sig("t0_tile_gemm_name", i32, tilep, C.c_char_p, sz)
    sig("t0_tile_gemm_wg_size", u32, tilep)
    sig("t0_tile_gemm_lds_total", u32, tilep)
    sig("t0_tile_auto_select", i32, u32, u32, u32, i32, tilep)
    sig("t0_tile_build_kernargs_m", i32, u64, u64, u64, u32, u32, u32, tilep, u8p, sz, C.POINTER(sz))
    sig("t0_tile_build_kernargs_epilogue", i32, u64, u64, u64, u32, u32, u32, tilep, u64, C.c_float, C.c_float, C.c_float,
        u8p, sz, C.POINTER(sz))
    sig("t0_tile_compute_grid", i32, tilep, u32, u32, u32p)
    sig("t0_f32_to_bf16", C.c_uint16, C.c_float)
    sig("t0_bf16_to_f32", C.c_float, C.c_uint16)
    sig("t0_rt_new", i32, i32, C.POINTER(vp))
    sig("t0_rt_free", None, vp)
    sig("t0_rt_is_poisoned", i32, vp)
    sig("t0_rt_mark_poisoned", None, vp)
    sig("t0_rt_synchronize", i32, vp)
    sig("t0_rt_wait_idle", i32, vp)
    sig("t0_rt_set_wait_limit_ns", i32, vp, u64)
    sig("t0_gemm_launch_grouped", i32, vp, C.POINTER(GemmArgs), sz)
    sig("t0_gemm_launch_gather", i32, vp, C.POINTER(GemmArgs), C.POINTER(C.c_uint64), u32)
    sig("t0_buf_ipc_export", i32, vp, C.POINTER(C.c_uint8))
    sig("t0_rt_ipc_open", i32, vp, C.POINTER(C.c_uint8), C.POINTER(C.c_uint64))
    sig("t0_rt_ipc_close", i32, vp, u64)
    sig("t0_mg_gemm_sharded_gathered", i32, vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), u32, u32, u32)
    sig("t0_rt_reserve_scratch", i32, vp, i32, sz)
    sig("t0_rt_w4_fused_scratch_bytes", sz, vp)
    sig("t0_rt_selftest_drop_one_load", i32, vp)
    sig("t0_int4_wmma_config_k16", i32, vp)
    sig("t0_int4_wmma_config_k32", i32, vp)
    sig("t0_rt_stream", vp, vp)
    sig("t0_rt_device", i32, vp)
    sig("t0_rt_sm_count", i32, vp)
    sig("t0_rt_launch_count", u64, vp)
    sig("t0_rt_last_kernel_clock", i32, vp, C.POINTER(C.c_double), C.POINTER(C.c_double))
    sig("t0_rt_timer_start", i32, vp)
    sig("t0_rt_timer_stop", i32, vp, C.POINTER(C.c_float))
    sig("t0_rt_alloc", i32, vp, sz, C.POINTER(vp))
    sig("t0_rt_alloc_zero", i32, vp, sz, C.POINTER(vp))
    sig("t0_rt_alloc_f32", i32, vp, sz, C.POINTER(vp))
    sig("t0_rt_recycle", None, vp, vp)
    sig("t0_rt_pool_cached_bytes", sz, vp)
    sig("t0_rt_pool_clear", None, vp)
    sig("t0_rt_read_f32", i32, vp, vp, sz, vp)
    sig("t0_rt_write_f32", i32, vp, vp, vp, sz)
    sig("t0_rt_upload_f32", i32, vp, vp, sz, C.POINTER(vp))
    sig("t0_buf_write", i32, vp, vp, sz)
    sig("t0_buf_read", i32, vp, vp, sz)
    sig("t0_buf_write_bytes", i32, vp, sz, vp, sz)
    sig("t0_buf_read_bytes", i32, vp, sz, vp, sz)
    sig("t0_buf_zero", i32, vp)
    sig("t0_buf_gpu_addr", u64, vp)
    sig("t0_buf_size", sz, vp)
    sig("t0_buf_free", None, vp)
    sig("t0_rt_ensure_gemm_kernel", i32, vp, cfgp, C.POINTER(vp))
    sig("t0_rt_ensure_tile_kernel", i32, vp, tilep, C.POINTER(vp))
    sig("t0_kernel_kernarg_size", u32, vp)
    sig("t0_kernel_name", C.c_char_p, vp)
    sig("t0_rt_kernel_cache_size", sz, vp)
    sig("t0_rt_dispatch", i32, vp, vp, u32p, u8p, sz)
    sig("t0_rt_dispatch_async", i32, vp, vp, u32p, u8p, sz, C.POINTER(sz))
    sig("t0_rt_dispatch_bench", i32, vp, vp, u32p, u8p, sz)
    sig("t0_gemm_launch", i32, vp, C.POINTER(GemmArgs))
    sig("t0_gemm_launch_batch", i32, vp, C.POINTER(GemmArgs), sz)
    sig("t0_gemm_launch_host_batch", i32, vp, C.POINTER(GemmArgs), sz)
    sig("t0_gemm_launch_host", i32, vp, C.POINTER(GemmArgs))
    sig("t0_rt_submit", i32, vp, vp, u32p, u8p, sz)
    sig("t0_rt_flush", i32, vp)
    sig("t0_shard_columns", i32, u32, u32, u32, u32p, u32p)
    sig("t0_mg_new", i32, i32, C.POINTER(vp))
    sig("t0_mg_free", None, vp)
    sig("t0_mg_size", i32, vp)
    sig("t0_mg_runtime", vp, vp, i32)
    sig("t0_mg_synchronize", i32, vp)
    sig("t0_mg_gemm_sharded", i32, vp, C.POINTER(u64), C.POINTER(u64), C.POINTER(u64), u32, u32, u32, u32, i32)
    sig("t0_mg_gemm_sharded_host", i32, vp, vp, vp, vp, u32, u32, u32)
    sig("t0_mg_all_gather_c", i32, vp, C.POINTER(u64), u32, u32)
    sig("t0_tuner_new", i32, C.POINTER(vp))
    sig("t0_tuner_with_cache_dir", i32, C.c_char_p, C.POINTER(vp))
    sig("t0_tuner_free", None, vp)
    sig("t0_tuner_configure", i32, vp, sz, sz)
    sig("t0_tuner_max_candidates", sz, vp)
    sig("t0_tuner_n_iters", sz, vp)
    sig("t0_tuner_cache_len", sz, vp)
    sig("t0_tuner_cache_dir", C.c_char_p, vp)
    sig("t0_tuner_tune", i32, vp, vp, u32, u32, u32, cfgp)
    sig("t0_tuner_result", i32, vp, u32, u32, u32, C.POINTER(C.c_double), C.POINTER(i32), C.POINTER(i32))
    sig("t0_tuner_save_cache", i32, vp, u32, u32, u32, cfgp, C.c_double)
    sig("t0_tuner_load_cache", i32, vp, u32, u32, u32, cfgp, C.POINTER(C.c_double))
    sig("t0_parse_json_number", i32, C.c_char_p, C.c_char_p, C.POINTER(C.c_double))
    sig("t0_tuner_invalidate", None, vp, u32, u32, u32)
    sig("t0_tuner_clear", None, vp)
    sig("t0_tuner_report", None, vp)
    sig("t0_tuner_benchmark_tile_ir", i32, vp, vp, C.POINTER(TileGemm), u32, u32, u32, C.POINTER(C.c_double))
    sig("t0_global_tuner", vp)
    sig("t0_auto_gemm", i32, vp, vp, vp, vp, u32, u32, u32, C.POINTER(C.c_double))
    sig("t0_dequant_int4", i32, vp, u64, u64, u64, u64, u32, u32, u32, i32)
    sig("t0_rt_ensure_dequant_kernel", i32, vp, u32, i32, C.POINTER(vp))
    sig("t0_w4_dequant", i32, vp, u64, u64, u64, u64, u32, u32, u32)
    sig("t0_w4a16_gemm", i32, vp, u64, u64, u64, u64, u64, u32, u32, u32, u32)
    sig("t0_w4a16_gemm_batch", i32, vp, C.POINTER(W4A16Args), sz)
    sig("t0_w4a16_gemm_grouped", i32, vp, C.POINTER(W4A16Args), sz)
    sig("t0_w4a16_gemm_tiled_grouped", i32, vp, C.POINTER(W4A16Args), sz)
    sig("t0_w4_tiled_bytes", sz, u32, u32, u32)
    sig("t0_w4_to_tiled", i32, vp, u64, u64, u64, u64, u32, u32, u32)
    sig("t0_w4a16_gemm_tiled", i32, vp, u64, u64, u64, u32, u32, u32, u32)
    sig("t0_w4a16_gemm_static", i32, vp, u64, u64, u64, u64, u64, u32, u32, u32, u32)
    tcp = C.POINTER(TileConfig)
    sig("t0_auto_schedule_tile_costs", i32, u32, u32, u32, C.POINTER(TileCost), i32)
    sig("t0_tile_config_name", i32, tcp, C.c_char_p, sz)
    sig("t0_tile_config_to_gemm_config", i32, tcp, C.POINTER(GemmConfig))
    sig("t0_tile_config_to_tile_gemm", i32, tcp, C.POINTER(TileGemm))
    sig("t0_tile_config_can_use_tile_ir", i32, tcp)
    wlp = C.POINTER(WarpLayout)
    for fn in ("t0_warp_layout_row_dominant", "t0_warp_layout_col_dominant", "t0_warp_layout_square", "t0_plan_single_dot_warps"):
        sig(fn, i32, u32, u32, u32, wlp)
    for fn in ("t0_warp_layout_wmma_row_blocks", "t0_warp_layout_wmma_col_tiles", "t0_warp_layout_wmma_ops_per_warp",
               "t0_warp_layout_acc_vgprs_per_warp", "t0_warp_layout_wg_size"):
        sig(fn, u32, wlp)
    sig("t0_warp_layout_is_compatible", i32, wlp, u32, u32)
    sig("t0_plan_flash_attention_warps", i32, u32, u32, u32, u32, wlp, wlp)
    f32 = C.c_float
    sig("t0_matmul_f32", i32, vp, u64, u64, u64, u32, u32, u32)
    sig("t0_matmul_f32_with_wt_bf16", i32, vp, u64, u64, u64, u32, u32, u32)
    sig("t0_matmul_f32_backward_data", i32, vp, u64, u64, u64, u32, u32, u32)
    sig("t0_matmul_f32_backward_weight", i32, vp, u64, u64, u64, u32, u32, u32)
    sig("t0_blas_gemm_f32", i32, vp, u32, u32, u32, f32, u64, u32, u64, u32, f32, u64, u32)
    sig("t0_blas_gemv_f32", i32, vp, u32, u32, f32, u64, u32, u64, u32, f32, u64, u32)
    sig("t0_w4_prepacked_bytes", sz, u32, u32, u32)
    sig("t0_w4_prepack", i32, vp, u64, u64, u64, u64, u32, u32, u32)
    sig("t0_w4a16_gemm_prepacked", i32, vp, u64, u64, u64, u32, u32, u32, u32)
    sig("t0_w4a16_gemm_prepacked_batch", i32, vp, C.POINTER(W4A16Args), sz)
    sig("t0_w4a16_gemm_static_scratch_bytes", sz)
    sig("t0_gptq_parse", i32, vp, sz, u32p, u32p, u32p, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz))
    sig("t0_gptq_gpu_buffer_size", sz, u32, u32, u32)
    sig("t0_gptq_to_b200", C.c_long, vp, vp, vp, u32, u32, u32, vp, vp, vp)
    sig("t0_fill_uniform_bf16", i32, vp, u64, u64, u64, u64)
    sig("t0_fill_u32", i32, vp, u64, u64, u64, u64)
    sig("t0_fill_range_bf16", i32, vp, u64, u64, u64, u64, C.c_float, C.c_float)

"""ctypes loader for the CPU oracle (test infrastructure only).

The oracle restates the reference's CPU reference GEMM / dequant arithmetic in
C (oracle.c).  Nothing in the product package imports this module; only the
tests, the smoke check and the benchmark's CPU-baseline leg do.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile oracle.c into liboracle.so (gcc, a few seconds)."""
    src = os.path.join(_HERE, "oracle.c")
    hdr = os.path.join(_HERE, "oracle.h")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= max(os.path.getmtime(src), os.path.getmtime(hdr))):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _declare(L: C.CDLL) -> None:
    u16, u32, u64, i32, f32 = C.c_uint16, C.c_uint32, C.c_uint64, C.c_int, C.c_float
    vp = C.c_void_p
    L.oracle_f32_to_bf16_trunc.restype = u16
    L.oracle_f32_to_bf16_trunc.argtypes = [f32]
    L.oracle_f32_to_bf16_rne.restype = u16
    L.oracle_f32_to_bf16_rne.argtypes = [f32]
    L.oracle_bf16_to_f32.restype = f32
    L.oracle_bf16_to_f32.argtypes = [u16]
    L.oracle_splitmix64.restype = u64
    L.oracle_splitmix64.argtypes = [u64, u64]
    L.oracle_fill_uniform_bf16.argtypes = [vp, u64, u64, u64]
    L.oracle_fill_u32.argtypes = [vp, u64, u64, u64]
    L.oracle_fill_range_bf16.argtypes = [vp, u64, u64, u64, f32, f32]
    L.oracle_fill_normal_bf16.argtypes = [vp, u64, u64]
    L.oracle_gemm_nt_bf16_rows.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32, i32]
    L.oracle_gemm_nt_bf16.argtypes = [vp, vp, vp, u32, u32, u32, i32]
    L.oracle_gemm_nn_bf16.argtypes = [vp, vp, vp, u32, u32, u32, i32]
    L.oracle_gemm_nt_bf16_f64.argtypes = [vp, vp, vp, u32, u32, u32, i32]
    L.oracle_gemm_nt_bf16_splitk.argtypes = [vp, vp, vp, vp, u32, u32, u32, u32, i32]
    L.oracle_f32_to_bf16_rne_array.argtypes = [vp, vp, u64]
    L.oracle_epilogue_gemm_gen.argtypes = [vp, vp, u32, u32, i32]
    L.oracle_epilogue_tile.argtypes = [vp, u32, u32, vp, i32, vp, f32, f32, f32]
    L.oracle_dequant_int4_ref_f32.argtypes = [vp, vp, vp, vp, u32, u32, u32]
    L.oracle_dequant_int4_ref_bf16.argtypes = [vp, vp, vp, vp, u32, u32, u32]
    L.oracle_dequant_w4_b200.argtypes = [vp, vp, vp, vp, u32, u32, u32]
    L.oracle_w4a16_gemm.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32, i32]
    L.oracle_gptq_parse.restype = i32
    L.oracle_gptq_parse.argtypes = [vp, C.c_size_t] + [C.POINTER(u32)] * 3 + [C.POINTER(C.c_size_t)] * 3
    L.oracle_gptq_to_b200.restype = C.c_long
    L.oracle_gptq_to_b200.argtypes = [vp, vp, vp, u32, u32, u32, vp, vp, vp]
    L.oracle_host_threads.restype = i32


# ---------------------------------------------------------------- helpers --

def host_threads() -> int:
    return int(lib().oracle_host_threads())


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) -> float32 (tile_ir.rs:4681: bits << 16)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_rne(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16_rne_array(_p(x), _p(out), x.size)
    return out


def f32_to_bf16_trunc(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def fill_uniform_bf16(n: int, seed: int, first_index: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    lib().oracle_fill_uniform_bf16(_p(out), n, seed, first_index)
    return out


def fill_u32(n: int, seed: int, first_index: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.uint32)
    lib().oracle_fill_u32(_p(out), n, seed, first_index)
    return out


def fill_range_bf16(n: int, seed: int, lo: float, hi: float, first_index: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    lib().oracle_fill_range_bf16(_p(out), n, seed, first_index, lo, hi)
    return out


def fill_normal_bf16(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    lib().oracle_fill_normal_bf16(_p(out), n, seed)
    return out


def gemm_nt(x: np.ndarray, wt: np.ndarray, m: int, k: int, n: int, threads: int = 0,
            rows: tuple[int, int] | None = None) -> np.ndarray:
    """y[m,n] f32 = x[m,k] @ wt[n,k]^T, reference arithmetic (tile_ir.rs:5021-5038)."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    wt = np.ascontiguousarray(wt, dtype=np.uint16)
    y = np.zeros((m, n), dtype=np.float32)
    r0, r1 = rows if rows is not None else (0, m)
    lib().oracle_gemm_nt_bf16_rows(_p(x), _p(wt), _p(y), m, k, n, r0, r1, threads)
    return y


def gemm_nn(x: np.ndarray, b: np.ndarray, m: int, k: int, n: int, threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    b = np.ascontiguousarray(b, dtype=np.uint16)
    y = np.zeros((m, n), dtype=np.float32)
    lib().oracle_gemm_nn_bf16(_p(x), _p(b), _p(y), m, k, n, threads)
    return y


def gemm_nt_f64(x: np.ndarray, wt: np.ndarray, m: int, k: int, n: int, threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    wt = np.ascontiguousarray(wt, dtype=np.uint16)
    y = np.zeros((m, n), dtype=np.float64)
    lib().oracle_gemm_nt_bf16_f64(_p(x), _p(wt), _p(y), m, k, n, threads)
    return y


def gemm_nt_splitk(x: np.ndarray, wt: np.ndarray, m: int, k: int, n: int, split_k: int,
                   threads: int = 0) -> tuple[np.ndarray, np.ndarray]:
    """Returns (planes[split_k,m,n], sum of planes in split order)."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    wt = np.ascontiguousarray(wt, dtype=np.uint16)
    planes = np.zeros((split_k, m, n), dtype=np.float32)
    ysum = np.zeros((m, n), dtype=np.float32)
    lib().oracle_gemm_nt_bf16_splitk(_p(x), _p(wt), _p(planes), _p(ysum), m, k, n, split_k, threads)
    return planes, ysum


def epilogue_gemm_gen(y: np.ndarray, bias: np.ndarray, mode: int) -> np.ndarray:
    y = np.array(y, dtype=np.float32, order="C", copy=True)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    lib().oracle_epilogue_gemm_gen(_p(y), _p(bias), y.shape[0], y.shape[1], mode)
    return y


TILE_EPI = {"bias": 0, "scale": 1, "relu": 2, "silu": 3, "gelu": 4, "abs": 5, "neg": 6, "clamp": 7}


def epilogue_tile(y: np.ndarray, ops: list[str], bias: np.ndarray | None = None, scale: float = 1.0,
                  clamp_min: float = 0.0, clamp_max: float = 0.0) -> np.ndarray:
    y = np.array(y, dtype=np.float32, order="C", copy=True)
    codes = np.array([TILE_EPI[o] for o in ops], dtype=np.int32)
    b = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
    lib().oracle_epilogue_tile(_p(y), y.shape[0], y.shape[1], _p(codes), len(codes),
                               _p(b) if b is not None else None, scale, clamp_min, clamp_max)
    return y


def dequant_int4_ref(packed: np.ndarray, scales: np.ndarray, zps: np.ndarray, rows: int, cols: int,
                     group_log2: int, bf16: bool = False) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    zps = np.ascontiguousarray(zps, dtype=np.int32)
    if bf16:
        out = np.empty((rows, cols), dtype=np.uint16)
        lib().oracle_dequant_int4_ref_bf16(_p(packed), _p(scales), _p(zps), _p(out), rows, cols, group_log2)
    else:
        out = np.empty((rows, cols), dtype=np.float32)
        lib().oracle_dequant_int4_ref_f32(_p(packed), _p(scales), _p(zps), _p(out), rows, cols, group_log2)
    return out


def dequant_w4_b200(packed: np.ndarray, scales: np.ndarray, zeros: np.ndarray, K: int, N: int,
                    group: int = 128) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    zeros = np.ascontiguousarray(zeros, dtype=np.uint32)
    out = np.empty((K, N), dtype=np.uint16)
    lib().oracle_dequant_w4_b200(_p(packed), _p(scales), _p(zeros), _p(out), K, N, group)
    return out


def w4a16_gemm(a: np.ndarray, packed: np.ndarray, scales: np.ndarray, zeros: np.ndarray,
               M: int, N: int, K: int, group: int = 128, threads: int = 0) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    zeros = np.ascontiguousarray(zeros, dtype=np.uint32)
    y = np.zeros((M, N), dtype=np.float32)
    lib().oracle_w4a16_gemm(_p(a), _p(packed), _p(scales), _p(zeros), _p(y), M, N, K, group, threads)
    return y


def w4_prepack(packed: np.ndarray, scales: np.ndarray, zeros: np.ndarray, K: int, N: int, group: int = 128) -> np.ndarray:
    """Tile-major streaming layout of the B200 W4A16 kernel (one uint8 buffer)."""
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    zeros = np.ascontiguousarray(zeros, dtype=np.uint32)
    off = (C.c_size_t * 3)()
    L = lib()
    L.oracle_w4_prepacked_layout.restype = C.c_size_t
    L.oracle_w4_prepacked_layout.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_size_t)]
    L.oracle_w4_prepack.restype = None
    L.oracle_w4_prepack.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32]
    total = L.oracle_w4_prepacked_layout(K, N, group, off)
    out = np.zeros(total, dtype=np.uint8)
    L.oracle_w4_prepack(_p(packed), _p(scales), _p(zeros), _p(out), K, N, group)
    return out


def w4_to_tiled(packed: np.ndarray, scales: np.ndarray, zeros: np.ndarray, K: int, N: int, group: int = 128) -> np.ndarray:
    """Tile-major layout of the B200 W4A16 kernel for 16 < M <= 128 (one uint8 buffer): every 256-column tile a matrix of its
    own, words [T][K/8][256] u32 (code k of a word in nibble (k >> 1) + 4 (k & 1)), then scales [T][K/group][256] bf16, then zero
    points [T][K/group][32] u32, columns past N zero.  (No counterpart in the reference: a pure index remap of the B200 row layout.)"""
    T = -(-N // 256)
    npad = T * 256
    pk = np.zeros((K // 8, npad), np.uint32)
    src = np.asarray(packed, np.uint32).reshape(K // 8, N)
    perm = np.zeros_like(src)
    for k in range(8):                      # code k of a word moves to nibble (k >> 1) + 4 (k & 1)
        perm |= ((src >> np.uint32(4 * k)) & np.uint32(0xF)) << np.uint32(4 * ((k >> 1) + 4 * (k & 1)))
    pk[:, :N] = perm
    sc = np.zeros((K // group, npad), np.uint16)
    sc[:, :N] = np.asarray(scales, np.uint16).reshape(K // group, N)
    zsrc = np.asarray(zeros, np.uint32).reshape(K // group, -1)
    zp = np.zeros((K // group, npad // 8), np.uint32)
    zp[:, :zsrc.shape[1]] = zsrc
    words = pk.reshape(K // 8, T, 256).transpose(1, 0, 2)
    sct = sc.reshape(K // group, T, 256).transpose(1, 0, 2)
    zpt = zp.reshape(K // group, T, 32).transpose(1, 0, 2)
    return np.concatenate([np.ascontiguousarray(words).view(np.uint8).reshape(-1), np.ascontiguousarray(sct).view(np.uint8).reshape(-1),
                           np.ascontiguousarray(zpt).view(np.uint8).reshape(-1)])


def gptq_parse(raw: bytes):
    """GptqWeight::from_bytes wire format (quant_kernels.rs:242-286) -> dict of arrays."""
    buf = np.frombuffer(raw, dtype=np.uint8)
    rows, cols, group = C.c_uint32(), C.c_uint32(), C.c_uint32()
    po, so, zo = C.c_size_t(), C.c_size_t(), C.c_size_t()
    rc = lib().oracle_gptq_parse(_p(buf), len(raw), C.byref(rows), C.byref(cols), C.byref(group),
                                 C.byref(po), C.byref(so), C.byref(zo))
    if rc != 0:
        raise ValueError("GPTQ data truncated")
    r, c, g = rows.value, cols.value, group.value
    n_params = (c // g) * r
    return {
        "rows": r, "cols": c, "group_size": g, "n_groups": c // g,
        "packed": buf[po.value:po.value + r * c // 2].copy(),
        "scales": np.frombuffer(raw, dtype="<f4", count=n_params, offset=so.value).copy(),
        "zero_points": np.frombuffer(raw, dtype="<i4", count=n_params, offset=zo.value).copy(),
    }


def gptq_to_b200(packed: np.ndarray, scales: np.ndarray, zps: np.ndarray, rows: int, cols: int, group: int):
    N, K = rows, cols
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    zps = np.ascontiguousarray(zps, dtype=np.int32)
    p = np.zeros((K // 8, N), dtype=np.uint32)
    s = np.zeros((K // group, N), dtype=np.uint16)
    z = np.zeros((K // group, (N + 7) // 8), dtype=np.uint32)
    inexact = lib().oracle_gptq_to_b200(_p(packed), _p(scales), _p(zps), rows, cols, group, _p(p), _p(s), _p(z))
    if inexact < 0:
        raise ValueError("zero point outside 0..15")
    return p, s, z, int(inexact)

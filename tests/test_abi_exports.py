"""The C-ABI library loads and exports every symbol include/t0b200.h declares (no compute calls)."""
import ctypes
import os
import re
import subprocess


def _declared_functions(header_path):
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(t0_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(t0):
    names = _declared_functions(t0.HEADER_PATH)
    assert len(names) > 60
    lib = ctypes.CDLL(t0.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_static_library_is_built(t0):
    assert os.path.exists(os.path.join(os.path.dirname(t0.LIB_PATH), "libt0b200.a"))


def test_struct_sizes_match_the_header(t0, tmp_path):
    # the ctypes mirrors must have the sizes the C compiler gives the records declared in the header
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include "t0b200.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu %zu\\n",'
                   'sizeof(t0_gemm_config),sizeof(t0_tile_gemm),sizeof(t0_gemm_args),sizeof(t0_w4a16_args),'
                   'sizeof(t0_tile_config),sizeof(t0_tile_cost),sizeof(t0_warp_layout));return 0;}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", os.path.dirname(t0.HEADER_PATH), str(src), "-o", str(exe)], check=True)
    sizes = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [ctypes.sizeof(t0.GemmConfig), ctypes.sizeof(t0.TileGemm), ctypes.sizeof(t0.GemmArgs), ctypes.sizeof(t0.W4A16Args),
                     ctypes.sizeof(t0.TileConfig), ctypes.sizeof(t0.TileCost), ctypes.sizeof(t0.WarpLayout)]
    assert t0.lib().t0_version() >= 100


def test_rust_bindings_cover_the_header(t0):
    # rust-gpu_b200/rust/ffi.rs is generated from the header; it must be current and declare every entry point
    import sys
    here = os.path.join(os.path.dirname(t0.LIB_PATH), "..", "rust")
    r = subprocess.run([sys.executable, os.path.join(here, "gen_ffi.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    text = open(os.path.join(here, "ffi.rs")).read()
    missing = [n for n in _declared_functions(t0.HEADER_PATH) if f"pub fn {n}(" not in text]
    assert not missing, missing
    for record in ("t0_gemm_config", "t0_tile_gemm", "t0_gemm_args", "t0_w4a16_args", "t0_tile_config", "t0_tile_cost", "t0_warp_layout"):
        assert f"pub struct {record} {{" in text

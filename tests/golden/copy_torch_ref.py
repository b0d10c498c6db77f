"""Copies the reference's PyTorch golden vectors into tests/golden/torch_ref/.

Usage: python tests/golden/copy_torch_ref.py <path to the clearnature/rust-gpu checkout>
The files are data (bf16/f32 little-endian arrays), copied byte for byte.
"""
import os
import shutil
import sys

FILES = ["x.bin", "w_gate.bin", "w_up.bin", "w_down.bin", "h_gate_f32ref.bin", "h_up_f32ref.bin",
         "h_gate_bf16acc.bin", "h_up_bf16acc.bin", "swiglu_bf16_trunc.bin", "y_bf16_f32acc.bin", "meta.txt"]

if __name__ == "__main__":
    src = os.path.join(sys.argv[1], "benchmarks", "torch_ref")
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch_ref")
    os.makedirs(dst, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
    print(f"copied {len(FILES)} files to {dst}")

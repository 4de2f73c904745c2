"""Builds oracle/_ref/libcurand_pin.so from oracle/curand_pin.cu (test infrastructure: the real cuRAND generator the
sampling oracle is pinned against).  Usage: python oracle/build_ref.py"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "curand_pin.cu")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libcurand_pin.so")
    if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    os.makedirs(out_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-use_fast_math", "-shared",
                    "-Xcompiler", "-fPIC", "-o", out, src, "-lcudart"], check=True)
    return out


if __name__ == "__main__":
    print(build(force=True))

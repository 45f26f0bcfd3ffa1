"""Recipe for oracle/_ref/libref_kernels.so: the reference's dependency-free CUDA kernels
(softmax.cuh, permute.cuh), compiled for sm_100a from the sources where they lie in the reference
checkout. TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [<reference checkout>]

The rest of the reference's kernel layer cannot be built this way: every GEMM / bmm / attention
source includes CUTLASS headers from a submodule that the checkout does not contain, layernorm
includes cub and cutlass/fast_math.h, and the fast_gelu of custom_math.cuh is a CUTLASS functor.
Outputs go to oracle/_ref/ only (ignored by git). Returns the library path, or None when no
reference checkout is present (then the GPU tests that use it skip).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import Optional

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
LIB = OUT_DIR / "libref_kernels.so"
DEFAULT_REFERENCE = "/root/reference"


def build(reference: Optional[str] = None, verbose: bool = False) -> Optional[Path]:
    ref = Path(reference or os.environ.get("AIT_REFERENCE_ROOT", DEFAULT_REFERENCE))
    inc = ref / "python" / "aitemplate" / "backend" / "cuda"
    if not (inc / "softmax" / "softmax.cuh").exists():
        return LIB if LIB.exists() else None
    src = HERE / "ref_kernels.cu"
    newest = max(src.stat().st_mtime, (inc / "softmax" / "softmax.cuh").stat().st_mtime,
                 (inc / "tensor" / "permute.cuh").stat().st_mtime)
    if LIB.exists() and LIB.stat().st_mtime >= newest:
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-shared",
           "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", str(inc), "-I", str(ref / "static" / "include"), str(src), "-o", str(LIB)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"reference kernels failed to compile:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True))

"""TEST INFRASTRUCTURE.  Compiles the reference's own CUDA kernel files, where
they lie in the reference checkout, together with oracle/ref_kernels_wrapper.cu
into oracle/_ref/libet_ref_kernels.so (sm_100a).  Only cuda/cuda_kernels.cu and
cuda/attention.cu are built, straight with nvcc: the reference's CMake build
and its TensorFlow op are not used (TensorFlow is absent).  -DNDEBUG as in the
reference's own build, whose launcher asserts contradict BERT sizes.

The result is a checker for the GPU tests (tests/test_reference_kernels_gpu.py);
it is never loaded by the product.  Usage: python oracle/build_ref.py [reference_dir]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libet_ref_kernels.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def build(reference_dir: str = "/root/reference") -> str | None:
    srcs = [os.path.join(reference_dir, "cuda", "cuda_kernels.cu"),
            os.path.join(reference_dir, "cuda", "attention.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return LIB if os.path.exists(LIB) else None       # no reference checkout here: keep what is built
    wrapper = os.path.join(HERE, "ref_kernels_wrapper.cu")
    deps = srcs + [wrapper]
    if os.path.exists(LIB) and all(os.path.getmtime(d) <= os.path.getmtime(LIB) for d in deps):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-DNDEBUG", "-w",
           "-Xcompiler", "-fPIC", "-shared", "-I", reference_dir, "-I", os.path.join(reference_dir, "cuda"),
           "-o", LIB, wrapper] + srcs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("building the reference kernels failed")
    return LIB


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))

"""Build libb200fp8.so in-tree with nvcc for sm_100a.

Usage: python -m tritonbench_b200.csrc.build [--force] [--verbose]
The library is written next to this file; it links the CUDA runtime statically and needs
nothing but the NVIDIA driver at run time.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["api.cu", "gemm_tc.cu", "gemm_skinny.cu", "gemm_simt.cu", "quantize.cu", "fused_quantize.cu", "gemm_splitk.cu", "gemm_blockwise.cu", "gemm_gemv.cu"]
HEADERS = ["ptx.cuh", "kernels.h", "streamk.cuh", "nanmax.cuh", os.path.join("..", "..", "include", "b200fp8.h")]
LIB_NAME = "libb200fp8.so"


def lib_path() -> str:
    return os.path.join(HERE, LIB_NAME)


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the library cannot be built on this machine")
    return nvcc


def needs_build() -> bool:
    out = lib_path()
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    deps = [os.path.join(HERE, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    out = lib_path()
    if not force and not needs_build():
        return out
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-lineinfo", "-O3", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC",
        "-cudart", "static",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", out] + [os.path.join(HERE, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

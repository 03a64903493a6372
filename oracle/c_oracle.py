"""ctypes access to the plain-C oracle (liboracle_fp8.so).  TEST INFRASTRUCTURE ONLY."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "liboracle_fp8.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "fp8_rowwise_oracle.c")
    if force or not os.path.exists(_PATH) or os.path.getmtime(_PATH) < os.path.getmtime(src):
        cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        subprocess.run(["make", "-C", _HERE, "-B", f"CC={cc}", "liboracle_fp8.so"], check=True, capture_output=True)
    return _PATH


def load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(build())
        lib.oracle_e4m3_to_f32.restype = ctypes.c_float
        lib.oracle_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        lib.oracle_f32_to_e4m3.restype = ctypes.c_uint8
        lib.oracle_f32_to_e4m3.argtypes = [ctypes.c_float]
        lib.oracle_row_quantize_f32.restype = None
        lib.oracle_row_quantize_f32.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
        lib.oracle_gemm_rowwise.restype = ctypes.c_int
        lib.oracle_gemm_rowwise.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int64] * 3
        _lib = lib
    return _lib


def gemm_rowwise(xq: np.ndarray, wq: np.ndarray, xs: np.ndarray, ws: np.ndarray, bias_bits=None) -> np.ndarray:
    """uint8 [M,K], uint8 [N,K], float32 [M], float32 [N], optional uint16 bf16 bits [N] -> uint16 bf16 bits [M,N]"""
    xq = np.ascontiguousarray(xq, dtype=np.uint8)
    wq = np.ascontiguousarray(wq, dtype=np.uint8)
    xs = np.ascontiguousarray(xs, dtype=np.float32)
    ws = np.ascontiguousarray(ws, dtype=np.float32)
    m, k = xq.shape
    n = wq.shape[0]
    y = np.empty((m, n), dtype=np.uint16)
    b = None
    if bias_bits is not None:
        bias_bits = np.ascontiguousarray(bias_bits, dtype=np.uint16)
        b = bias_bits.ctypes.data
    rc = load().oracle_gemm_rowwise(xq.ctypes.data, wq.ctypes.data, xs.ctypes.data, ws.ctypes.data, b, y.ctypes.data, m, n, k)
    if rc != 0:
        raise MemoryError("oracle_gemm_rowwise could not allocate scratch memory")
    return y


def row_quantize(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.shape, dtype=np.uint8)
    s = np.empty(x.shape[0], dtype=np.float32)
    load().oracle_row_quantize_f32(x.ctypes.data, x.shape[0], x.shape[1], q.ctypes.data, s.ctypes.data)
    return q, s

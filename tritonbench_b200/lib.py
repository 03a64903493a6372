"""ctypes binding of libb200fp8.so (the C ABI in include/b200fp8.h).

The library is the product: if it is missing or does not load, everything that needs it raises.
There is no CPU or PyTorch fallback behind these calls.
"""
import ctypes
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libb200fp8.so")

OK = 0
BAD_ARG = 1
UNSUPPORTED_ARCH = 2
UNSUPPORTED_ALIGNMENT = 3
WORKSPACE_TOO_SMALL = 4
LAUNCH_FAILED = 5
DEVICE_TIMEOUT = 6
TOO_LARGE = 7

VARIANT_AUTO = 0
VARIANT_TC_1CTA = 1
VARIANT_TC_2CTA = 2
VARIANT_SKINNY = 3
VARIANT_SIMT = 4
VARIANT_TC_SPLITK = 5
VARIANT_GEMV = 6
FLAG_NO_TMA_STORE = 0x10
FLAG_PDL = 0x20
FLAG_OUT_FP16 = 0x40


def flag_splitk_config(block_n: int, split: int) -> int:
    """B200FP8_FLAG_SPLITK_CONFIG(block_n, split): force the tc_splitk tile width and cluster size (0 = library's choice)."""
    return ((block_n // 16) << 8) | (split << 13)


DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2
QUANT_OPERATOR, QUANT_FP32 = 0, 1
PRODUCER_RMS_NORM, PRODUCER_SILU_MUL = 1, 2
VARIANTS = {
    "auto": VARIANT_AUTO,
    "tc_1cta": VARIANT_TC_1CTA,
    "tc_2cta": VARIANT_TC_2CTA,
    "skinny": VARIANT_SKINNY,
    "simt": VARIANT_SIMT,
    "tc_splitk": VARIANT_TC_SPLITK,
    "gemv": VARIANT_GEMV,
}
WORKSPACE_HEADER_BYTES = 256
IPC_HANDLE_BYTES = 64

# every symbol include/b200fp8.h declares
EXPORTED_SYMBOLS = (
    "b200fp8_abi_version",
    "b200fp8_status_string",
    "b200fp8_last_cuda_error",
    "b200fp8_workspace_bytes",
    "b200fp8_workspace_init",
    "b200fp8_gemm_rowwise",
    "b200fp8_query_status",
    "b200fp8_describe_plan",
    "b200fp8_host_ctx_create",
    "b200fp8_host_ctx_destroy",
    "b200fp8_gemm_rowwise_host",
    "b200fp8_host_ctx_set_weights",
    "b200fp8_host_ctx_set_panels",
    "b200fp8_gemm_rowwise_noalloc",
    "b200fp8_gemm_rowwise_gather",
    "b200fp8_shared_buffer_create",
    "b200fp8_shared_buffer_open",
    "b200fp8_shared_buffer_close",
    "b200fp8_shared_buffer_destroy",
    "b200fp8_noalloc_status",
    "b200fp8_row_quantize",
    "b200fp8_fused_row_quantize",
    "b200fp8_block_quantize",
    "b200fp8_gemm_rowwise_grouped",
    "b200fp8_selftest_wait_timeout",
    "b200fp8_gemm_blockwise",
)

_lib: Optional[ctypes.CDLL] = None


class B200Fp8Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def load() -> ctypes.CDLL:
    """Load the shared library once and declare the argument types of every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m tritonbench_b200.csrc.build` "
            "(needs nvcc); there is no fallback implementation"
        )
    lib = ctypes.CDLL(LIB_PATH)
    c_void_p, c_int64, c_size_t, c_uint32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_size_t, ctypes.c_uint32
    lib.b200fp8_abi_version.restype = ctypes.c_int
    lib.b200fp8_abi_version.argtypes = []
    lib.b200fp8_status_string.restype = ctypes.c_char_p
    lib.b200fp8_status_string.argtypes = [ctypes.c_int]
    lib.b200fp8_last_cuda_error.restype = ctypes.c_int
    lib.b200fp8_last_cuda_error.argtypes = []
    lib.b200fp8_workspace_bytes.restype = c_size_t
    lib.b200fp8_workspace_bytes.argtypes = [c_int64, c_int64, c_int64, c_uint32]
    lib.b200fp8_workspace_init.restype = ctypes.c_int
    lib.b200fp8_workspace_init.argtypes = [c_void_p, c_size_t, c_void_p]
    lib.b200fp8_gemm_rowwise.restype = ctypes.c_int
    lib.b200fp8_gemm_rowwise.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
        c_void_p, c_size_t, c_uint32, c_void_p,
    ]
    lib.b200fp8_query_status.restype = ctypes.c_int
    lib.b200fp8_query_status.argtypes = [c_void_p, ctypes.POINTER(c_uint32)]
    lib.b200fp8_describe_plan.restype = ctypes.c_int
    lib.b200fp8_describe_plan.argtypes = [c_int64, c_int64, c_int64, c_uint32, ctypes.c_char_p, c_size_t]
    lib.b200fp8_host_ctx_create.restype = ctypes.c_int
    lib.b200fp8_host_ctx_create.argtypes = [c_int64, c_int64, c_int64, c_uint32, ctypes.POINTER(c_void_p)]
    lib.b200fp8_host_ctx_destroy.restype = ctypes.c_int
    lib.b200fp8_host_ctx_destroy.argtypes = [c_void_p]
    lib.b200fp8_gemm_rowwise_host.restype = ctypes.c_int
    lib.b200fp8_gemm_rowwise_host.argtypes = [c_void_p] * 7
    lib.b200fp8_host_ctx_set_weights.restype = ctypes.c_int
    lib.b200fp8_host_ctx_set_weights.argtypes = [c_void_p] * 4
    lib.b200fp8_host_ctx_set_panels.restype = ctypes.c_int
    lib.b200fp8_host_ctx_set_panels.argtypes = [c_void_p, c_int64, c_int64]
    lib.b200fp8_gemm_rowwise_noalloc.restype = ctypes.c_int
    lib.b200fp8_gemm_rowwise_noalloc.argtypes = [c_void_p] * 6 + [c_int64] * 6 + [c_void_p]
    lib.b200fp8_gemm_rowwise_gather.restype = ctypes.c_int
    lib.b200fp8_gemm_rowwise_gather.argtypes = (
        [c_void_p] * 5 + [ctypes.POINTER(c_void_p), ctypes.c_int] + [c_int64] * 6 + [c_void_p, c_size_t, c_uint32, c_void_p]
    )
    lib.b200fp8_shared_buffer_create.restype = ctypes.c_int
    lib.b200fp8_shared_buffer_create.argtypes = [c_size_t, ctypes.POINTER(c_void_p), c_void_p, c_size_t]
    lib.b200fp8_shared_buffer_open.restype = ctypes.c_int
    lib.b200fp8_shared_buffer_open.argtypes = [c_void_p, c_size_t, ctypes.POINTER(c_void_p)]
    lib.b200fp8_shared_buffer_close.restype = ctypes.c_int
    lib.b200fp8_shared_buffer_close.argtypes = [c_void_p]
    lib.b200fp8_shared_buffer_destroy.restype = ctypes.c_int
    lib.b200fp8_shared_buffer_destroy.argtypes = [c_void_p]
    lib.b200fp8_noalloc_status.restype = ctypes.c_int
    lib.b200fp8_noalloc_status.argtypes = [ctypes.POINTER(c_uint32)]
    lib.b200fp8_gemm_rowwise_grouped.restype = ctypes.c_int
    lib.b200fp8_gemm_rowwise_grouped.argtypes = (
        [c_void_p] * 5 + [c_int64] + [c_void_p] + [c_int64] * 6 + [c_void_p, c_size_t, c_uint32, c_void_p]
    )
    lib.b200fp8_selftest_wait_timeout.restype = ctypes.c_int
    lib.b200fp8_selftest_wait_timeout.argtypes = [c_void_p, c_uint32, c_void_p]
    lib.b200fp8_gemm_blockwise.restype = ctypes.c_int
    lib.b200fp8_gemm_blockwise.argtypes = [c_void_p] * 5 + [c_int64] * 8 + [c_void_p, c_size_t, c_uint32, c_void_p]
    lib.b200fp8_fused_row_quantize.restype = ctypes.c_int
    lib.b200fp8_fused_row_quantize.argtypes = [ctypes.c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                               ctypes.c_float, ctypes.c_int, c_void_p, c_int64, c_void_p, c_void_p]
    lib.b200fp8_block_quantize.restype = ctypes.c_int
    lib.b200fp8_block_quantize.argtypes = [c_void_p, ctypes.c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p,
                                           c_int64, c_void_p]
    lib.b200fp8_row_quantize.restype = ctypes.c_int
    lib.b200fp8_row_quantize.argtypes = [c_void_p, ctypes.c_int, ctypes.c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p]
    if lib.b200fp8_abi_version() != 1:
        raise RuntimeError("libb200fp8.so has an ABI version this binding does not know")
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().b200fp8_status_string(status).decode()


def check(status: int, what: str) -> None:
    """Raise for a non-zero status. Unsupported shapes map to NotImplementedError, which the
    TritonBench harness prints as "not supported" (tritonbench/utils/triton_op.py:1502-1503)."""
    if status == OK:
        return
    msg = f"{what}: {status_string(status)} (status {status}"
    if status == LAUNCH_FAILED:
        msg += f", cuda error {load().b200fp8_last_cuda_error()}"
    msg += ")"
    if status in (UNSUPPORTED_ALIGNMENT, TOO_LARGE):
        raise NotImplementedError(msg)
    raise B200Fp8Error(status, msg)


def describe_plan(m: int, n: int, k: int, flags: int = 0) -> str:
    buf = ctypes.create_string_buffer(512)
    check(load().b200fp8_describe_plan(m, n, k, flags, buf, len(buf)), "describe_plan")
    return buf.value.decode()

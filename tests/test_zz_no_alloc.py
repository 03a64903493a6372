"""The entry point for hosts that may not allocate device memory (b200fp8_gemm_rowwise_noalloc).

Some hosts give every byte of HBM to their own arena and refuse any cudaMalloc from a library, so
they can neither let the library allocate nor carve out a workspace to pass in.  For them the decode
kernel can run on a fixed 8 MiB scratch array that is part of the loaded library.  This test calls
that entry point through the C ABI (ctypes, no torch wrapper around the call) twice in a row and
checks each result against the regular entry point given a caller-owned workspace, within the
tolerance every GPU test here uses (1 bf16 ulp + 1e-2 * RMS).  The second call matters: the array
keeps the first call's contents.  This file is collected last on purpose.
"""
import ctypes

import pytest
import torch

from oracle import fp8_rowwise_oracle as orc

pytestmark = pytest.mark.gpu


def _call_noalloc(lib_mod, xq, wq, xs, ws, bias, out):
    m, k = xq.shape
    n = wq.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    return lib_mod.load().b200fp8_gemm_rowwise_noalloc(
        xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), bias.data_ptr() if bias is not None else None,
        out.data_ptr(), m, n, k, xq.stride(0), wq.stride(0), out.stride(0), stream,
    )


def _call_regular(lib_mod, xq, wq, xs, ws, bias, out, workspace):
    m, k = xq.shape
    n = wq.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    return lib_mod.load().b200fp8_gemm_rowwise(
        xq.data_ptr(), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), bias.data_ptr() if bias is not None else None,
        out.data_ptr(), m, n, k, xq.stride(0), wq.stride(0), out.stride(0),
        workspace.data_ptr(), workspace.numel(), lib_mod.VARIANT_SKINNY, stream,
    )


def test_noalloc_entry_point_matches_regular_entry_point_twice_in_a_row(cuda_device):
    from tritonbench_b200 import lib as lib_mod
    from tritonbench_b200 import quantize

    cdll = lib_mod.load()
    # two different decode shapes, so that the second call finds the first call's leftovers
    cases = [(16, 4096, 2048, True), (5, 2304, 2304, False)]
    for (m, n, k, with_bias) in cases:
        xq, wq, xs, ws = [t.cuda() for t in quantize.make_inputs(m, n, k, device="cpu", x_seed=m, w_std=0.02)]
        bias = torch.randn(n, device="cuda").to(torch.bfloat16) if with_bias else None
        workspace = torch.zeros(cdll.b200fp8_workspace_bytes(m, n, k, lib_mod.VARIANT_SKINNY), dtype=torch.uint8, device="cuda")
        want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        assert _call_regular(lib_mod, xq, wq, xs, ws, bias, want, workspace) == lib_mod.OK
        for call in range(2):
            got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            before = torch.cuda.memory_allocated()
            assert _call_noalloc(lib_mod, xq, wq, xs, ws, bias, got) == lib_mod.OK
            assert torch.cuda.memory_allocated() == before
            torch.cuda.synchronize()
            word = ctypes.c_uint32(123)
            assert cdll.b200fp8_noalloc_status(ctypes.byref(word)) == lib_mod.OK and word.value == 0
            res = orc.compare(got, want)
            assert res["ok"], (m, n, k, call, res)
        # and against the CPU oracle, like every other kernel test
        ref = orc.gemm_rowwise(xq.cpu(), wq.cpu(), xs.cpu(), ws.cpu(), bias.cpu() if bias is not None else None)
        assert orc.compare(got, ref)["ok"]


def test_noalloc_entry_point_rejects_what_does_not_fit(cuda_device):
    from tritonbench_b200 import lib as lib_mod

    cdll = lib_mod.load()
    one = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = one.data_ptr()
    f = cdll.b200fp8_gemm_rowwise_noalloc
    # more than 128 rows: not a decode shape
    assert f(p, p, p, p, None, p, 129, 256, 256, 256, 256, 256, None) == lib_mod.TOO_LARGE
    # partial sums of 128 tokens x 28672 columns need more than the 8 MiB array
    assert cdll.b200fp8_workspace_bytes(128, 28672, 8192, lib_mod.VARIANT_SKINNY) > (8 << 20)
    assert f(p, p, p, p, None, p, 128, 28672, 8192, 8192, 8192, 28672, None) == lib_mod.TOO_LARGE
    assert f(None, p, p, p, None, p, 16, 256, 256, 256, 256, 256, None) == lib_mod.BAD_ARG
    assert lib_mod.status_string(lib_mod.TOO_LARGE) == "size exceeds the supported maximum"

"""The CUDA rowwise quantiser against the reference's own quantiser (golden fixtures) and the oracle:
byte-exact codes and bit-exact scales."""
import os

import numpy as np
import pytest
import torch

from oracle import fp8_rowwise_oracle as orc

pytestmark = pytest.mark.gpu


def _bf16(bits):
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def _same(q, s, q_want, s_want, what):
    assert torch.equal(q.view(torch.uint8).cpu(), q_want.view(torch.uint8).cpu()), what
    assert torch.equal(s.cpu(), s_want.cpu()), what


def test_matches_reference_fixture_bit_for_bit(cuda_device, golden_dir):
    from tritonbench_b200 import ops

    d = np.load(os.path.join(golden_dir, "ref_quantizer_bf16_128x256x512.npz"))
    for xk, qk, sk in (("x_bf16", "xq", "x_scale"), ("w_bf16", "wq", "w_scale")):
        q, s = ops.fp8_row_quantize(_bf16(d[xk]).cuda())
        assert np.array_equal(q.view(torch.uint8).cpu().numpy(), d[qk])
        assert np.array_equal(s.cpu().numpy(), d[sk])


@pytest.mark.parametrize("name,dtype", [("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)])
def test_edge_rows_match_reference_fixture(cuda_device, golden_dir, name, dtype):
    from tritonbench_b200 import ops

    d = np.load(os.path.join(golden_dir, "ref_quantizer_edge_rows.npz"))
    q, s = ops.fp8_row_quantize(torch.from_numpy(d["rows"]).to(dtype).cuda())
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), d[f"q_{name}"])
    assert np.array_equal(s.cpu().numpy(), d[f"s_{name}"], equal_nan=True)


@pytest.mark.parametrize("shape", [(1, 16), (3, 7), (17, 130), (64, 8192), (5, 16384), (2, 40000), (300, 1000), (1024, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_operator_recipe_matches_oracle_on_random_and_ragged_rows(cuda_device, shape, dtype):
    from tritonbench_b200 import ops

    g = torch.Generator().manual_seed(shape[0] * 7 + shape[1])
    x = (torch.randn(shape, generator=g) * torch.rand((shape[0], 1), generator=g) * 50).to(dtype)
    x[0, 0] = 0.0
    q_want, s_want = orc.row_quantize_reference(x)
    q, s = ops.fp8_row_quantize(x.cuda())
    _same(q, s, q_want, s_want, f"{shape} {dtype}")


def test_fp32_recipe_matches_oracle_and_feeds_the_gemm(cuda_device):
    from tritonbench_b200 import ops, quantize

    g = torch.Generator().manual_seed(4)
    x = torch.randn((257, 1040), generator=g)
    w = torch.randn((520, 1040), generator=g) * 0.02
    x[5] = 0.0
    xq, xs = ops.fp8_row_quantize(x.cuda(), recipe="fp32")
    wq, ws = ops.fp8_row_quantize(w.cuda(), recipe="fp32")
    _same(xq, xs, *orc.row_quantize(x), "x fp32 recipe")
    _same(wq, ws, *orc.row_quantize(w), "w fp32 recipe")
    _same(xq, xs, *quantize.fp8_row_quantize_fp32(x), "host-side product quantiser")
    y = ops.fp8_gemm_rowwise(xq, wq, xs, ws)
    assert orc.compare(y, orc.gemm_rowwise(xq, wq, xs, ws))["ok"]


def test_strided_input_and_unaligned_rows(cuda_device):
    from tritonbench_b200 import ops

    g = torch.Generator().manual_seed(9)
    big = torch.randn((40, 300), generator=g).to(torch.bfloat16).cuda()
    for view in (big[:, :256], big[:, 3:259], big[:, :77]):
        q, s = ops.fp8_row_quantize(view)
        _same(q, s, *orc.row_quantize_reference(view.cpu()), str(view.shape))


def test_bad_arguments(cuda_device):
    from tritonbench_b200 import ops

    with pytest.raises(ValueError):
        ops.fp8_row_quantize(torch.zeros((4, 4), device="cuda", dtype=torch.int32))
    with pytest.raises(ValueError):
        ops.fp8_row_quantize(torch.zeros((4, 4), dtype=torch.bfloat16))
    with pytest.raises(Exception):
        ops.fp8_row_quantize(torch.zeros((4, 16), device="cuda", dtype=torch.bfloat16), recipe="fp32")

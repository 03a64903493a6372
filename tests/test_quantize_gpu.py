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


def _canon_nan_codes(q):
    """e4m3 codes with both NaN patterns (0x7F, 0xFF) mapped to 0x7F: the sign of a NaN is not part of the contract."""
    q = np.asarray(q, dtype=np.uint8)
    return np.where((q & 0x7F) == 0x7F, np.uint8(0x7F), q)


@pytest.mark.parametrize("name,dtype", [("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)])
def test_rows_with_nan_and_infinity_match_reference_fixture(cuda_device, golden_dir, name, dtype):
    """torch's max / clamp propagate NaN: one NaN makes the row's scale and all of its codes NaN; an infinity gives an
    infinite scale, zero codes and a NaN where the infinity was.  Fixture made by the reference's own function."""
    from tritonbench_b200 import ops

    d = np.load(os.path.join(golden_dir, "ref_quantizer_nonfinite.npz"))
    q, s = ops.fp8_row_quantize(torch.from_numpy(d["rows"]).to(dtype).cuda())
    assert np.array_equal(_canon_nan_codes(q.view(torch.uint8).cpu().numpy()), _canon_nan_codes(d[f"q_{name}"]))
    assert np.array_equal(s.cpu().numpy(), d[f"s_{name}"], equal_nan=True)
    qb, sb = ops.fp8_block_quantize(_bf16(d["block_x_bf16"]).cuda())
    assert np.array_equal(_canon_nan_codes(qb.view(torch.uint8).cpu().numpy()), _canon_nan_codes(d["block_q"]))
    assert np.array_equal(sb.cpu().numpy(), d["block_scale"], equal_nan=True)


@pytest.mark.parametrize("shape", [(200, 2048), (300, 4096), (5, 16384), (3, 40000), (9, 1001)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_nan_and_infinity_in_every_kernel_form(cuda_device, shape, dtype):
    """The same rule in the warp-per-row, persistent and CTA-per-row kernels (and their tails), against the oracle."""
    from tritonbench_b200 import ops

    g = torch.Generator().manual_seed(shape[1])
    x = torch.randn(shape, generator=g).to(dtype)
    x[0, shape[1] - 1] = float("nan")
    x[1, shape[1] // 2] = float("inf")
    x[2, 0] = float("-inf")
    q_want, s_want = orc.row_quantize_reference(x)
    q, s = ops.fp8_row_quantize(x.cuda())
    assert np.array_equal(_canon_nan_codes(q.view(torch.uint8).cpu().numpy()), _canon_nan_codes(q_want.view(torch.uint8).numpy()))
    assert np.array_equal(s.cpu().numpy(), s_want.numpy(), equal_nan=True)


# the later ones sit on either side of the boundaries between the three kernels (one warp per row up to 2560 elements and
# from 64 rows, persistent with one warp per 1024 elements up to 16384, one CTA per row beyond) and make a persistent
# CTA walk over many rows
@pytest.mark.parametrize("shape", [(1, 16), (3, 7), (17, 130), (64, 8192), (5, 16384), (2, 40000), (300, 1000), (1024, 4096),
                                   (63, 2048), (64, 2048), (200, 2560), (200, 2568), (3000, 2816), (200, 8200), (77, 512), (5000, 8192),
                                   (2000, 5120), (900, 13312), (700, 16384), (50, 16392)])
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


# ------------------------------------------------------------------ producer + quantiser in one kernel
def _check_fused(q, scale, y_ref):
    """q, scale from the kernel against the oracle's fp32 activation y_ref: the scale is rowabsmax / 448 up to
    the last bits of y, and every code is the oracle's code for y / scale or its neighbour (a last-bit
    difference in y or in the scale may move a value across a rounding boundary)."""
    from oracle import fp8_rowwise_oracle as orc

    q_ref, s_ref = orc.row_quantize(y_ref)
    scale = scale.cpu()
    assert torch.allclose(scale, s_ref, rtol=2e-6, atol=0), (scale - s_ref).abs().max()
    got = orc.decode_e4m3(q.cpu().view(torch.uint8))
    want = orc.decode_e4m3(q_ref.view(torch.uint8))
    differ = got != want
    assert differ.float().mean().item() < 2e-3, differ.float().mean().item()
    # a differing code is the neighbouring e4m3 value: at most one step of 2^-3 relative (or the subnormal step)
    step = torch.maximum(want.abs() * 0.125, torch.full_like(want, 2.0 ** -9))
    assert bool(((got - want).abs() <= step * 1.001).all())


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(16, 8192), (128, 2304), (3, 1000), (5, 20000), (64, 4104), (7, 33), (1500, 4096), (3000, 2816),
                                   # the persistent kernel with 16, 13 and 1 warps per row, and rows enough for its ring to wrap
                                   (300, 16384), (700, 13312), (40000, 512), (4000, 8192)])
@pytest.mark.parametrize("round_bf16", [False, True])
def test_rms_norm_quantiser(cuda_device, shape, round_bf16):
    from oracle import fp8_rowwise_oracle as orc
    from tritonbench_b200 import ops

    rows, cols = shape
    gen = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=gen) * 3).to(torch.bfloat16)
    w = torch.randn(cols, generator=gen).to(torch.bfloat16)
    q, scale = ops.rms_norm_fp8_rowwise_quant(x.cuda(), w.cuda(), eps=1e-5, round_bf16=round_bf16)
    _check_fused(q, scale, orc.rms_norm_rows(x, w, 1e-5, round_bf16))


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(16, 8192), (128, 2304), (3, 1000), (5, 20000), (64, 4104), (7, 33), (1500, 4096), (3000, 2816),
                                   # the persistent kernel with 16, 13 and 1 warps per row, and many rows per CTA
                                   (300, 16384), (700, 13312), (40000, 512), (4000, 8192)])
@pytest.mark.parametrize("round_bf16", [False, True])
def test_silu_mul_quantiser(cuda_device, shape, round_bf16):
    from oracle import fp8_rowwise_oracle as orc
    from tritonbench_b200 import ops

    rows, cols = shape
    gen = torch.Generator().manual_seed(2 * rows + cols)
    x1 = (torch.randn(rows, cols, generator=gen) * 4).to(torch.bfloat16)
    x2 = torch.randn(rows, cols, generator=gen).to(torch.bfloat16)
    q, scale = ops.silu_mul_fp8_rowwise_quant(x1.cuda(), x2.cuda(), round_bf16=round_bf16)
    _check_fused(q, scale, orc.silu_mul_rows(x1, x2, round_bf16))


@pytest.mark.gpu
def test_fused_quantiser_feeds_the_gemm_and_handles_strided_and_zero_rows(cuda_device):
    """End to end: rms_norm -> quantise -> GEMM against the oracle's fp32 pipeline; a row view with a
    pitch larger than its width; an all-zero row (scale = 1e-12 / 448, codes 0)."""
    from oracle import fp8_rowwise_oracle as orc
    from tritonbench_b200 import ops, quantize

    gen = torch.Generator().manual_seed(5)
    m, n, k = 48, 512, 1024
    big = (torch.randn(m, k + 64, generator=gen) * 2).to(torch.bfloat16)
    big[3] = 0
    x = big[:, :k]
    wd = torch.randn(k, generator=gen).to(torch.bfloat16)
    wq, ws = quantize.fp8_row_quantize_fp32(torch.randn(n, k, generator=gen))
    xq, xs = ops.rms_norm_fp8_rowwise_quant(big.cuda()[:, :k], wd.cuda())
    assert float(xs[3]) == pytest.approx(1e-12 / 448, rel=1e-6, abs=0)
    assert int((xq[3].view(torch.uint8) & 0x7F).max()) == 0  # +0 or -0 (zero times a negative weight)
    y = ops.fp8_gemm_rowwise(xq, wq.cuda(), xs, ws.cuda())
    xq_ref, xs_ref = orc.row_quantize(orc.rms_norm_rows(x, wd))
    ref = orc.gemm_rowwise(xq_ref, wq, xs_ref, ws)
    # a handful of activation codes may differ by one step from the oracle's: compare with the e4m3 step in the budget
    err = (y.cpu().float() - ref.float()).abs()
    assert float(err.max()) <= float(orc.tolerance(ref.float()).max()) + 0.05 * float(ref.float().abs().max())
    ops.check_device_status()


# ------------------------------------------------------------------ 128x128 block quantiser
def test_block_quantiser_matches_reference_fixture_bit_for_bit(cuda_device, golden_dir):
    from tritonbench_b200 import ops

    d = np.load(os.path.join(golden_dir, "ref_block_quantizer_200x300.npz"))
    q, s = ops.fp8_block_quantize(_bf16(d["x_bf16"]).cuda())
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), d["q"])
    assert np.array_equal(s.cpu().numpy(), d["scale"])


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (1, 1), (130, 129), (1000, 520), (513, 2048), (4096, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_block_quantiser_matches_oracle(cuda_device, shape, dtype):
    from tritonbench_b200 import ops

    g = torch.Generator().manual_seed(shape[0] + 3 * shape[1])
    x = (torch.randn(shape, generator=g) * 20).to(dtype)
    x[0, 0] = 0.0
    if shape[0] > 128:
        x[128:, :128] = 0.0  # a block of zeros: multiplier 448 / 1e-12
    q_want, s_want = orc.block_quantize_reference(x)
    q, s = ops.fp8_block_quantize(x.cuda())
    _same(q, s, q_want, s_want, f"{shape} {dtype}")
    # a view with a row pitch that breaks the 16-byte alignment takes the element path
    wide = torch.zeros((shape[0], shape[1] + 3), dtype=dtype)
    wide[:, : shape[1]] = x
    q2, s2 = ops.fp8_block_quantize(wide.cuda()[:, : shape[1]])
    _same(q2, s2, q_want, s_want, f"{shape} {dtype} strided")

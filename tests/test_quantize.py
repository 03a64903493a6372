"""Host-side input logic: the product's quantiser and generators against the oracle's."""
import numpy as np
import torch

from oracle import fp8_rowwise_oracle as orc
from tritonbench_b200 import quantize


def test_reference_style_quantizer_matches_oracle_restatement():
    g = torch.Generator().manual_seed(1)
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        x = torch.randn((33, 72), generator=g).to(dt)
        q, s = quantize.fp8_row_quantize(x)
        qo, so = orc.row_quantize_reference(x)
        assert torch.equal(q.view(torch.uint8), qo.view(torch.uint8)) and torch.equal(s, so)
        assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32


def test_fp32_recipe_matches_oracle_and_golden(golden_dir):
    import os

    d = np.load(os.path.join(golden_dir, "config1_seed0_128x256x512.npz"))
    xq, wq, xs, ws = quantize.make_inputs(128, 256, 512, device="cpu", x_seed=0)
    assert np.array_equal(xq.view(torch.uint8).numpy(), d["xq"])
    assert np.array_equal(wq.view(torch.uint8).numpy(), d["wq"])
    assert np.array_equal(xs.numpy(), d["x_scale"]) and np.array_equal(ws.numpy(), d["w_scale"])


def test_generators_are_deterministic_and_shard_seeds_differ():
    a = quantize.make_quantized(64, 128, seed=3)
    b = quantize.make_quantized(64, 128, seed=3)
    c = quantize.make_quantized(64, 128, seed=4)
    assert torch.equal(a[0].view(torch.uint8), b[0].view(torch.uint8)) and torch.equal(a[1], b[1])
    assert not torch.equal(a[0].view(torch.uint8), c[0].view(torch.uint8))


def test_chunked_generation_equals_one_shot():
    a = quantize.make_quantized(100, 64, seed=9, chunk_rows=100)
    b = quantize.make_quantized(100, 64, seed=9, chunk_rows=1000)
    assert torch.equal(a[0].view(torch.uint8), b[0].view(torch.uint8))


def test_student_t_rows_have_heavy_tails_and_never_overflow():
    q, s = quantize.make_quantized(256, 512, seed=0, dist="student_t3")
    v = orc.decode_e4m3(q)
    assert torch.isfinite(v).all() and float(v.abs().max()) == 448.0
    assert float(s.max() / s.median()) > 3.0  # some rows carry a large outlier


def test_every_row_hits_full_scale():
    q, _ = quantize.make_quantized(32, 64, seed=2)
    assert bool((orc.decode_e4m3(q).abs().amax(dim=1) == 448.0).all())


def test_block_quantizer_matches_oracle_restatement():
    g = torch.Generator().manual_seed(6)
    for shape in ((200, 300), (128, 128), (1, 16), (257, 130)):
        x = torch.randn(shape, generator=g).to(torch.bfloat16)
        q, s = quantize.fp8_block_quantize(x)
        qo, so = orc.block_quantize_reference(x)
        assert torch.equal(q.view(torch.uint8), qo.view(torch.uint8)) and torch.equal(s, so)

"""The oracle against the golden fixtures (made by tests/golden/make_golden.py from the reference's
own quantiser) and against itself (Python/torch restatement vs plain-C restatement)."""
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import fp8_rowwise_oracle as orc


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_e4m3_decode_table_matches_torch_for_all_256_bytes(golden_dir):
    want = _load(golden_dir, "e4m3_all_bytes.npz")["values"]
    got = orc.e4m3_decode_table()
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])
    assert np.isnan(got[0x7F]) and np.isnan(got[0xFF])
    assert got[0x7E] == 448.0 and got[0xFE] == -448.0
    assert got[0x01] == 2.0 ** -9 and got[0x00] == 0.0 and got[0x80] == 0.0 and np.signbit(got[0x80])


def test_c_decode_matches_python_decode():
    lib = c_oracle.load()
    table = orc.e4m3_decode_table()
    for b in range(256):
        v = lib.oracle_e4m3_to_f32(b)
        assert (np.isnan(v) and np.isnan(table[b])) or v == table[b]


def test_c_encode_round_trips_every_finite_byte():
    lib = c_oracle.load()
    table = orc.e4m3_decode_table()
    for b in range(256):
        if np.isnan(table[b]):
            continue
        assert lib.oracle_f32_to_e4m3(float(table[b])) == b


def test_c_encode_matches_torch_cast_on_random_values():
    lib = c_oracle.load()
    g = torch.Generator().manual_seed(3)
    for std in (100.0, 1.0, 0.01):
        x = (torch.randn(20000, generator=g) * std).clamp(-448, 448)
        want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        got = np.array([lib.oracle_f32_to_e4m3(float(v)) for v in x.numpy()], dtype=np.uint8)
        assert np.array_equal(got, want)


def test_quantizer_restatement_matches_reference_fixture(golden_dir):
    d = _load(golden_dir, "ref_quantizer_bf16_128x256x512.npz")
    for name, qname, sname in (("x_bf16", "xq", "x_scale"), ("w_bf16", "wq", "w_scale")):
        x = _bf16(d[name])
        q, s = orc.row_quantize_reference(x)
        assert np.array_equal(q.view(torch.uint8).numpy(), d[qname])
        assert np.array_equal(s.numpy(), d[sname])


@pytest.mark.parametrize("name,dtype", [("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)])
def test_quantizer_restatement_matches_reference_on_edge_rows(golden_dir, name, dtype):
    d = _load(golden_dir, "ref_quantizer_edge_rows.npz")
    q, s = orc.row_quantize_reference(torch.from_numpy(d["rows"]).to(dtype))
    assert np.array_equal(q.view(torch.uint8).numpy(), d[f"q_{name}"])
    assert np.array_equal(s.numpy(), d[f"s_{name}"], equal_nan=True)


def _canon_nan_codes(q):
    """e4m3 codes with both NaN patterns (0x7F, 0xFF) mapped to 0x7F: the sign of a NaN is not part of the contract."""
    q = np.asarray(q, dtype=np.uint8)
    return np.where((q & 0x7F) == 0x7F, np.uint8(0x7F), q)


@pytest.mark.parametrize("name,dtype", [("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)])
def test_quantizer_restatement_matches_reference_on_rows_with_nan_and_infinity(golden_dir, name, dtype):
    """A NaN makes its whole row NaN (scale and codes); an infinity gives scale inf, zero codes and one NaN."""
    d = _load(golden_dir, "ref_quantizer_nonfinite.npz")
    q, s = orc.row_quantize_reference(torch.from_numpy(d["rows"]).to(dtype))
    assert np.array_equal(_canon_nan_codes(q.view(torch.uint8).numpy()), _canon_nan_codes(d[f"q_{name}"]))
    assert np.array_equal(s.numpy(), d[f"s_{name}"], equal_nan=True)
    assert np.isnan(d[f"s_{name}"][[1, 3]]).all() and np.isinf(d[f"s_{name}"][2])
    assert (_canon_nan_codes(d[f"q_{name}"][1]) == 0x7F).all()


def test_block_quantizer_restatement_matches_reference_on_blocks_with_nan_and_infinity(golden_dir):
    d = _load(golden_dir, "ref_quantizer_nonfinite.npz")
    q, s = orc.block_quantize_reference(_bf16(d["block_x_bf16"]))
    assert np.array_equal(_canon_nan_codes(q.view(torch.uint8).numpy()), _canon_nan_codes(d["block_q"]))
    assert np.array_equal(s.numpy(), d["block_scale"], equal_nan=True)


def test_gemm_oracle_matches_golden_outputs_bit_for_bit(golden_dir):
    for f in ("config1_seed0_128x256x512.npz", "ref_quantizer_bf16_128x256x512.npz"):
        d = _load(golden_dir, f)
        y = orc.gemm_rowwise(
            torch.from_numpy(d["xq"]), torch.from_numpy(d["wq"]), torch.from_numpy(d["x_scale"]), torch.from_numpy(d["w_scale"])
        )
        assert torch.equal(y, _bf16(d["y_bf16"]))


def test_cast_decode_equals_table_decode():
    allb = torch.arange(256, dtype=torch.uint8).repeat(4, 1)
    ones = torch.ones(4)
    a = orc.gemm_rowwise(allb[:, :127], allb[:, :127], ones, ones, keep_fp32=True, decode="table")
    b = orc.gemm_rowwise(allb[:, :127], allb[:, :127], ones, ones, keep_fp32=True, decode="cast")
    assert torch.equal(a, b)
    t = orc.decode_e4m3(allb[0])
    c = allb[0].view(torch.float8_e4m3fn).to(torch.float32)
    assert torch.equal(torch.nan_to_num(t, nan=-1.0), torch.nan_to_num(c, nan=-1.0))


def test_c_gemm_oracle_within_tolerance_of_golden(golden_dir):
    # the C oracle adds in ascending k, torch's matmul in blocks: equal up to fp32 summation order
    d = _load(golden_dir, "config1_seed0_128x256x512.npz")
    y = c_oracle.gemm_rowwise(d["xq"], d["wq"], d["x_scale"], d["w_scale"])
    res = orc.compare(_bf16(y.view(np.int16)), _bf16(d["y_bf16"]))
    assert res["ok"], res
    assert res["max_ratio"] < 0.6


def test_c_quantizer_matches_python_benchmark_recipe():
    g = torch.Generator().manual_seed(11)
    x = torch.randn((37, 130), generator=g)
    x[5] = 0.0
    x[7, 3] = 1e6
    q, s = orc.row_quantize(x)
    qc, sc = c_oracle.row_quantize(x.numpy())
    assert np.array_equal(sc, s.numpy())
    assert np.array_equal(qc, q.view(torch.uint8).numpy())


def test_oracles_agree_with_bias_and_ragged_shapes():
    g = torch.Generator().manual_seed(5)
    for (m, n, k) in ((1, 1, 1), (3, 5, 7), (17, 33, 130), (64, 96, 256)):
        xq, xs = orc.row_quantize(torch.randn((m, k), generator=g))
        wq, ws = orc.row_quantize(torch.randn((n, k), generator=g) * 0.02)
        bias = torch.randn(n, generator=g).to(torch.bfloat16)
        yp = orc.gemm_rowwise(xq, wq, xs, ws, bias)
        yc = c_oracle.gemm_rowwise(
            xq.view(torch.uint8).numpy(), wq.view(torch.uint8).numpy(), xs.numpy(), ws.numpy(),
            bias.view(torch.int16).numpy().view(np.uint16),
        )
        assert orc.compare(_bf16(yc.view(np.int16)), yp)["ok"]


def test_zero_row_quantizes_to_zero_bytes_and_tiny_scale():
    q, s = orc.row_quantize(torch.zeros((2, 16)))
    assert int(q.view(torch.uint8).max()) == 0
    assert np.allclose(s.numpy(), 1e-12 / 448.0)


def test_tolerance_is_one_ulp_plus_one_percent_rms():
    ref = torch.tensor([[1.0, 2.0, 3.0, -4.0]])
    rms = float(ref.pow(2).mean().sqrt())
    tol = orc.tolerance(ref)
    want = torch.tensor([[2.0 ** -7, 2.0 ** -6, 2.0 ** -6, 2.0 ** -5]]) + 1e-2 * rms
    assert torch.allclose(tol, want)
    assert orc.compare(ref.to(torch.bfloat16), ref.to(torch.bfloat16))["ok"]
    off = ref.clone()
    off[0, 0] += 0.2
    assert not orc.compare(off.to(torch.bfloat16), ref.to(torch.bfloat16))["ok"]


def test_flops_and_bytes_follow_the_reference_metrics():
    assert orc.flops(128, 256, 512) == 2 * 128 * 256 * 512
    assert orc.flops(128, 256, 512, bias=True) == 2 * 128 * 256 * 512 + 2 * 128 * 256
    assert abs(orc.gbytes(16, 28672, 8192) - (16 * 8192 + 28672 * 8192 + 2 * 16 * 28672) / 1e9) < 1e-12


def test_builtin_shape_list_fixture(golden_dir):
    shapes = _load(golden_dir, "ref_builtin_shapes.npz")["shapes"]
    assert shapes.shape == (20, 3)
    assert tuple(shapes[7]) == (16, 13312, 13312)  # the one shape the reference's run-config tracks


def test_block_quantizer_restatement_matches_reference_fixture(golden_dir):
    d = _load(golden_dir, "ref_block_quantizer_200x300.npz")
    q, s = orc.block_quantize_reference(_bf16(d["x_bf16"]))
    assert np.array_equal(q.view(torch.uint8).numpy(), d["q"])
    assert np.array_equal(s.numpy(), d["scale"])
    assert s.shape == (2, 3)


def test_blockwise_gemm_oracle_reduces_to_rowwise_when_scales_are_uniform():
    g = torch.Generator().manual_seed(2)
    xq, _ = orc.row_quantize(torch.randn((130, 300), generator=g))
    wq, _ = orc.row_quantize(torch.randn((70, 300), generator=g))
    xs = torch.full((2, 3), 0.5)
    ws = torch.full((1, 3), 0.25)
    a = orc.gemm_blockwise(xq, wq, xs, ws)
    b = orc.gemm_rowwise(xq, wq, torch.full((130,), 0.5), torch.full((70,), 0.25))
    assert torch.equal(a, b)

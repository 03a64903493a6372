"""The operator boundary on a B200: our backend next to the baseline column, accuracy = 1."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
METRICS = "latency,tflops,gbps,speedup,accuracy"


def test_standalone_operator_on_gpu(cuda_device):
    from tritonbench_b200 import operator as standalone

    standalone._attach_default_backends()
    for shape in (["--m", "512", "--n", "1024", "--k", "1024"], ["--m", "16", "--n", "4096", "--k", "2048", "--bias"]):
        args, extra = standalone.get_parser().parse_known_args(
            ["--device", "cuda", "--metrics", METRICS, "--only", "torch_dequant_ref,b200_native,scaled_mm", "--iter", "20"] + shape
        )
        res = standalone.Operator(args, extra).run(args.warmup, args.iter)
        _, cells = res.rows[0]
        assert cells["b200_native"]["accuracy"] is True, cells
        assert cells["b200_native"]["latency"] > 0 and cells["b200_native"]["tflops"] > 0
        assert "b200-accuracy" in res.headers() and "b200-speedup" in res.headers()


def test_plugin_through_the_reference_harness_on_gpu(cuda_device):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tritonbench")):
        pytest.skip("no installed copy of the tritonbench package on this machine")
    sys.path.insert(0, ref)
    from tritonbench_b200 import tritonbench_plugin as plug

    out = plug.run(
        ["--op", plug.OP_NAME, "--device", "cuda", "--metrics", METRICS, "--only", "torch_dequant_ref,b200_native",
         "--m", "1024", "--n", "2048", "--k", "1024"]
    )
    text = str(out)
    assert "b200-tflops" in text and "b200-accuracy" in text, text
    x_val, cells = out.result[0][0], out.result[0][1]
    assert tuple(x_val) == (1024, 2048, 1024)
    assert cells["b200_native"].accuracy is True
    assert cells["b200_native"].latency is not None


def test_roofline_columns_through_the_reference_harness(cuda_device):
    """`pct_fp8_peak` and `pct_hbm`: roofline fractions against B200 figures next to the stock metrics."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tritonbench")):
        pytest.skip("no installed copy of the tritonbench package on this machine")
    sys.path.insert(0, ref)
    from tritonbench_b200 import tritonbench_plugin as plug

    out = plug.run(
        ["--op", plug.OP_NAME, "--device", "cuda", "--metrics", "latency,tflops,gbps,pct_fp8_peak,pct_hbm", "--only", "b200_native",
         "--m", "16", "--n", "28672", "--k", "8192"]
    )
    text = str(out)
    assert "b200-pct_fp8_peak" in text and "b200-pct_hbm" in text, text
    cell = out.result[0][1]["b200_native"]
    fp8_peak, hbm = plug._b200_peaks()
    assert abs(cell.extra_metrics["pct_hbm"] - 100.0 * cell.extra_metrics["gbps"] / hbm) < 0.5  # gbps is the operator's own metric
    assert abs(cell.extra_metrics["pct_fp8_peak"] - 100.0 * cell.tflops / fp8_peak) < 0.5
    assert 40.0 < cell.extra_metrics["pct_hbm"] < 110.0  # a decode shape: HBM-bound


def test_fp8_gemm_operator_backend_through_the_reference_harness(cuda_device):
    """The sibling operator `fp8_gemm`: our column next to its own torch._scaled_mm baseline, both output types."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tritonbench")):
        pytest.skip("no installed copy of the tritonbench package on this machine")
    sys.path.insert(0, ref)
    from tritonbench_b200 import tritonbench_plugin as plug

    for extra in ([], ["--scaling_rowwise"]):
        out = plug.run(
            ["--op", "fp8_gemm", "--device", "cuda", "--metrics", "latency,tflops,speedup,accuracy", "--only",
             "torch_fp8_gemm,b200_native", "--m", "1024", "--n", "2048", "--k", "1024"] + extra
        )
        assert "b200-tflops" in str(out)
        cells = out.result[0][1]
        assert cells["b200_native"].accuracy is True, extra


def test_grouped_operator_backend_through_the_reference_harness(cuda_device):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tritonbench")):
        pytest.skip("no installed copy of the tritonbench package on this machine")
    sys.path.insert(0, ref)
    from tritonbench_b200 import tritonbench_plugin as plug

    out = plug.run(
        ["--op", "fp8_gemm_rowwise_grouped", "--device", "cuda", "--metrics", "latency,tflops,speedup,accuracy", "--only",
         "torch_dequant_ref,b200_native", "--m", "2048", "--n", "1024", "--k", "1024", "--group_size", "4"]
    )
    assert "b200-tflops" in str(out)
    cells = out.result[0][1]
    assert cells["b200_native"].accuracy is True


def test_blockwise_operator_backend_through_the_reference_harness(cuda_device):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tritonbench")):
        pytest.skip("no installed copy of the tritonbench package on this machine")
    sys.path.insert(0, ref)
    from tritonbench_b200 import tritonbench_plugin as plug

    out = plug.run(
        ["--op", "fp8_gemm_blockwise", "--device", "cuda", "--metrics", "latency,tflops,speedup,accuracy", "--only",
         "torch_dequant_ref,b200_native", "--m", "2048", "--n", "2048", "--k", "2048"]
    )
    assert "b200-tflops" in str(out)
    cells = out.result[0][1]
    assert cells["b200_native"].accuracy is True


@pytest.mark.parametrize("backend", ["b200_rms_norm_fused", "b200_rms_norm_quant", "b200_silu_mul_fused", "b200_silu_mul_quant"])
def test_fused_quant_operator_backends_through_the_reference_harness(cuda_device, backend):
    """`--op fp8_fused_quant_gemm_rowwise`: RMS norm (or SiLU-mul) + quantiser in one kernel, then the GEMM; each of
    the four backends against the torch pipeline of its own definition, at the tolerance derived from one e4m3
    step on a small fraction of the activations (atol 0.1 sqrt(K), a tenth of an output's sigma; rtol 1.6e-2)."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tritonbench")):
        pytest.skip("no installed copy of the tritonbench package on this machine")
    sys.path.insert(0, ref)
    from tritonbench_b200 import tritonbench_plugin as plug

    baseline = plug.FUSED_BASELINES[backend]
    for shape in (["--m", "64", "--n", "1024", "--k", "2048"], ["--m", "512", "--n", "768", "--k", "4096"]):
        out = plug.run(
            ["--op", "fp8_fused_quant_gemm_rowwise", "--device", "cuda", "--metrics", "latency,tflops,accuracy", "--baseline", baseline,
             "--only", f"{baseline},{backend}"] + shape
        )
        cells = out.result[0][1]
        assert cells[backend].accuracy is True, (backend, shape)
        assert cells[backend].latency is not None
    atol, rtol = plug.fused_quant_tolerance(2048)
    assert abs(atol - 4.525) < 1e-3 and rtol == 1.6e-2

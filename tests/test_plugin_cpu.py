"""Host-side boundary logic on CPU: the plugin against the real TritonBench harness (when a copy of
the package is importable) and the standalone operator that mirrors its interface."""
import io
import os
import sys

import numpy as np
import pytest
import torch

from oracle import c_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHAPE = ["--m", "128", "--n", "256", "--k", "512"]


def _c_oracle_backend(self, xq, wq, x_scale, w_scale, bias):
    """Test-only CPU stand-in for a kernel backend: the plain-C oracle."""

    def fn():
        y = c_oracle.gemm_rowwise(
            xq.view(torch.uint8).numpy(), wq.view(torch.uint8).numpy(), x_scale.numpy(), w_scale.numpy(),
            None if bias is None else bias.view(torch.int16).numpy().view(np.uint16),
        )
        return torch.from_numpy(y.view(np.int16)).view(torch.bfloat16)

    return fn


@pytest.fixture(scope="module")
def harness():
    """Put a copy of the reference package on sys.path: the offline install under baseline/_ref, else the
    checkout named by TRITONBENCH_ROOT.  No copy -> these tests are skipped (the standalone-operator tests still run)."""
    for cand in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("TRITONBENCH_ROOT", "")):
        if cand and os.path.isdir(os.path.join(cand, "tritonbench")):
            sys.path.insert(0, cand)
            sys.dont_write_bytecode = True
            return cand
    pytest.skip("no tritonbench package available")


def test_plugin_registers_on_the_stock_operator(harness):
    from tritonbench_b200 import tritonbench_plugin as plug

    cls = plug.register()
    from tritonbench.utils import triton_op

    reg = triton_op.REGISTERED_BENCHMARKS[plug.OP_NAME]
    assert plug.BACKEND in reg and reg[plug.BACKEND].label == "b200"
    assert reg[plug.BACKEND].enabled == torch.cuda.is_available()
    assert triton_op.BASELINE_BENCHMARKS[plug.OP_NAME] == "torch_dequant_ref"
    assert callable(getattr(cls, plug.BACKEND)) and cls.__name__ == "Operator"
    assert plug.register() is cls  # idempotent


def test_plugin_runs_through_the_reference_harness_on_cpu(harness, capsys):
    from tritonbench_b200 import tritonbench_plugin as plug

    cls = plug.register()
    from tritonbench.utils.triton_op import register_benchmark

    register_benchmark(operator_name=plug.OP_NAME, func_name="cpu_standin", enabled=True)(_c_oracle_backend)
    setattr(cls, "cpu_standin", _c_oracle_backend)
    out = plug.run(
        ["--op", plug.OP_NAME, "--device", "cpu", "--metrics", "latency,tflops,gbps,speedup,accuracy",
         "--only", "torch_dequant_ref,cpu_standin"] + SHAPE
    )
    text = str(out)
    for col in ("(M, N, K)", "torch_dequant_ref-latency", "cpu_standin-tflops", "cpu_standin-speedup", "cpu_standin-accuracy"):
        assert col in text, text
    assert "torch_dequant_ref-accuracy" not in text  # the baseline column gets no accuracy cell
    x_val, cells = out.result[0][0], out.result[0][1]
    assert tuple(x_val) == (128, 256, 512)
    acc = [m.accuracy for name, m in cells.items() if name == "cpu_standin"]
    assert acc == [True]


def test_shape_flags_survive_the_b200_override(harness, monkeypatch):
    """On a B200 the stock __init__ throws the --m/--n/--k shape away; the plugin puts it back."""
    from tritonbench_b200 import tritonbench_plugin as plug

    cls = plug.register()
    module = sys.modules[cls.__module__]
    monkeypatch.setattr(module, "is_cuda", lambda: True)
    monkeypatch.setattr(module, "get_nvidia_gpu_model", lambda: "NVIDIA B200")
    from tritonbench.utils.parser import get_parser

    args, extra = get_parser().parse_known_args(["--op", plug.OP_NAME, "--device", "cpu"] + SHAPE)
    op = cls(tb_args=args, extra_args=extra)
    assert op.shapes == [(128, 256, 512)]
    assert args.atol == 1e-3 and args.rtol == 1.6e-2


def test_b200_backend_refuses_cpu_tensors():
    from tritonbench_b200 import tritonbench_plugin as plug

    t = torch.zeros((2, 16), dtype=torch.uint8)
    with pytest.raises(NotImplementedError):
        plug.b200_native(None, t, t, torch.ones(2), torch.ones(2), None)


# ------------------------------------------------------------------ standalone operator
def test_standalone_operator_table_and_metrics():
    from tritonbench_b200 import operator as standalone

    standalone._attach_default_backends()
    standalone.register_benchmark(func_name="cpu_standin")(_c_oracle_backend)
    setattr(standalone.Operator, "cpu_standin", _c_oracle_backend)
    args, extra = standalone.get_parser().parse_known_args(
        ["--device", "cpu", "--metrics", "latency,tflops,gbps,speedup,accuracy", "--only", "torch_dequant_ref,cpu_standin,b200_native",
         "--warmup", "5", "--iter", "20"] + SHAPE
    )
    op = standalone.Operator(args, extra)
    res = op.run(args.warmup, args.iter)
    assert res.headers()[0] == "(M, N, K)"
    assert "cpu_standin-accuracy" in res.headers() and "torch_dequant_ref-accuracy" not in res.headers()
    x, cells = res.rows[0]
    assert x == (128, 256, 512)
    assert cells["cpu_standin"]["accuracy"] is True and cells["cpu_standin"]["speedup"] > 0
    assert cells["b200_native"]["latency"] == "not supported"  # CPU tensors: the library has no CPU path
    flops = 2 * 128 * 256 * 512
    assert abs(cells["torch_dequant_ref"]["tflops"] - flops / cells["torch_dequant_ref"]["latency"] / 1e12 * 1e3) < 1e-9
    buf = io.StringIO()
    res.write_csv_to_file(buf)
    assert buf.getvalue().splitlines()[0].startswith("(M, N, K);")


def test_standalone_operator_shapes_inputs_and_strict_flags():
    from tritonbench_b200 import operator as standalone

    args, extra = standalone.get_parser().parse_known_args(["--device", "cpu"])
    op = standalone.Operator(args, extra)
    assert len(op.shapes) == 20 and op.shapes[7] == (16, 13312, 13312)
    args, extra = standalone.get_parser().parse_known_args(["--device", "cpu", "--bias"] + SHAPE)
    op = standalone.Operator(args, extra)
    xq, wq, xs, ws, bias = next(op.get_input_iter())
    assert xq.dtype == torch.float8_e4m3fn and tuple(wq.shape) == (256, 512) and xs.dtype == torch.float32
    assert bias is not None and bias.dtype == torch.bfloat16 and op.flops((xq, wq, xs, ws, bias)) == 2 * 128 * 256 * 512 + 2 * 128 * 256
    again = next(standalone.Operator(args, extra).get_input_iter())
    assert torch.equal(again[0].view(torch.uint8), xq.view(torch.uint8))  # seeded
    with pytest.raises(SystemExit):
        standalone.Operator(*standalone.get_parser().parse_known_args(["--device", "cpu", "--not_a_flag"]))


def test_builtin_shapes_equal_the_reference_list(golden_dir):
    from tritonbench_b200 import operator as standalone

    shapes = np.load(os.path.join(golden_dir, "ref_builtin_shapes.npz"))["shapes"]
    assert [tuple(int(v) for v in s) for s in shapes] == standalone.BUILDIN_SHAPES

"""Registers the B200 library as a backend of TritonBench's `fp8_gemm_rowwise` operator.

    python -m tritonbench_b200.tritonbench_plugin --op fp8_gemm_rowwise --m 8192 --n 8192 --k 8192 \
        --metrics latency,tflops,gbps,speedup,accuracy

is `python run.py --op fp8_gemm_rowwise ...` with three more columns in the result table:

    b200               this library (b200fp8_gemm_rowwise through ctypes), CUDA devices only
    torch_dequant_ref  (xq.float() @ wq.float().T) * x_scale[:, None] * w_scale[None, :] in fp32 -> bf16 (the
                       products of e4m3 values are exact in fp32, so only the order of the fp32 additions
                       differs from a tensor-core kernel's; scaling the operands first instead rounds every
                       product and fails the harness's tolerance on one element in 10^8 at K = 13312),
                       registered as the BASELINE so that `speedup` and `accuracy` have a reference column
                       on machines where every stock backend is disabled (all of them are on a B200:
                       tritonbench/operators/fp8_gemm_rowwise/operator.py:88-91,101-102)
    scaled_mm          torch._scaled_mm with rowwise scales (cuBLASLt), CUDA only, the library comparator

Registration follows the precedent of the ATen operator loader, which registers backends from
outside the operator's module: `register_benchmark(operator_name=..., func_name=...)` stores the
metadata and the function itself is attached to the class
(tritonbench/operator_loader/aten/loader.py:66-71; tritonbench/utils/triton_op.py:583-616,765-785).

Two adjustments are applied to the stock operator class, both needed on a B200:
  * the stock `__init__` discards `--m/--n/--k` when `nvidia-smi` reports an "NVIDIA B200"
    (operator.py:174-185); the wrapper re-applies them after construction;
  * the harness compares backends with `torch.testing.assert_close` at bf16 default tolerances
    (triton_op.py:1143-1179), whose atol of 1e-5 rejects results that differ by one bf16 ulp near zero;
    when the user passes no `--atol/--rtol` the wrapper sets atol = 1e-3 and rtol = 1.6e-2.
The stock module imports `get_fp8_constants` from FBGEMM at load; where FBGEMM is not installed a
one-function stand-in is provided so that the module loads (with its FBGEMM backends disabled).
"""
import importlib
import os
import sys
import types
from typing import Callable, List, Optional

import torch

OP_NAME = "fp8_gemm_rowwise"
BACKEND = "b200_native"
_registered = False


def _install_fbgemm_standin() -> bool:
    """Make `from fbgemm_gpu.experimental.gemm.triton_gemm.fp8_gemm import get_fp8_constants` work
    when FBGEMM is absent.  Only that one function exists in the stand-in, so the stock backends'
    own imports still fail and stay disabled.  Returns True if a stand-in was installed."""
    try:
        importlib.import_module("fbgemm_gpu.experimental.gemm.triton_gemm.fp8_gemm")
        return False
    except Exception:
        pass
    names = [
        "fbgemm_gpu",
        "fbgemm_gpu.experimental",
        "fbgemm_gpu.experimental.gemm",
        "fbgemm_gpu.experimental.gemm.triton_gemm",
        "fbgemm_gpu.experimental.gemm.triton_gemm.fp8_gemm",
    ]
    for n in names:
        mod = types.ModuleType(n)
        mod.__path__ = []
        mod.__b200_standin__ = True
        sys.modules[n] = mod
    sys.modules[names[-1]].get_fp8_constants = lambda: (torch.float8_e4m3fn, None, 448.0, 1e-12)
    return True


# ------------------------------------------------------------------ backends
def b200_native(self, xq, wq, x_scale, w_scale, bias) -> Callable:
    """The library call.  Set-up (workspace) happens here, untimed; the closure only enqueues."""
    if not xq.is_cuda:
        raise NotImplementedError("b200 backend runs on CUDA devices only; there is no CPU path")
    from . import ops

    # The harness replays this closure back to back on fixed inputs (operator.py:156): nothing writes wq
    # while it runs, so decode-shaped calls may overlap their predecessor's tail (B200FP8_OVERLAP=0 turns it off).
    overlap = xq.shape[0] <= 128 and os.environ.get("B200FP8_OVERLAP", "1") != "0"
    return ops.make_gemm_fn(xq, wq, x_scale, w_scale, bias, overlap=overlap)


def torch_dequant_ref(self, xq, wq, x_scale, w_scale, bias) -> Callable:
    def fn():
        y = (xq.to(torch.float32) @ wq.to(torch.float32).T) * (x_scale[:, None] * w_scale[None, :])
        if bias is not None:
            y = y + bias.to(torch.float32)
        return y.to(torch.bfloat16)

    return fn


def scaled_mm(self, xq, wq, x_scale, w_scale, bias) -> Callable:
    if not xq.is_cuda:
        raise NotImplementedError("torch._scaled_mm takes rowwise scales on CUDA only")

    def fn():
        return torch._scaled_mm(
            xq, wq.t(), scale_a=x_scale[:, None], scale_b=w_scale[None, :], bias=bias, out_dtype=torch.bfloat16
        )

    return fn


# ------------------------------------------------------------------ roofline metrics
# The reference's own roofline table has no correct B200 entry (tritonbench/utils/gpu_utils.py:37-46 copies the H100
# row), so `--metrics ...,pct_fp8_peak,pct_hbm` adds two columns computed against the B200's figures: measured ones
# from MEASURED_PEAKS.json at the repository root when that file exists (fp8 peak = 2 x the cuBLAS bf16 rate, HBM =
# the copy bandwidth), else the datasheet's dense FP8 4500 TFLOP/s and 8000 GB/s.
def _b200_peaks():
    import json

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return 2.0 * float(p["bf16_tflops"]), float(p["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 4500.0, 8000.0


def _latency_ms(metrics) -> float:
    """The harness's latency object divides like a number (its p50, components/do_bench/run.py:12-100)."""
    lat = metrics.latency
    return float(getattr(lat, "p50", lat))


def pct_fp8_peak(self, fn, example_inputs, metrics) -> float:
    """Per cent of the dense FP8 tensor peak: the operator's own flops (operator.py:248-259) over its latency."""
    flops = self.flops(fn, example_inputs, metrics)
    return 100.0 * (flops / _latency_ms(metrics) / 1e12 * 1e3) / _b200_peaks()[0]


def pct_hbm(self, fn, example_inputs, metrics) -> float:
    """Per cent of the HBM bandwidth: the operator's own byte count |a| + |b| + |c| (operator.py:261-271) over its latency."""
    xq, wq = example_inputs[0], example_inputs[1]
    nbytes = xq.numel() * xq.element_size() + wq.numel() * wq.element_size() + xq.shape[0] * wq.shape[0] * 2
    return 100.0 * (nbytes / 1e9 / _latency_ms(metrics) * 1e3) / _b200_peaks()[1]


def _register_roofline_metrics(cls) -> None:
    """register_metric() derives the operator from the function's module (triton_op.py:619-644), so functions
    defined here are entered into the registry directly and attached to the class."""
    from tritonbench.utils.triton_op import REGISTERED_METRICS

    for fn in (pct_fp8_peak, pct_hbm):
        if fn.__name__ not in REGISTERED_METRICS[OP_NAME]:
            REGISTERED_METRICS[OP_NAME].append(fn.__name__)
        setattr(cls, fn.__name__, fn)


def b200_fp8_gemm(self, a, b) -> Callable:
    """Backend for the sibling operator `fp8_gemm` (tritonbench/operators/fp8_gemm/fp8_gemm.py:47-101): the same
    kernels with unit scales; bf16 output with `--scaling_rowwise`, fp16 output with per-tensor scales, exactly
    as the operator's own `torch_fp8_gemm` baseline chooses."""
    if not a.is_cuda:
        raise NotImplementedError("b200 backend runs on CUDA devices only; there is no CPU path")
    from . import ops

    rowwise = bool(getattr(self.extra_args, "scaling_rowwise", False))
    out_dtype = torch.bfloat16 if rowwise else torch.float16
    m, n = a.shape[0], b.shape[1]
    ones_m = torch.ones(m, dtype=torch.float32, device=a.device)
    ones_n = torch.ones(n, dtype=torch.float32, device=a.device)
    overlap = m <= 128 and os.environ.get("B200FP8_OVERLAP", "1") != "0"
    return ops.make_gemm_fn(a, b.t(), ones_m, ones_n, None, overlap=overlap, out_dtype=out_dtype)


def register_fp8_gemm():
    """Add the backend to the `fp8_gemm` operator.  Returns the operator class."""
    from tritonbench.utils.triton_op import REGISTERED_BENCHMARKS, register_benchmark

    module = importlib.import_module("tritonbench.operators.fp8_gemm.fp8_gemm")
    cls = module.Operator
    if BACKEND not in REGISTERED_BENCHMARKS.get("fp8_gemm", {}):
        register_benchmark(operator_name="fp8_gemm", func_name=BACKEND, label="b200", enabled=torch.cuda.is_available())(
            b200_fp8_gemm
        )
        setattr(cls, BACKEND, b200_fp8_gemm)
    return cls


def b200_grouped(self, group_A, group_B, m_sizes, a_scale, b_scale) -> Callable:
    """Backend for `fp8_gemm_rowwise_grouped` (tritonbench/operators/fp8_gemm_rowwise_grouped/operator.py:412-470)."""
    if not group_A.is_cuda:
        raise NotImplementedError("b200 backend runs on CUDA devices only; there is no CPU path")
    from . import ops

    groups = m_sizes.numel()
    out = torch.empty((group_A.shape[0], group_B.shape[0] // groups), dtype=torch.bfloat16, device=group_A.device)
    sizes = m_sizes.to(torch.int32).contiguous()
    ws = ops.get_workspace(group_A.device, 256)  # allocated here, outside the timed / captured region
    return lambda: ops.fp8_gemm_rowwise_grouped(group_A, group_B, sizes, a_scale, b_scale, out=out, workspace=ws)


def torch_dequant_grouped_ref(self, group_A, group_B, m_sizes, a_scale, b_scale) -> Callable:
    """fp32 dequantise-then-matmul per group: the baseline column where FBGEMM's grouped kernels are absent."""
    sizes = [int(v) for v in m_sizes.cpu().tolist()]
    n = group_B.shape[0] // len(sizes)

    def fn():
        outs, r0 = [], 0
        for g, rows in enumerate(sizes):
            x = group_A[r0 : r0 + rows].to(torch.float32) * a_scale[r0 : r0 + rows, None]
            w = group_B[g * n : (g + 1) * n].to(torch.float32) * b_scale[g * n : (g + 1) * n, None]
            outs.append((x @ w.T).to(torch.bfloat16))
            r0 += rows
        return torch.cat(outs)

    return fn


def register_grouped():
    """Add the backends to the `fp8_gemm_rowwise_grouped` operator.  Returns the operator class."""
    _install_fbgemm_standin()
    from tritonbench.utils.triton_op import REGISTERED_BENCHMARKS, register_benchmark

    op = "fp8_gemm_rowwise_grouped"
    module = importlib.import_module(f"tritonbench.operators.{op}.operator")
    cls = module.Operator
    if BACKEND not in REGISTERED_BENCHMARKS.get(op, {}):
        register_benchmark(operator_name=op, func_name=BACKEND, label="b200", enabled=torch.cuda.is_available())(b200_grouped)
        setattr(cls, BACKEND, b200_grouped)
        register_benchmark(operator_name=op, func_name="torch_dequant_ref", baseline=True)(torch_dequant_grouped_ref)
        setattr(cls, "torch_dequant_ref", torch_dequant_grouped_ref)
    return cls


def b200_blockwise(self, xq, wq, x_scale, w_scale) -> Callable:
    """Backend for `fp8_gemm_blockwise` (tritonbench/operators/fp8_gemm_blockwise/operator.py:139-149)."""
    if not xq.is_cuda:
        raise NotImplementedError("b200 backend runs on CUDA devices only; there is no CPU path")
    from . import ops

    x_scale = x_scale.to(xq.device).contiguous()  # the stock quantiser leaves the scales where it computed them
    w_scale = w_scale.to(xq.device).contiguous()
    out = torch.empty((xq.shape[0], wq.shape[0]), dtype=torch.bfloat16, device=xq.device)
    ws = ops.get_workspace(xq.device, 256)
    return lambda: ops.fp8_gemm_blockwise(xq, wq, x_scale, w_scale, out=out, workspace=ws)


def torch_dequant_blockwise_ref(self, xq, wq, x_scale, w_scale) -> Callable:
    """fp32 dequantise-then-matmul with the block scales expanded: the baseline column where FBGEMM is absent."""
    m, k = xq.shape
    n = wq.shape[0]
    xs = x_scale.to(xq.device).repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)[:m, :k]
    ws = w_scale.to(xq.device).repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)[:n, :k]
    return lambda: ((xq.to(torch.float32) * xs) @ (wq.to(torch.float32) * ws).T).to(torch.bfloat16)


def register_blockwise():
    """Add the backends to the `fp8_gemm_blockwise` operator.  Its module imports fbgemm_gpu.experimental.gen_ai
    for side effects only; where FBGEMM is absent an empty stand-in module lets it load (its own backends stay off)."""
    if _install_fbgemm_standin() or getattr(sys.modules.get("fbgemm_gpu"), "__b200_standin__", False):
        name = "fbgemm_gpu.experimental.gen_ai"
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__b200_standin__ = True
            sys.modules[name] = mod
            sys.modules["fbgemm_gpu.experimental"].gen_ai = mod
    from tritonbench.utils.triton_op import REGISTERED_BENCHMARKS, register_benchmark

    op = "fp8_gemm_blockwise"
    module = importlib.import_module(f"tritonbench.operators.{op}.operator")
    cls = module.Operator
    if BACKEND not in REGISTERED_BENCHMARKS.get(op, {}):
        register_benchmark(operator_name=op, func_name=BACKEND, label="b200", enabled=torch.cuda.is_available())(b200_blockwise)
        setattr(cls, BACKEND, b200_blockwise)
        register_benchmark(operator_name=op, func_name="torch_dequant_ref", baseline=True)(torch_dequant_blockwise_ref)
        setattr(cls, "torch_dequant_ref", torch_dequant_blockwise_ref)
    return cls


def _fused_backend(producer: str, round_bf16: bool) -> Callable:
    """Backend factory for `fp8_fused_quant_gemm_rowwise`: producer + quantiser in one kernel, then the GEMM.  The
    closure runs both kernels, as the stock backends do (operator.py:86-131 time the quantiser with the GEMM)."""

    def backend(self, x1, x2, wq, w_scale, wd) -> Callable:
        if not x1.is_cuda:
            raise NotImplementedError("b200 backend runs on CUDA devices only; there is no CPU path")
        from . import ops

        m, k = x1.shape
        n = wq.shape[0]
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x1.device)
        workspace = ops.get_workspace(x1.device, ops.workspace_bytes(m, n, k))
        w_scale = w_scale.contiguous()

        # decode-sized calls: the GEMM starts while the quantiser runs (it reads W - which nothing writes - early, and
        # xq / xs only after the quantiser has completed); B200FP8_OVERLAP=0 turns it off
        overlap = m <= 128 and os.environ.get("B200FP8_OVERLAP", "1") != "0"

        def fn():
            if producer == "rms_norm":
                xq, xs = ops.rms_norm_fp8_rowwise_quant(x1, wd, round_bf16=round_bf16)
            else:
                xq, xs = ops.silu_mul_fp8_rowwise_quant(x1, x2, round_bf16=round_bf16)
            return ops.fp8_gemm_rowwise(xq, wq, xs, w_scale, out=out, workspace=workspace, overlap=overlap)

        return fn

    return backend


def _torch_fused_ref(producer: str, round_bf16: bool = False) -> Callable:
    """fp32 torch pipeline of the same definition as the backend it checks: producer (with the activation rounded
    to bf16 first when `round_bf16`, i.e. a producer kernel followed by a quantiser), rowwise quantiser,
    dequantised fp32 GEMM."""

    def backend(self, x1, x2, wq, w_scale, wd) -> Callable:
        def fn():
            a = x1.to(torch.float32)
            if producer == "rms_norm":
                y = (a * torch.rsqrt(a.pow(2).mean(dim=1, keepdim=True) + 1e-5)) * wd.to(torch.float32)[None, :]
            else:
                y = a * torch.sigmoid(a) * x2.to(torch.float32)
            if round_bf16:
                y = y.to(torch.bfloat16).to(torch.float32)
            scale = y.abs().amax(dim=1).clamp(min=1e-12) / 448.0
            yq = (y / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
            out = (yq.to(torch.float32) @ wq.to(torch.float32).T) * (scale[:, None] * w_scale[None, :])
            return out.to(torch.bfloat16)

        return fn

    return backend


# baseline of the matching definition for each of the four backends (`--baseline NAME --only NAME,<backend>`)
FUSED_BASELINES = {
    "b200_rms_norm_fused": "torch_rms_norm_ref",
    "b200_rms_norm_quant": "torch_rms_norm_bf16_ref",
    "b200_silu_mul_fused": "torch_silu_mul_ref",
    "b200_silu_mul_quant": "torch_silu_mul_bf16_ref",
}


def fused_quant_tolerance(k: int):
    """(atol, rtol) for comparing a fused-quantiser backend with the torch pipeline of the same definition.
    The two compute the activation y with different fp32 operation orders (and exponentials), so a fraction of the
    activations (0.2 % measured; more when y is rounded to bf16 first, where a last-bit difference can move y by a
    whole bf16 step) lands on the other side of an e4m3 rounding boundary: one step, up to 1/8 of that element.
    With unit-variance inputs (the operator draws x, w and the norm weight from N(0,1)) an output has
    sigma ~ sqrt(K); a flipped large activation moves every output of its row by up to |y| |w| / 8.  Measured on a
    B200 over four shapes (K = 2048 ... 8192), the largest deviation beyond rtol was 0.030 sqrt(K) for the backends
    that keep y in fp32 and 0.072 sqrt(K) for those that round it to bf16.  atol = 0.1 sqrt(K) (a tenth of an
    output's sigma); rtol is two bf16 steps, as for the plain GEMM."""
    return 0.1 * float(k) ** 0.5, 1.6e-2


def _standin_quantize_fp8_row(a, scale_ub=None, zero_start_index_M=None, use_triton=True, output_device=None):
    """Stand-in for FBGEMM's `quantize_fp8_row` used by input generators when FBGEMM is absent:
    fp32 arithmetic, scale = max(rowabsmax, 1e-12) / 448, returns (a_fp8, scale)."""
    from . import quantize

    return quantize.fp8_row_quantize_fp32(a.reshape(-1, a.shape[-1]))


def register_fused_quant():
    """Add backends to `fp8_fused_quant_gemm_rowwise` (RMS norm or SiLU-mul producer, rowwise quantiser, GEMM).
    Its module needs `fbgemm_gpu.experimental.gen_ai`, `quantize_fp8_row` and `matmul_fp8_row` to import and its own
    producers come from a Meta-internal package, so every stock backend is disabled here; the stand-ins only let the
    module load and its input generator run.  The operator compares every backend with ONE baseline although it holds
    four functions; the default baseline is the fp32 rms_norm pipeline, and `--baseline NAME` (FUSED_BASELINES) selects
    the torch pipeline that matches another backend's definition."""
    standin = _install_fbgemm_standin() or getattr(sys.modules.get("fbgemm_gpu"), "__b200_standin__", False)
    if standin:
        name = "fbgemm_gpu.experimental.gen_ai"
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__b200_standin__ = True
            sys.modules[name] = mod
            sys.modules["fbgemm_gpu.experimental"].gen_ai = mod
        fp8_gemm_mod = sys.modules["fbgemm_gpu.experimental.gemm.triton_gemm.fp8_gemm"]
        fp8_gemm_mod.quantize_fp8_row = _standin_quantize_fp8_row

        def _absent(*args, **kwargs):
            raise NotImplementedError("FBGEMM is not installed")

        fp8_gemm_mod.matmul_fp8_row = _absent
    from tritonbench.utils.triton_op import REGISTERED_BENCHMARKS, register_benchmark

    op = "fp8_fused_quant_gemm_rowwise"
    module = importlib.import_module(f"tritonbench.operators.{op}.operator")
    cls = module.Operator
    if "b200_rms_norm_fused" not in REGISTERED_BENCHMARKS.get(op, {}):
        cuda = torch.cuda.is_available()
        for name, producer, rounded in (
            ("b200_rms_norm_fused", "rms_norm", False),
            ("b200_rms_norm_quant", "rms_norm", True),
            ("b200_silu_mul_fused", "silu_mul", False),
            ("b200_silu_mul_quant", "silu_mul", True),
        ):
            fn = _fused_backend(producer, rounded)
            fn.__name__ = name
            register_benchmark(operator_name=op, func_name=name, enabled=cuda)(fn)
            setattr(cls, name, fn)
        for name, producer, rounded, baseline in (
            ("torch_silu_mul_ref", "silu_mul", False, False),
            ("torch_silu_mul_bf16_ref", "silu_mul", True, False),
            ("torch_rms_norm_bf16_ref", "rms_norm", True, False),
            ("torch_rms_norm_ref", "rms_norm", False, True),  # last: the default baseline
        ):
            ref = _torch_fused_ref(producer, rounded)
            ref.__name__ = name
            register_benchmark(operator_name=op, func_name=name, baseline=baseline)(ref)
            setattr(cls, name, ref)
    return cls


def _wrap_init(cls) -> None:
    stock_init = cls.__init__
    if getattr(stock_init, "__b200_wrapped__", False):
        return
    op_module = sys.modules[cls.__module__]

    def __init__(self, tb_args, extra_args: Optional[List[str]] = None):
        stock_init(self, tb_args, extra_args)
        parsed = op_module.parse_args(self.extra_args or [])
        if parsed.m and parsed.n and parsed.k:
            self.shapes = [(parsed.m, parsed.n, parsed.k)]
        if getattr(tb_args, "atol", None) is None and getattr(tb_args, "rtol", None) is None:
            tb_args.atol, tb_args.rtol = 1e-3, 1.6e-2

    __init__.__b200_wrapped__ = True
    cls.__init__ = __init__


def register(with_comparators: bool = True):
    """Import the stock operator and add our backends to it.  Idempotent.  Returns the class."""
    global _registered
    _install_fbgemm_standin()
    from tritonbench.utils.triton_op import register_benchmark

    module = importlib.import_module(f"tritonbench.operators.{OP_NAME}.operator")
    cls = module.Operator
    if _registered:
        return cls
    cuda = torch.cuda.is_available()
    register_benchmark(operator_name=OP_NAME, func_name=BACKEND, label="b200", enabled=cuda)(b200_native)
    setattr(cls, BACKEND, b200_native)
    if with_comparators:
        # registered last with baseline=True: the harness takes the last baseline registered
        # (triton_op.py:608-609), overriding the stock (disabled) CUTLASS baseline
        register_benchmark(operator_name=OP_NAME, func_name="scaled_mm", enabled=cuda)(scaled_mm)
        setattr(cls, "scaled_mm", scaled_mm)
        register_benchmark(operator_name=OP_NAME, func_name="torch_dequant_ref", baseline=True)(torch_dequant_ref)
        setattr(cls, "torch_dequant_ref", torch_dequant_ref)
    _wrap_init(cls)
    _register_roofline_metrics(cls)
    _registered = True
    return cls


def run(argv: List[str]):
    """Equivalent of the reference's run.py `_run` (run.py:39-100) for this one operator.  Without an
    importable `tritonbench` package the same command line is served by the standalone operator in
    tritonbench_b200/operator.py, which mirrors the interface."""
    try:
        importlib.import_module("tritonbench.utils.triton_op")
    except ImportError:
        from . import operator as standalone

        return standalone.run(argv)
    register()
    from tritonbench.operators import load_opbench_by_name
    from tritonbench.utils.parser import get_parser

    args, extra = get_parser().parse_known_args(argv)
    if args.op == "fp8_gemm":
        register_fp8_gemm()
    elif args.op == "fp8_gemm_rowwise_grouped":
        register_grouped()
        if args.atol is None and args.rtol is None:
            args.atol, args.rtol = 1e-3, 1.6e-2
    elif args.op == "fp8_gemm_blockwise":
        register_blockwise()
        if args.atol is None and args.rtol is None:
            args.atol, args.rtol = 1e-3, 1.6e-2
    elif args.op == "fp8_fused_quant_gemm_rowwise":
        register_fused_quant()
        if args.atol is None and args.rtol is None:
            from tritonbench.operators.fp8_fused_quant_gemm_rowwise import operator as fused_op

            shape_args = fused_op.parse_args(list(extra))
            k_max = shape_args.k if (shape_args.m and shape_args.n and shape_args.k) else max(s[2] for s in fused_op.BUILDIN_SHAPES)
            args.atol, args.rtol = fused_quant_tolerance(k_max)
    elif args.op != OP_NAME:
        raise SystemExit(
            f"this plugin serves --op {OP_NAME}, fp8_gemm, fp8_gemm_rowwise_grouped, fp8_gemm_blockwise and "
            "fp8_fused_quant_gemm_rowwise only"
        )
    opbench = load_opbench_by_name(args.op)(tb_args=args, extra_args=extra)
    try:
        opbench.run(args.warmup, args.iter)
    finally:
        metrics = opbench.output
        if not args.skip_print:
            if args.csv:
                metrics.write_csv_to_file(sys.stdout)
            else:
                print(metrics)
    return metrics


if __name__ == "__main__":
    run(sys.argv[1:])

"""Standalone `fp8_gemm_rowwise` operator with the interface of the TritonBench one, for machines
where the `tritonbench` package is not installed.  Same names, argument meaning and error behaviour
as the reference for this one operator:

  * operator flags `--m --n --k --bias` and the 20 built-in shapes
    (tritonbench/operators/fp8_gemm_rowwise/operator.py:21-63,107-128)
  * input generator: bf16 randn under seed 1337, rowwise e4m3 quantisation, optional bf16 bias
    (operator.py:280-297; tritonbench/utils/env_utils.py:20)
  * backends are methods `name(self, xq, wq, x_scale, w_scale, bias) -> zero-argument callable`,
    registered with `register_benchmark(...)` (tritonbench/utils/triton_op.py:583-616,765-785)
  * metrics `latency, tflops, gbps, speedup, accuracy` with the reference's definitions
    (operator.py:248-271; triton_op.py:1143-1179,1264-1284); CUDA latency is measured by CUDA-graph
    replay, the reference's default for this operator (operator.py:156; components/do_bench/run.py:190-199)
  * a failing backend becomes an error cell with `--keep-going`; NotImplementedError reads
    "not supported" (triton_op.py:1500-1507)
  * result table headed "(M, N, K)" with one `<label>-<metric>` column per backend and metric.

When the real package is importable, tritonbench_plugin.register() is the drop-in and this file is unused.
"""
import argparse
import statistics
import sys
import time
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Callable, Dict, Generator, List, Optional, Tuple

import torch

from . import quantize

BUILDIN_SHAPES = [
    (1, 2304, 2048), (1, 8192, 16384), (4, 4096, 2304), (4, 13312, 2048), (8, 2304, 2304), (8, 8192, 6656),
    (16, 4096, 6656), (16, 13312, 13312), (32, 2304, 16384), (32, 8192, 13312), (64, 4096, 2048),
    (64, 13312, 2048), (128, 2304, 6656), (128, 8192, 2304), (2048, 8192, 2048), (2048, 13312, 6656),
    (4096, 2304, 13312), (4096, 13312, 2304), (16384, 4096, 16384), (16384, 8192, 13312),
]
SEED = 1337
DEFAULT_METRICS = ["tflops", "speedup", "accuracy"]


@dataclass
class Backend:
    name: str
    label: str
    baseline: bool
    enabled: bool


REGISTERED_BENCHMARKS: "OrderedDict[str, Backend]" = OrderedDict()
BASELINE_BENCHMARK: Dict[str, str] = {}


def register_benchmark(operator_name=None, func_name=None, baseline=False, enabled=True, fwd_only=False, label=None):
    def decorator(function):
        name = func_name or function.__name__
        REGISTERED_BENCHMARKS[name] = Backend(name, label or name, baseline, enabled)
        if baseline:
            BASELINE_BENCHMARK["name"] = name
        return function

    return decorator


def get_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(allow_abbrev=False)
    p.add_argument("--op", default="fp8_gemm_rowwise")
    p.add_argument("--device", default="cuda")
    p.add_argument("--metrics", default=None)
    p.add_argument("--only", default=None)
    p.add_argument("--skip", default=None)
    p.add_argument("--baseline", default=None)
    p.add_argument("--atol", type=float, default=None)
    p.add_argument("--rtol", type=float, default=None)
    p.add_argument("--num-inputs", type=int, default=None)
    p.add_argument("--input-id", type=int, default=0)
    p.add_argument("--warmup", type=int, default=25)
    p.add_argument("--iter", type=int, default=100)
    p.add_argument("--csv", action="store_true")
    p.add_argument("--keep-going", action="store_true")
    p.add_argument("--skip-print", action="store_true")
    p.add_argument("--cudagraph", action="store_true")
    return p


def parse_args(args: List[str]) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="fp8 gemm rowwise operator")
    p.add_argument("--m", type=int)
    p.add_argument("--n", type=int)
    p.add_argument("--k", type=int)
    p.add_argument("--bias", action="store_true", default=False)
    p.add_argument("--llama", action="store_true")
    p.add_argument("--prefill", default=False, action="store_true")
    p.add_argument("--no_fp8_fast_accum", dest="fp8_fast_accum", action="store_false")
    p.add_argument("--no_use_tma", dest="use_tma", default=None, action="store_false")
    p.add_argument("--use_tma", dest="use_tma", action="store_true")
    p.add_argument("--use_persistent", dest="no_use_persistent", default=None, action="store_false")
    p.add_argument("--no_use_persistent", dest="no_use_persistent", action="store_true")
    p.add_argument("--warp_specialization", action="store_true")
    return p.parse_args(args)  # strict, like the reference: unknown flags are an error


class Result:
    """Rows of (x_val, {backend: {metric: value}}) printed in the reference's table layout."""

    def __init__(self, metrics: List[str], backends: List[Backend], baseline: Optional[str]):
        self.metrics, self.backends, self.baseline = metrics, backends, baseline
        self.rows: List[Tuple[Any, Dict[str, Dict[str, Any]]]] = []

    def headers(self) -> List[str]:
        h = ["(M, N, K)"]
        for b in self.backends:
            for m in self.metrics:
                if b.name == self.baseline and m in ("speedup", "accuracy"):
                    continue
                h.append(f"{b.label}-{m}")
        return h

    def table(self) -> List[List[Any]]:
        out = []
        for x, cells in self.rows:
            row = [x]
            for b in self.backends:
                for m in self.metrics:
                    if b.name == self.baseline and m in ("speedup", "accuracy"):
                        continue
                    row.append(cells.get(b.name, {}).get(m))
            out.append(row)
        return out

    def __str__(self) -> str:
        try:
            from tabulate import tabulate

            return tabulate(self.table(), headers=self.headers(), stralign="right")
        except ImportError:
            lines = ["  ".join(self.headers())]
            lines += ["  ".join(str(c) for c in r) for r in self.table()]
            return "\n".join(lines)

    def write_csv_to_file(self, f) -> None:
        f.write(";".join(self.headers()) + "\n")
        for r in self.table():
            f.write(";".join(str(float(c)) if isinstance(c, bool) else str(c) for c in r) + "\n")


def _latency_ms_cuda(fn: Callable, warmup_ms: int, rep_ms: int) -> float:
    """CUDA-graph replay: n back-to-back calls in one graph, replayed 10 times, median per call."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            fn()
        e1.record()
        torch.cuda.synchronize()
        est = max(e0.elapsed_time(e1) / 5, 1e-3)
        n_repeat = max(1, min(1000, int(rep_ms / est)))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(n_repeat):
                fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(10):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            graph.replay()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) / n_repeat)
    torch.cuda.current_stream().wait_stream(side)
    return statistics.median_low(times)


def _latency_ms_cpu(fn: Callable, warmup_ms: int, rep_ms: int) -> float:
    fn()
    t0 = time.perf_counter()
    for _ in range(5):
        fn()
    est = max((time.perf_counter() - t0) / 5 * 1e3, 1e-3)
    for _ in range(max(1, int(warmup_ms / est))):
        fn()
    times = []
    for _ in range(max(1, int(rep_ms / est))):
        t0 = time.perf_counter_ns()
        fn()
        times.append((time.perf_counter_ns() - t0) / 1e6)
    return statistics.median_low(times)


class Operator:
    DEFAULT_METRICS = DEFAULT_METRICS
    DEFAULT_PRECISION = "fp8"
    name = "fp8_gemm_rowwise"

    def __init__(self, tb_args: argparse.Namespace, extra_args: Optional[List[str]] = None):
        self.tb_args = tb_args
        self.extra_args = extra_args or []
        self.device = tb_args.device
        self.use_cuda_graphs = True
        op_args = parse_args(self.extra_args)
        if op_args.m and op_args.n and op_args.k:
            self.shapes = [(op_args.m, op_args.n, op_args.k)]
        elif op_args.llama:
            raise NotImplementedError("--llama shapes are not available outside the reference's internal build")
        else:
            self.shapes = list(BUILDIN_SHAPES)
        self.bias = op_args.bias
        self.required_metrics = tb_args.metrics.split(",") if tb_args.metrics else list(self.DEFAULT_METRICS)
        self._only = tb_args.only.split(",") if tb_args.only else None
        self._skip = tb_args.skip.split(",") if tb_args.skip else []
        self._input_id = tb_args.input_id
        self._num_inputs = tb_args.num_inputs
        self.output: Optional[Result] = None

    # ---- inputs (operator.py:280-297)
    def get_input_iter(self) -> Generator:
        torch.manual_seed(SEED)
        for m, n, k in self.shapes:
            x = torch.randn((m, k), device=self.device, dtype=torch.bfloat16)
            w = torch.randn((n, k), device=self.device, dtype=torch.bfloat16)
            xq, x_scale = quantize.fp8_row_quantize(x)
            wq, w_scale = quantize.fp8_row_quantize(w)
            bias = torch.randn((n,), device=self.device, dtype=torch.bfloat16) if self.bias else None
            yield xq, wq, x_scale, w_scale, bias

    def get_x_val(self, example_inputs) -> Tuple[int, int, int]:
        xq, wq = example_inputs[0], example_inputs[1]
        return (xq.shape[0], wq.shape[0], xq.shape[1])

    def flops(self, example_inputs) -> int:
        xq, wq, _, _, bias = example_inputs
        m, k = xq.shape
        n = wq.shape[0]
        return 2 * m * n * k + (2 * m * n if bias is not None else 0)

    def gbps(self, fn: Callable, example_inputs, latency_ms: float) -> float:
        a, b = example_inputs[0], example_inputs[1]
        c = fn()
        nbytes = lambda t: t.numel() * t.element_size()  # noqa: E731
        return (nbytes(a) + nbytes(b) + nbytes(c)) / 1e9 / latency_ms * 1e3

    def accuracy(self, fn: Callable, baseline_fn: Callable) -> bool:
        try:
            kw = {}
            if self.tb_args.atol is not None or self.tb_args.rtol is not None:
                kw = {"atol": self.tb_args.atol or 0.0, "rtol": self.tb_args.rtol or 0.0}
            else:
                kw = {"atol": 1e-3, "rtol": 1.6e-2}
            torch.testing.assert_close(fn(), baseline_fn(), **kw)
            return True
        except AssertionError:
            return False

    # ---- run loop (triton_op.py:810-942)
    def _selected(self) -> List[Backend]:
        if self._only:
            missing = [n for n in self._only if n not in REGISTERED_BENCHMARKS]
            if missing:
                raise ValueError(f"unknown backend(s) {missing}; registered: {list(REGISTERED_BENCHMARKS)}")
            picked = [REGISTERED_BENCHMARKS[n] for n in self._only]
        else:
            picked = [b for b in REGISTERED_BENCHMARKS.values() if b.enabled and b.name not in self._skip]
        base = self.tb_args.baseline or BASELINE_BENCHMARK.get("name")
        picked.sort(key=lambda b: 0 if b.name == base else 1)  # baseline column first
        return picked

    def run(self, warmup: int = 25, rep: int = 100) -> Result:
        backends = self._selected()
        base_name = self.tb_args.baseline or BASELINE_BENCHMARK.get("name")
        if base_name not in [b.name for b in backends]:
            base_name = None
        result = Result(self.required_metrics, backends, base_name)
        self.output = result
        latency = _latency_ms_cuda if str(self.device).startswith("cuda") else _latency_ms_cpu
        for idx, inputs in enumerate(self.get_input_iter()):
            if idx < self._input_id:
                continue
            if self._num_inputs is not None and idx >= self._input_id + self._num_inputs:
                break
            cells: Dict[str, Dict[str, Any]] = {}
            base_fn, base_lat = None, None
            for b in backends:
                cell: Dict[str, Any] = {}
                try:
                    fn = getattr(self, b.name)(*inputs)
                    lat = latency(fn, warmup, rep)
                    cell["latency"] = lat
                    cell["tflops"] = self.flops(inputs) / lat / 1e12 * 1e3
                    if "gbps" in self.required_metrics:
                        cell["gbps"] = self.gbps(fn, inputs, lat)
                    if b.name == base_name:
                        base_fn, base_lat = fn, lat
                    elif base_fn is not None:
                        cell["speedup"] = base_lat / lat
                        if "accuracy" in self.required_metrics:
                            cell["accuracy"] = self.accuracy(fn, base_fn)
                except NotImplementedError:
                    cell = {m: "not supported" for m in self.required_metrics}
                except torch.cuda.OutOfMemoryError:
                    cell = {m: "CUDA OOM" for m in self.required_metrics}
                except Exception as e:  # noqa: BLE001
                    if not self.tb_args.keep_going:
                        raise
                    cell = {m: f"error: {e}" for m in self.required_metrics}
                cells[b.name] = cell
            result.rows.append((self.get_x_val(inputs), cells))
        return result


def _attach_default_backends() -> None:
    from . import tritonbench_plugin as plug

    cuda = torch.cuda.is_available()
    if "torch_dequant_ref" in REGISTERED_BENCHMARKS:
        return
    register_benchmark(func_name=plug.BACKEND, label="b200", enabled=cuda)(plug.b200_native)
    setattr(Operator, plug.BACKEND, plug.b200_native)
    register_benchmark(func_name="scaled_mm", enabled=cuda)(plug.scaled_mm)
    setattr(Operator, "scaled_mm", plug.scaled_mm)
    register_benchmark(func_name="torch_dequant_ref", baseline=True)(plug.torch_dequant_ref)
    setattr(Operator, "torch_dequant_ref", plug.torch_dequant_ref)


def run(argv: List[str]) -> Result:
    _attach_default_backends()
    args, extra = get_parser().parse_known_args(argv)
    if args.op != Operator.name:
        raise SystemExit(f"this module serves --op {Operator.name} only")
    op = Operator(args, extra)
    try:
        op.run(args.warmup, args.iter)
    finally:
        if op.output is not None and not args.skip_print:
            if args.csv:
                op.output.write_csv_to_file(sys.stdout)
            else:
                print(op.output)
    return op.output


if __name__ == "__main__":
    run(sys.argv[1:])

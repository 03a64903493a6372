#!/usr/bin/env python
"""Benchmark of the FP8 rowwise-scaled GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one pass of the GEMM over one batch of synthetic input.  The default workload is the
square configuration M = N = K = 8192 per GPU (X and Y sharded by rows, W replicated: with N GPUs
the job is the M = N*8192 prefill problem, i.e. M = 65536 at 8 GPUs).  Rank 0 prints ONE JSON line.

  value      whole-job TFLOP/s with inputs resident in HBM, timed with CUDA events on the launching
             stream over exactly K back-to-back steps, max over ranks
  e2e        the same metric through the host-buffer C-ABI call (b200fp8_gemm_rowwise_host): every
             step copies X, W and the scales from pinned host memory, runs the kernel and copies Y back;
             with the PCIe rates measured in the same process and the fraction of that bound it reaches
  roofline   achieved vs the measured tensor peak (large M) or HBM peak (decode workload)
  cpu_baseline  the CPU oracle (torch fp32 dequantise-then-matmul) timed on a bounded row sample
  parity     rows of the Y each timed loop produced last, sampled and compared with the CPU oracle inside
             this run; a failure makes the process exit non-zero
  also       (default workload only) the other benchmark configurations, each timed and checked the same
             way: the four decode shapes with ordinary and with overlapped launches, the four irregular
             shapes, the M = 65536 prefill problem split over the ranks (strong scaling) without and with
             the all-gather of Y, and the square workload sustained for at least a second

`--impl reference` times the CPU path alone (all host threads) and prints the same line shape.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fp8_gemm_rowwise_tflops"
UNIT = "TFLOP/s"
L2_BYTES = 126e6

WORKLOADS = {
    # name: (M per GPU, N, K, x_std, w_std, dist, bound)
    "square_8192": (8192, 8192, 8192, 1.0, 1.0, "normal", "tensor"),
    "decode_m1": (1, 28672, 8192, 1.0, 0.02, "normal", "hbm"),
    "decode_m16": (16, 28672, 8192, 1.0, 0.02, "normal", "hbm"),
    "decode_m64": (64, 28672, 8192, 1.0, 0.02, "normal", "hbm"),
    "decode_m128": (128, 28672, 8192, 1.0, 0.02, "normal", "hbm"),
    "irregular_1000x5120x3584": (1000, 5120, 3584, 1.0, 1.0, "student_t3", "tensor"),
    "irregular_3000x7168x2048": (3000, 7168, 2048, 1.0, 1.0, "student_t3", "tensor"),
    "irregular_4096x14336x4096": (4096, 14336, 4096, 1.0, 1.0, "student_t3", "tensor"),
    "irregular_777x1024x8192": (777, 1024, 8192, 1.0, 1.0, "student_t3", "tensor"),
}
PREFILL_M, PREFILL_N, PREFILL_K = 65536, 8192, 8192
PARITY_ROWS = 64


def measured_peaks():
    """(fp8 tensor peak TFLOP/s burst, sustained, HBM GB/s, note).  The fp8 peak is twice the measured cuBLAS
    bf16 figure: kind::f8f6f4 runs on the same tensor pipe at twice the bf16 rate."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return (2.0 * float(p["bf16_tflops"]), 2.0 * float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                float(p["hbm_gbs"]), "of measured (fp8 peak = 2 x cuBLAS bf16)")
    return 2.0 * 1590.0, 2.0 * 1400.0, 6650.0, "of fallback (fp8 peak = 2 x 1.59 PFLOP/s burst, 2 x 1.4 sustained)"


def ncu_traffic(workload: str, plan: str):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the ncu capture recorded for
    this workload in profiles/ncu_traffic.md, or (None, why) when the table has no row for the workload or the
    row was captured with another kernel plan than the one the library picks now."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.md")
    if not os.path.exists(path):
        return None, "profiles/ncu_traffic.md is missing"
    for line in open(path):
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) < 5 or cells[0] != workload:
            continue
        want = cells[1].strip("`")
        if not plan.startswith(want):
            return None, f"profiles/ncu_traffic.md holds a capture of plan '{want}', the library now picks another"
        return float(cells[2]), f"profiles/{cells[4]} @ {cells[3]}"
    return None, "no ncu capture of this workload in profiles/ncu_traffic.md"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs (reading only)."""

    REASONS = {
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000080: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(index))
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons), "samples": 0}
        return {
            "sm_mhz": statistics.median(self.samples),
            "sm_min_mhz": min(self.samples),
            "sm_max_mhz": self.sm_max,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def physical_gpu_index(local_index: int) -> int:
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        parts = visible.split(",")
        if local_index < len(parts) and parts[local_index].strip().isdigit():
            return int(parts[local_index])
    return local_index


class NumaBinding:
    """While active, the calling thread runs on the CPUs NVML lists as close to the GPU, so that pinned host
    buffers allocated (and first touched) inside land on the GPU's own NUMA node.  The previous affinity is
    restored on exit.  Reads NVML only; changes nothing but this process's own CPU affinity."""

    def __init__(self, local_index: int):
        self.cpus, self.note, self._saved = None, "not bound", None
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(local_index))
            words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
            near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
            allowed = os.sched_getaffinity(0)
            if near & allowed:
                self.cpus = near & allowed
                self.note = f"{len(self.cpus)} of {len(allowed)} allowed CPUs are near the GPU"
            else:
                self.note = "NVML lists no allowed CPU near the GPU"
        except Exception as e:  # no NVML, no affinity support: stay where we are
            self.note = f"not bound ({type(e).__name__})"

    def __enter__(self):
        if self.cpus:
            self._saved = os.sched_getaffinity(0)
            os.sched_setaffinity(0, self.cpus)
        return self

    def __exit__(self, *exc):
        if self._saved is not None:
            os.sched_setaffinity(0, self._saved)


def host_threads(world: int = 1) -> int:
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, n // max(world, 1))


def cpu_oracle_rate(xq, wq, xs, ws, target_seconds: float, steps: int = 1, warmup: int = 0):
    """Times the CPU oracle on the first R rows of X, R sized from a probe so that one step takes about
    target_seconds.  Returns (TFLOP/s, threads, sample description, seconds per step)."""
    from oracle import fp8_rowwise_oracle as orc

    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1 to its ranks)
    try:
        torch.set_num_threads(host_threads())
    except RuntimeError:
        pass
    m, k = xq.shape
    n = wq.shape[0]

    def once(rows):
        t0 = time.perf_counter()
        orc.gemm_rowwise(xq[:rows], wq, xs[:rows], ws, decode="cast")
        return time.perf_counter() - t0

    # two probes separate the fixed cost (dequantising W) from the cost per row of X
    r_a, r_b = min(m, 32), min(m, 160)
    once(r_a)
    t_a, t_b = once(r_a), once(r_b)
    per_row = max((t_b - t_a) / max(r_b - r_a, 1), 1e-7)
    fixed = max(t_a - r_a * per_row, 0.0)
    rows = int(max(r_a, min(m, (target_seconds - fixed) / per_row)))
    for _ in range(warmup):
        orc.gemm_rowwise(xq[:rows], wq, xs[:rows], ws, decode="cast")
    times = []
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        orc.gemm_rowwise(xq[:rows], wq, xs[:rows], ws, decode="cast")
        times.append(time.perf_counter() - t0)
    t = sum(times) / len(times)
    sample = (
        f"rows 0..{rows - 1} of X against all of W ({rows}x{n}x{k}); torch CPU: X.float()*x_scale, W.float()*w_scale, "
        f"fp32 matmul, bf16 cast; {len(times)} timed pass(es)"
    )
    return orc.flops(rows, n, k) / t / 1e12, torch.get_num_threads(), sample, t


def run_reference(args, workload):
    """The reference's own path for this operator on a B200 box is the fp32 dequantise-then-matmul torch
    form on the host cores (every stock backend is disabled on B200 and FBGEMM is not in the tree)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from tritonbench_b200 import quantize

    m, n, k, x_std, w_std, dist, _ = WORKLOADS[workload]
    xq, wq, xs, ws = quantize.make_inputs(m, n, k, device="cpu", x_seed=0, dist=dist, x_std=x_std, w_std=w_std)
    rate, threads, sample, t_step = cpu_oracle_rate(xq, wq, xs, ws, target_seconds=1.5, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": rate,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": t_step * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp8_e4m3",
        "data": "synthetic",
        "config": {"workload": workload, "M_per_gpu": m, "N": n, "K": k, "step": sample},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- own arm
class Run:
    """State shared by the legs of one bench process: rank, device, barrier, max-over-ranks timing."""

    def __init__(self, args):
        import torch.distributed as td

        from tritonbench_b200 import dist as shard
        from tritonbench_b200 import lib

        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
        lib.load()  # fail loudly when the CUDA library is missing
        self.td, self.shard = td, shard
        self.rank, self.local_rank, self.world = shard.env_rank_world()
        if self.world != args.gpus:
            if self.world == 1 and args.gpus > 1:
                raise SystemExit(f"--gpus {args.gpus} needs a torchrun launch with {args.gpus} ranks")
            args.gpus = self.world
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self.grouped = shard.init_process_group("nccl") if self.world > 1 else False
        self.launches = 0
        self.parity_failures = []
        try:
            torch.set_num_threads(min(16, host_threads(self.world)))  # for the in-run oracle checks
        except RuntimeError:
            pass

    def barrier(self):
        torch.cuda.synchronize(self.device)
        if self.grouped:
            self.td.barrier()
        torch.cuda.synchronize(self.device)

    def max_over_ranks(self, value: float) -> float:
        if not self.grouped:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        self.td.all_reduce(t, op=self.td.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, ok: bool) -> bool:
        return self.max_over_ranks(0.0 if ok else 1.0) == 0.0

    def time_steps(self, step, steps, warmup, sampler=None):
        """ms per step: CUDA events on the launching stream around exactly `steps` back-to-back steps, barrier and
        synchronise on both sides, max over ranks."""
        from tritonbench_b200 import ops

        for i in range(warmup):
            step(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler is not None:
            sampler.__enter__()
        try:
            self.barrier()
            e0.record()
            for i in range(steps):
                step(i)
            e1.record()
            self.barrier()
        finally:
            if sampler is not None:
                sampler.__exit__(None, None, None)
        ops.check_device_status(self.device)
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps

    def parity(self, what, y, xq, wq, xs, ws, seed=0):
        """PARITY_ROWS rows of y (first and last among them) against the CPU oracle on the same operands."""
        from oracle import fp8_rowwise_oracle as orc  # the checker, never the thing measured

        m = xq.shape[0]
        g = torch.Generator().manual_seed(seed)
        rows = torch.randperm(m, generator=g)[: min(m, PARITY_ROWS)]
        if m > 1:
            rows[0], rows[-1] = 0, m - 1
        rows = rows.sort().values
        dev_rows = rows.to(xq.device)
        ref = orc.gemm_rowwise(xq[dev_rows].cpu(), wq.cpu(), xs[dev_rows].cpu(), ws.cpu(), decode="cast")
        res = orc.compare(y[rows.to(y.device)], ref)
        out = {"checked_rows": int(rows.numel()), "checked_elements": int(ref.numel()), "max_ratio": round(res["max_ratio"], 4),
               "ok": bool(res["ok"]), "bound": "1 bf16 ulp + 1e-2 RMS(ref)"}
        if not out["ok"]:
            self.parity_failures.append(f"rank {self.rank}: {what}: {res}")
        return out


def make_sets(quantize, m, n, k, dist_name, x_std, w_std, device, x_seed, w_seed, min_bytes, share_w=None):
    """Operand / output sets to rotate through so that no step finds its operands in L2 from the step before:
    enough copies that one trip around them moves more than `min_bytes`.  W is drawn once (every set multiplies
    the same weights); with share_w False each set has its own copy of it, so that W is cold as well."""
    wq, ws = quantize.make_quantized(n, k, seed=w_seed, device=device, dist=dist_name, std=w_std)
    per_set_private = m * k + 2 * m * n
    if share_w is None:
        share_w = n * k >= 2 * L2_BYTES  # a W this large cannot survive in L2 between steps anyway
    per_set = per_set_private + (0 if share_w else n * k)
    count = 3 if share_w else int(max(3, min(48, min_bytes // max(per_set, 1) + 1)))
    sets = []
    for b in range(count):
        xq, xs = quantize.make_quantized(m, k, seed=x_seed + 1000 * b, device=device, dist=dist_name, std=x_std)
        w_b = wq if (share_w or b == 0) else wq.clone()
        sets.append((xq, xs, w_b, torch.empty((m, n), dtype=torch.bfloat16, device=device)))
    return sets, wq, ws, count * per_set + (n * k if share_w else 0)


def gemm_leg(run, name, shape, dist_name, x_std, w_std, bound, steps, warmup, modes=("ordinary",), x_seed=None, sampler=None,
             min_seconds=0.0, share_w=None):
    """Times one GEMM shape on this rank (every rank runs the same leg on its own GPU) and checks the last Y."""
    from tritonbench_b200 import lib, ops, quantize

    m, n, k = shape
    fp8_peak, fp8_sustained, hbm_peak, peak_note = measured_peaks()
    seed = run.shard.shard_seed(run.rank) if x_seed is None else x_seed
    sets, wq, ws, rotation_bytes = make_sets(quantize, m, n, k, dist_name, x_std, w_std, run.device, seed, run.shard.W_SEED,
                                             2.2 * L2_BYTES, share_w=share_w)
    workspace = ops.get_workspace(run.device, ops.workspace_bytes(m, n, k))
    flops = 2.0 * m * n * k
    alg_bytes = m * k + n * k + 2 * m * n + 4 * (m + n)
    out = {"M": m, "N": n, "K": k, "plan": lib.describe_plan(m, n, k).split(" workspace=")[0],
           "l2": f"{len(sets)} operand sets rotated ({rotation_bytes / 1e6:.0f} MB per trip; L2 is 126 MB)", "steps": steps}
    first_y = None
    for mode in modes:
        overlap = mode == "overlapped"

        def step(i, overlap=overlap):
            xq, xs, w_b, y = sets[i % len(sets)]
            ops.fp8_gemm_rowwise(xq, w_b, xs, ws, out=y, workspace=workspace, overlap=overlap)

        n_steps = steps
        if min_seconds > 0.0:  # size the loop from a short probe so that it lasts at least min_seconds
            probe = run.time_steps(step, 10, warmup)
            n_steps = int(max(steps, min_seconds * 1e3 / probe + 1))
        ms = run.time_steps(step, n_steps, warmup, sampler=sampler)
        run.launches += n_steps
        last = (n_steps - 1) % len(sets)
        xq, xs, w_b, y = sets[last]
        rec = {"us_per_step": round(ms * 1e3, 3), "tflops": round(flops / (ms * 1e-3) / 1e12, 2),
               "gbs": round(alg_bytes / (ms * 1e-3) / 1e9, 1), "steps": n_steps}
        if bound == "hbm":
            rec["frac_of_hbm"] = round(rec["gbs"] / hbm_peak, 4)
        else:
            rec["frac_of_fp8_peak"] = round(rec["tflops"] / (fp8_sustained if min_seconds > 0 else fp8_peak), 4)
        if first_y is None:
            rec["parity"] = run.parity(f"{name} {mode}", y, xq, w_b, xs, ws, seed=m + n)
            first_y = y.clone()
        else:  # same operands, same buffer: the launch mode must not change a bit of the result
            same = bool(torch.equal(y, first_y))
            rec["parity"] = {"identical_to": modes[0], "ok": same}
            if not same:
                run.parity_failures.append(f"rank {run.rank}: {name} {mode}: differs from the {modes[0]} launches")
        out[mode] = rec
    out["peak"] = {"hbm_gbs": hbm_peak} if bound == "hbm" else {"fp8_tflops": fp8_sustained if min_seconds > 0 else fp8_peak}
    out["peak_source"] = peak_note
    return out


def prefill_leg(run, steps, warmup):
    """Strong scaling of the M = 65536 prefill problem: 65536 / world rows per rank, W replicated; the GEMM alone,
    and the GEMM followed by the in-place NCCL all-gather that assembles Y on every rank."""
    from tritonbench_b200 import lib, ops, quantize

    world, rank, device = run.world, run.rank, run.device
    m_total, n, k = PREFILL_M, PREFILL_N, PREFILL_K
    rows = m_total // world
    wq, ws = quantize.make_quantized(n, k, seed=run.shard.W_SEED, device=device)
    xq, xs = quantize.make_quantized(rows, k, seed=run.shard.shard_seed(rank), device=device)
    full, mine = run.shard.gathered_output(m_total, n, world, rank, device)
    workspace = ops.get_workspace(device, ops.workspace_bytes(rows, n, k))
    flops_total = 2.0 * m_total * n * k

    def gemm(i):
        ops.fp8_gemm_rowwise(xq, wq, xs, ws, out=mine, workspace=workspace)

    ms = run.time_steps(gemm, steps, warmup)
    run.launches += steps
    out = {
        "M_total": m_total, "N": n, "K": k, "rows_per_rank": rows, "scaling": "strong",
        "plan": lib.describe_plan(rows, n, k).split(" workspace=")[0],
        "l2": f"per-rank working set {(rows * k + n * k + 2 * rows * n) / 1e6:.0f} MB per step (L2 is 126 MB)",
        "gemm_only": {"ms_per_step": round(ms, 4), "tflops_total": round(flops_total / (ms * 1e-3) / 1e12, 1),
                      "tflops_per_gpu": round(flops_total / world / (ms * 1e-3) / 1e12, 1), "steps": steps,
                      "parity": run.parity("prefill_65536 gemm", mine, xq, wq, xs, ws, seed=7)},
    }
    if run.grouped:
        def gemm_gather(i):
            ops.fp8_gemm_rowwise(xq, wq, xs, ws, out=mine, workspace=workspace)
            run.shard.all_gather_rows(full, world)

        ms_g = run.time_steps(gemm_gather, steps, warmup)
        run.launches += steps
        # the gathered buffer holds every rank's shard: check the rows of the NEXT rank's shard against the oracle
        other = (rank + 1) % world
        xq_o, xs_o = quantize.make_quantized(rows, k, seed=run.shard.shard_seed(other), device=device)
        gathered = (world - 1) * 2 * rows * n
        out["with_all_gather"] = {
            "ms_per_step": round(ms_g, 4), "tflops_total": round(flops_total / (ms_g * 1e-3) / 1e12, 1), "steps": steps,
            "gathered_bytes_per_rank": gathered,
            "nvlink_gbs_if_serial": round(gathered / max((ms_g - ms) * 1e-3, 1e-9) / 1e9, 1),
            "how": "GEMM into this rank's slice of the [M,N] buffer, then in-place NCCL all_gather_into_tensor, same stream",
            "parity": run.parity("prefill_65536 gathered shard of the next rank", full[other * rows:(other + 1) * rows],
                                 xq_o, wq, xs_o, ws, seed=9),
        }
        # the same result from ONE kernel per rank: the GEMM's epilogue stores every tile into all ranks' copies of Y
        # (peer memory over NVLink); a one-element all-reduce orders the ranks after each step
        shared = run.shard.SharedRows(m_total, n, world, rank, device)
        copies = shared.my_rows_everywhere()
        token = torch.zeros(1, device=device)

        def fused(i):
            ops.fp8_gemm_rowwise_gather(xq, wq, xs, ws, copies, ldy=n, workspace=workspace)
            run.td.all_reduce(token)

        ms_f = run.time_steps(fused, steps, warmup)
        run.launches += steps
        same = bool(torch.equal(shared.full, full))
        if not same:
            run.parity_failures.append(f"rank {rank}: prefill_65536 fused gather differs from GEMM + NCCL all-gather")
        out["with_fused_all_gather"] = {
            "ms_per_step": round(ms_f, 4), "tflops_total": round(flops_total / (ms_f * 1e-3) / 1e12, 1), "steps": steps,
            "gathered_bytes_per_rank": gathered,
            "nvlink_gbs_out_per_gpu": round(gathered / (ms_f * 1e-3) / 1e9, 1),
            "nvlink_floor_ms": round(gathered / 770e9 * 1e3, 4),
            "how": "b200fp8_gemm_rowwise_gather: each tile TMA-stored into every rank's copy of Y (CUDA IPC mappings) from the "
                   "epilogue, then a one-element NCCL all-reduce as the barrier between ranks; nvlink_floor_ms = bytes a GPU "
                   "must send / 770 GB/s (the measured peer-copy rate)",
            "identical_to_nccl_path": same,
            "parity": run.parity("prefill_65536 fused gather, shard of the next rank", shared.full[other * rows:(other + 1) * rows],
                                 xq_o, wq, xs_o, ws, seed=10),
        }
        run.barrier()
        shared.close()
    return out


def measure_pcie(device, nbytes=128 << 20, reps=3):
    """Pinned host <-> device copy rates of this process, GB/s: each direction alone, and both at once."""
    h_a = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_b = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_a = torch.empty(nbytes, dtype=torch.uint8, device=device)
    d_b = torch.empty(nbytes, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def timed(fn):
        best = float("inf")
        for _ in range(reps + 1):
            torch.cuda.synchronize(device)
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize(device)
            best = min(best, time.perf_counter() - t0)
        return best

    def h2d():
        with torch.cuda.stream(s1):
            d_a.copy_(h_a, non_blocking=True)

    def d2h():
        with torch.cuda.stream(s2):
            h_b.copy_(d_b, non_blocking=True)

    def both():
        h2d()
        d2h()

    t_up, t_down, t_both = timed(h2d), timed(d2h), timed(both)
    return {"h2d_gbs": round(nbytes / t_up / 1e9, 2), "d2h_gbs": round(nbytes / t_down / 1e9, 2),
            "duplex_gbs_per_direction": round(nbytes / t_both / 1e9, 2), "copy_bytes": nbytes}


def e2e_leg(run, m, n, k, xq, xs, wq, ws, steps, flops_step_rank):
    """Wall clock over `steps` synchronous host-buffer calls (each: H2D copies, kernels, D2H copies), max over ranks;
    once with W sent by every call, once with W kept on the device; the last Y of each checked against the oracle."""
    from tritonbench_b200 import ops

    binding = NumaBinding(run.local_rank)
    with binding:  # pinned pages are placed where the allocating thread runs
        h_x = xq.view(torch.uint8).cpu().contiguous().pin_memory()
        h_w = wq.view(torch.uint8).cpu().contiguous().pin_memory()
        h_xs, h_ws = xs.cpu().pin_memory(), ws.cpu().pin_memory()
        h_out = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    # copy rates: every rank at the same time (what the calls below compete for), and rank 0 on its own
    run.barrier()
    pcie = measure_pcie(run.device)
    pcie_alone = None
    if run.world > 1:
        run.barrier()
        if run.rank == 0:
            pcie_alone = measure_pcie(run.device)
        run.barrier()
    host = ops.HostGemm(m, n, k)

    def loop(send_w: bool):
        args = (h_x, h_w if send_w else None, h_xs, h_ws if send_w else None)
        for _ in range(2):
            host(*args, out=h_out)
        run.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            host(*args, out=h_out)
        return run.max_over_ranks(time.perf_counter() - t0) / steps

    t_full = loop(True)
    parity_full = run.parity("e2e", h_out, xq, wq, xs, ws, seed=3)
    h_out.fill_(0)
    t_res = loop(False)  # W, w_scale of the last upload stay in the context
    parity_res = run.parity("e2e weights resident", h_out, xq, wq, xs, ws, seed=4)
    host.close()
    world = run.world
    h2d = m * k + n * k + 4 * (m + n)
    d2h = 2 * m * n
    bound_s = max(h2d / (pcie["h2d_gbs"] * 1e9), d2h / (pcie["d2h_gbs"] * 1e9))
    bound_res_s = max((m * k + 4 * m) / (pcie["h2d_gbs"] * 1e9), d2h / (pcie["d2h_gbs"] * 1e9))
    return {
        "value": world * flops_step_rank / t_full / 1e12,
        "unit": UNIT,
        "h2d_bytes_per_step": world * h2d,
        "d2h_bytes_per_step": world * d2h,
        "steps": steps,
        "ms_per_step": t_full * 1e3,
        "api": "b200fp8_gemm_rowwise_host (pinned host buffers in, pinned host buffer out, synchronous; X and W panels "
               "uploaded alternately, each newly computable strip of Y multiplied and downloaded at once)",
        "pcie": pcie,
        "pcie_one_rank_alone": pcie_alone,
        "pcie_bound_ms": bound_s * 1e3,
        "pcie_frac": bound_s / t_full,
        "pcie_frac_note": "max(h2d bytes / measured h2d rate, d2h bytes / measured d2h rate) / call time, with rank 0's rates "
                          "measured while every rank copies at once; 1.0 would need uploads and downloads to overlap completely",
        "aggregate_pcie_gbs": {"h2d": world * h2d / t_full / 1e9, "d2h": world * d2h / t_full / 1e9},
        "numa": binding.note,
        "parity": parity_full,
        "weights_resident": {
            "value": world * flops_step_rank / t_res / 1e12, "unit": UNIT, "ms_per_step": t_res * 1e3,
            "h2d_bytes_per_step": world * (m * k + 4 * m), "d2h_bytes_per_step": world * d2h,
            "pcie_frac": bound_res_s / t_res,
            "api": "b200fp8_host_ctx_set_weights once, then b200fp8_gemm_rowwise_host with wq = NULL (X up, Y down)",
            "parity": parity_res,
        },
    }


def run_own(args, workload):
    from tritonbench_b200 import lib, ops, quantize

    run = Run(args)
    rank, world, device = run.rank, run.world, run.device
    m, n, k, x_std, w_std, dist_name, bound = WORKLOADS[workload]
    steps, warmup = args.steps, max(args.warmup, 3)
    fp8_peak, fp8_sustained, hbm_peak, peak_note = measured_peaks()

    # W from the common seed on every rank (replicated), this rank's X rows from its shard seed.
    # Operand sets are rotated so that no step finds its X or Y in L2 from the step before.
    # (the headline workload keeps ONE W, as a serving job does: the 192 MB of X and Y that every step moves
    # through the 126 MB L2 leave little of the 64 MB W behind)
    sets, wq, ws, rotation_bytes = make_sets(quantize, m, n, k, dist_name, x_std, w_std, device, run.shard.shard_seed(rank),
                                             run.shard.W_SEED, 2.2 * L2_BYTES, share_w=True if workload == "square_8192" else None)
    workspace = ops.get_workspace(device, ops.workspace_bytes(m, n, k))
    # decode shapes: successive steps may overlap (each kernel reads only W before its predecessor is done)
    overlap = m <= 128 and not args.no_overlap

    def step(i):
        xq, xs, w_b, y = sets[i % len(sets)]
        ops.fp8_gemm_rowwise(xq, w_b, xs, ws, out=y, workspace=workspace, overlap=overlap)

    sampler = ClockSampler(run.local_rank, period_s=0.0005)  # the timed region may last only a few milliseconds
    ms_per_step = run.time_steps(step, steps, warmup, sampler=sampler)
    run.launches += steps
    timed_launches = steps
    flops_step_rank = 2.0 * m * n * k
    value = world * flops_step_rank / (ms_per_step * 1e-3) / 1e12
    last = sets[(steps - 1) % len(sets)]
    parity = run.parity("main", last[3], last[0], last[2], last[1], ws, seed=1)

    # ---- end to end through the host-buffer C-ABI entry point ----
    e2e = None
    if not args.kernel_only:
        e2e = e2e_leg(run, m, n, k, sets[0][0], sets[0][1], wq, ws, min(steps, 10), flops_step_rank)

    # ---- the other benchmark configurations (default workload only) ----
    also = None
    if workload == "square_8192" and not args.kernel_only and not args.no_also:
        also = {}
        leg_steps = max(args.also_steps, 20)
        for name in ("decode_m1", "decode_m16", "decode_m64", "decode_m128"):
            mm, nn, kk, xs_, ws_, dn, bd = WORKLOADS[name]
            also[name] = gemm_leg(run, name, (mm, nn, kk), dn, xs_, ws_, bd, max(leg_steps, 200), warmup,
                                  modes=("ordinary", "overlapped"), x_seed=0)
        for name in sorted(w for w in WORKLOADS if w.startswith("irregular_")):
            mm, nn, kk, xs_, ws_, dn, bd = WORKLOADS[name]
            also[name] = gemm_leg(run, name, (mm, nn, kk), dn, xs_, ws_, bd, leg_steps, warmup, x_seed=0)
        also["prefill_65536"] = prefill_leg(run, max(10, min(steps, 20)), warmup)
        sustained_sampler = ClockSampler(run.local_rank, period_s=0.02)
        sus = gemm_leg(run, "sustained", (m, n, k), dist_name, x_std, w_std, bound, steps, warmup, sampler=sustained_sampler,
                       min_seconds=args.sustained_seconds, share_w=True)
        sus["clocks"] = sustained_sampler.summary()
        sus["note"] = f"the headline workload back to back for at least {args.sustained_seconds} s; fraction of the sustained peak"
        also["sustained_square_8192"] = sus

    # ---- optional: the weak-scaling workload followed by an in-place NCCL all-gather of Y ----
    gather = None
    if run.grouped and args.gather:
        full, mine = run.shard.gathered_output(m * world, n, world, rank, device)

        def gemm_gather(i):
            xq, xs, w_b, _ = sets[i % len(sets)]
            ops.fp8_gemm_rowwise(xq, w_b, xs, ws, out=mine, workspace=workspace)
            run.shard.all_gather_rows(full, world)

        g_ms = run.time_steps(gemm_gather, steps, 2)
        gather = {
            "ms_per_step": g_ms,
            "value": world * flops_step_rank / (g_ms * 1e-3) / 1e12,
            "unit": UNIT,
            "gathered_bytes_per_rank": (world - 1) * 2 * m * n,
            "note": "GEMM into this rank's slice of the [M,N] buffer, then in-place NCCL all-gather, same stream",
        }

    all_ok = run.all_true(not run.parity_failures)
    if rank == 0:
        alg_bytes = m * k + n * k + 2 * m * n + 4 * (m + n)
        plan = lib.describe_plan(m, n, k)
        if bound == "tensor":
            achieved = flops_step_rank / (ms_per_step * 1e-3) / 1e12
            roofline = {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak}
        else:
            achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak}
        roofline["traffic"], roofline["traffic_source"] = ncu_traffic(workload, plan)
        roofline["peak_source"] = peak_note
        roofline["kernel"] = plan.split(" ")[0]
        roofline["algorithmic_flops_per_launch"] = flops_step_rank
        roofline["algorithmic_bytes_per_launch"] = alg_bytes

        cpu = None
        if world == 1 and not args.kernel_only:
            rate, threads, sample, _ = cpu_oracle_rate(sets[0][0].cpu(), wq.cpu(), sets[0][1].cpu(), ws.cpu(), target_seconds=12.0)
            cpu = {"value": rate, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}

        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": steps,
            "warmup": warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "fp8_e4m3",
            "data": "synthetic",
            "config": {
                "workload": workload,
                "M_per_gpu": m,
                "M_total": m * world,
                "N": n,
                "K": k,
                "sharding": f"rows of X and Y over {world} GPU(s), W replicated, no collective in the timed GEMM",
                "inputs": f"X ~ {dist_name}(std {x_std}), W ~ {dist_name}(std {w_std}), rowwise e4m3, fp32 scales; W seed 0, X seed 1+rank",
                "l2": f"{len(sets)} X and Y buffers rotated, {rotation_bytes / 1e6:.0f} MB per trip; per-step working set "
                      f"{alg_bytes / 1e6:.0f} MB (L2 is 126 MB)",
                "plan": plan,
                "launch": "programmatic dependent launch: a step may start (prefetching W only) before the previous step has finished"
                if overlap else "stream-ordered launches",
            },
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "parity": parity,
            "parity_all_legs_ok": all_ok,
            "gpu_launches": timed_launches * world,
            "gpu_launches_per_rank": timed_launches,
            "gpu_launches_all_legs_per_rank": run.launches,
            "clocks": sampler.summary(),
        }
        if also is not None:
            line["also"] = also
        if gather is not None:
            line["with_all_gather"] = gather
        print(json.dumps(line), flush=True)
    if run.parity_failures:
        print("PARITY FAILURE\n" + "\n".join(run.parity_failures), file=sys.stderr, flush=True)
    if run.grouped:
        run.td.barrier()
        run.td.destroy_process_group()
    if not all_ok:
        sys.exit(3)


AUX_WORKLOADS = ("row_quantize", "rms_norm_quantize", "silu_mul_quantize", "block_quantize", "blockwise_gemm", "rowwise_gemm")


def run_aux(args):
    """Times ONE kernel next to the hot path on one GPU - the quantisers, the block-scaled GEMM, or a single
    rowwise GEMM shape with a chosen variant - with CUDA events over --steps back-to-back calls after --warmup
    calls, and prints a small JSON line.  These are the commands the ncu summaries under profiles/ run; they
    are not the driver's bench line.  Sizes: --m rows, --k columns (quantisers); --m --n --k (GEMMs)."""
    from tritonbench_b200 import ops, quantize

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    m, n, k = args.m or 8192, args.n or 8192, args.k or 8192
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    what = args.workload
    nbytes, flops = None, None
    if what in ("row_quantize", "block_quantize", "rms_norm_quantize", "silu_mul_quantize"):
        if what.endswith("_quantize") and what not in ("row_quantize", "block_quantize"):
            dt = torch.bfloat16
        x = torch.randn((m, k), device="cuda", dtype=dt)
        nbytes = m * k * (x.element_size() + 1) + 4 * m
        if what == "row_quantize":
            fn = lambda: ops.fp8_row_quantize(x)  # noqa: E731
        elif what == "block_quantize":
            fn = lambda: ops.fp8_block_quantize(x)  # noqa: E731
        elif what == "rms_norm_quantize":
            w = torch.randn((k,), device="cuda", dtype=dt)
            fn = lambda: ops.rms_norm_fp8_rowwise_quant(x, w, round_bf16=args.round_bf16)  # noqa: E731
        else:
            x2 = torch.randn((m, k), device="cuda", dtype=dt)
            nbytes += m * k * 2
            fn = lambda: ops.silu_mul_fp8_rowwise_quant(x, x2, round_bf16=args.round_bf16)  # noqa: E731
    else:
        x = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
        w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
        out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        flops = 2.0 * m * n * k
        if what == "blockwise_gemm":
            xq, xs = quantize.fp8_block_quantize(x)
            wq, ws = quantize.fp8_block_quantize(w)
            fn = lambda: ops.fp8_gemm_blockwise(xq, wq, xs, ws, out=out)  # noqa: E731
        else:
            xq, xs = ops.fp8_row_quantize(x)
            wq, ws = ops.fp8_row_quantize(w)
            fn = lambda: ops.fp8_gemm_rowwise(xq, wq, xs, ws, out=out, variant=args.variant)  # noqa: E731
    for _ in range(max(args.warmup, 0)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_status()
    us = e0.elapsed_time(e1) / args.steps * 1e3
    line = {"workload": what, "M": m, "N": n if flops else None, "K": k, "dtype": args.dtype if nbytes else "fp8_e4m3",
            "steps": args.steps, "warmup": args.warmup, "us_per_call": round(us, 2)}
    if nbytes:
        line["gbs"] = round(nbytes / us / 1e3, 1)
    if flops:
        line["tflops"] = round(flops / us / 1e6, 1)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + list(AUX_WORKLOADS), default="square_8192")
    ap.add_argument("--m", type=int, help="single-kernel workloads: rows")
    ap.add_argument("--n", type=int, help="single-kernel GEMM workloads: columns of Y")
    ap.add_argument("--k", type=int, help="single-kernel workloads: columns of X")
    ap.add_argument("--dtype", choices=["bf16", "fp16", "fp32"], default="bf16", help="quantiser workloads: input type")
    ap.add_argument("--round-bf16", action="store_true", help="producer + quantiser workloads: round the activation to bf16 first")
    ap.add_argument("--variant", default="auto", help="rowwise_gemm workload: kernel variant")
    ap.add_argument("--gather", action="store_true", help="N>1: also time the weak-scaling GEMM + in-place NCCL all-gather of Y")
    ap.add_argument("--no-overlap", action="store_true", help="decode workloads: plain stream-ordered launches")
    ap.add_argument("--no-also", action="store_true", help="default workload: skip the legs for the other configurations")
    ap.add_argument("--also-steps", type=int, default=200, help="timed steps of each leg under `also`")
    ap.add_argument("--sustained-seconds", type=float, default=1.0)
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the device-timed loop of the workload (for short profiler captures; not a bench run)")
    args = ap.parse_args()
    if args.workload in AUX_WORKLOADS:
        run_aux(args)
    elif args.impl == "reference":
        run_reference(args, args.workload)
    else:
        run_own(args, args.workload)


if __name__ == "__main__":
    main()

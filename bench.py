#!/usr/bin/env python
"""Benchmark of the FP8 rowwise-scaled GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one pass of the GEMM over one batch of synthetic input.  The default workload is the
square configuration M = N = K = 8192 per GPU (X and Y sharded by rows, W replicated: with N GPUs
the job is the M = N*8192 prefill problem, i.e. M = 65536 at 8 GPUs).  Rank 0 prints ONE JSON line.

  value      whole-job TFLOP/s with inputs resident in HBM, timed with CUDA events on the launching
             stream over exactly K back-to-back steps, max over ranks
  e2e        the same metric through the host-buffer C-ABI call (b200fp8_gemm_rowwise_host): every
             step copies X, W and the scales from pinned host memory, runs the kernel and copies Y back
  roofline   achieved vs the measured tensor peak (large M) or HBM peak (decode workload)
  cpu_baseline  the CPU oracle (torch fp32 dequantise-then-matmul) timed on a bounded row sample

`--impl reference` times that CPU path alone (all host threads) and prints the same line shape.
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

# per-launch DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; None where no capture of that workload exists
NCU_TRAFFIC_BYTES = {
    "square_8192": 462.2e6,
    "decode_m16": 241.3e6,
}


def measured_peaks():
    """(fp8 tensor peak TFLOP/s, HBM GB/s, note).  The fp8 peak is twice the measured cuBLAS bf16
    figure: kind::f8f6f4 runs on the same tensor pipe at twice the bf16 rate."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return 2.0 * float(p["bf16_tflops"]), float(p["hbm_gbs"]), "of measured (fp8 peak = 2 x cuBLAS bf16 burst)"
    return 2.0 * 1590.0, 6650.0, "of fallback (fp8 peak = 2 x 1.59 PFLOP/s)"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000080: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
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
            "sm_max_mhz": self.sm_max,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def cpu_oracle_rate(xq, wq, xs, ws, target_seconds: float, steps: int = 1, warmup: int = 0):
    """Times the CPU oracle on the first R rows of X, R sized from a probe so that one step takes about
    target_seconds.  Returns (TFLOP/s, threads, sample description, seconds per step)."""
    from oracle import fp8_rowwise_oracle as orc

    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1 to its ranks)
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, RuntimeError):
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


def time_e2e(ops, m, n, k, x_pair, wq, ws, e2e_steps, barrier, grouped, device, world, flops_step_rank):
    """Wall-clock over e2e_steps synchronous host-buffer calls (each: H2D copies, kernel, D2H copy)."""
    import torch.distributed as td

    host = ops.HostGemm(m, n, k)
    h_in = [t.cpu().contiguous().pin_memory() for t in (x_pair[0].view(torch.uint8), wq.view(torch.uint8), x_pair[1], ws)]
    h_out = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        host(*h_in, out=h_out)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host(*h_in, out=h_out)
    t_e2e = time.perf_counter() - t0
    host.close()
    if grouped:
        t = torch.tensor([t_e2e], dtype=torch.float64, device=device)
        td.all_reduce(t, op=td.ReduceOp.MAX)
        t_e2e = float(t.item())
    return t_e2e, world * flops_step_rank * e2e_steps / t_e2e / 1e12


def run_own(args, workload):
    import torch.distributed as td

    from tritonbench_b200 import dist as shard
    from tritonbench_b200 import lib, ops, quantize

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    lib.load()  # fail loudly when the CUDA library is missing

    rank, local_rank, world = shard.env_rank_world()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs a torchrun launch with {args.gpus} ranks")
        args.gpus = world
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    grouped = shard.init_process_group("nccl") if world > 1 else False

    m, n, k, x_std, w_std, dist_name, bound = WORKLOADS[workload]
    steps, warmup = args.steps, max(args.warmup, 3)

    # W from the common seed on every rank (replicated), this rank's X rows from its shard seed.
    # Three X / Y buffers are rotated so that no step finds its X or Y in L2 from the step before.
    n_buf = 3
    wq, ws = quantize.make_quantized(n, k, seed=shard.W_SEED, device=device, dist=dist_name, std=w_std)
    xs_list = [
        quantize.make_quantized(m, k, seed=shard.shard_seed(rank) + 1000 * b, device=device, dist=dist_name, std=x_std)
        for b in range(n_buf)
    ]
    outs = [torch.empty((m, n), dtype=torch.bfloat16, device=device) for _ in range(n_buf)]
    workspace = ops.get_workspace(device, ops.workspace_bytes(m, n, k))

    # decode shapes: successive steps may overlap (each kernel reads only W before its predecessor is done)
    overlap = m <= 128 and not args.no_overlap

    def step(i):
        xq, xs = xs_list[i % n_buf]
        ops.fp8_gemm_rowwise(xq, wq, xs, ws, out=outs[i % n_buf], workspace=workspace, overlap=overlap)

    def barrier():
        torch.cuda.synchronize(device)
        if grouped:
            td.barrier()
        torch.cuda.synchronize(device)

    for i in range(warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        barrier()
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        barrier()
    ops.check_device_status(device)
    t_ms = e0.elapsed_time(e1)
    if grouped:
        t = torch.tensor([t_ms], dtype=torch.float64, device=device)
        td.all_reduce(t, op=td.ReduceOp.MAX)
        t_ms = float(t.item())
    ms_per_step = t_ms / steps
    flops_step_rank = 2.0 * m * n * k
    value = world * flops_step_rank / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the host-buffer C-ABI entry point ----
    e2e_steps = 0 if args.kernel_only else min(steps, 10)
    t_e2e, e2e_value = None, None
    if e2e_steps:
        t_e2e, e2e_value = time_e2e(ops, m, n, k, xs_list[0], wq, ws, e2e_steps, barrier, grouped, device, world, flops_step_rank)
    h2d = world * (m * k + n * k + 4 * (m + n))
    d2h = world * 2 * m * n

    # ---- optional: assemble Y on every rank with an in-place NCCL all-gather after each GEMM ----
    gather = None
    if grouped and args.gather:
        full, mine = shard.gathered_output(m * world, n, world, rank, device)
        for i in range(2):
            ops.fp8_gemm_rowwise(xs_list[0][0], wq, xs_list[0][1], ws, out=mine, workspace=workspace)
            shard.all_gather_rows(full, world)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for i in range(steps):
            xq, xs = xs_list[i % n_buf]
            ops.fp8_gemm_rowwise(xq, wq, xs, ws, out=mine, workspace=workspace)
            shard.all_gather_rows(full, world)
        g1.record()
        barrier()
        t = torch.tensor([g0.elapsed_time(g1)], dtype=torch.float64, device=device)
        td.all_reduce(t, op=td.ReduceOp.MAX)
        g_ms = float(t.item()) / steps
        gather = {
            "ms_per_step": g_ms,
            "value": world * flops_step_rank / (g_ms * 1e-3) / 1e12,
            "unit": UNIT,
            "gathered_bytes_per_rank": (world - 1) * 2 * m * n,
            "note": "GEMM into this rank's slice of the [M,N] buffer, then in-place NCCL all-gather, same stream",
        }

    if rank == 0:
        fp8_peak, hbm_peak, peak_note = measured_peaks()
        alg_bytes = m * k + n * k + 2 * m * n + 4 * (m + n)
        if bound == "tensor":
            achieved = flops_step_rank / (ms_per_step * 1e-3) / 1e12
            roofline = {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak}
        else:
            achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak}
        roofline["traffic"] = NCU_TRAFFIC_BYTES.get(workload)
        roofline["peak_source"] = peak_note
        roofline["kernel"] = lib.describe_plan(m, n, k).split(" ")[0]
        roofline["algorithmic_flops_per_launch"] = flops_step_rank
        roofline["algorithmic_bytes_per_launch"] = alg_bytes

        cpu = None
        if world == 1 and not args.kernel_only:
            xq_h, xs_h = xs_list[0][0].cpu(), xs_list[0][1].cpu()
            rate, threads, sample, _ = cpu_oracle_rate(xq_h, wq.cpu(), xs_h, ws.cpu(), target_seconds=12.0)
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
                "l2": f"{n_buf} X and Y buffers rotated; per-step working set {alg_bytes / 1e6:.0f} MB (L2 is 126 MB)",
                "plan": lib.describe_plan(m, n, k),
                "launch": "programmatic dependent launch: a step may start (prefetching W only) before the previous step has finished"
                if overlap else "stream-ordered launches",
            },
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": None if not e2e_steps else {
                "value": e2e_value,
                "unit": UNIT,
                "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h,
                "steps": e2e_steps,
                "ms_per_step": t_e2e / e2e_steps * 1e3,
                "api": "b200fp8_gemm_rowwise_host (pinned host buffers in, pinned host buffer out, synchronous)",
            },
            "gpu_launches": steps * world,
            "gpu_launches_per_rank": steps,
            "clocks": sampler.summary(),
        }
        if gather is not None:
            line["with_all_gather"] = gather
        print(json.dumps(line), flush=True)
    if grouped:
        td.barrier()
        td.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="square_8192")
    ap.add_argument("--gather", action="store_true", help="N>1: also time GEMM + in-place NCCL all-gather of Y")
    ap.add_argument("--no-overlap", action="store_true", help="decode workloads: plain stream-ordered launches")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (for short profiler captures; not a bench run)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args, args.workload)
    else:
        run_own(args, args.workload)


if __name__ == "__main__":
    main()

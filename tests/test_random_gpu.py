"""Seeded random shapes through every GEMM entry point other than the plain rowwise call (which
tests/test_gemm_gpu.py draws at random against cuBLASLt): grouped, block-scaled, the host-buffer pipeline with
random panel sizes, and the GEMM that stores into several copies of Y.  Each case is compared with the CPU oracle
under the tolerance the benchmark specification states, and canary values around the outputs must survive."""
import random

import pytest
import torch

from oracle import fp8_rowwise_oracle as orc

pytestmark = pytest.mark.gpu


def _close(y, ref, what):
    res = orc.compare(y, ref)
    assert res["ok"], f"{what}: {res}"


def _quantized(rows, cols, seed, std=1.0, dist="normal"):
    from tritonbench_b200 import quantize

    return quantize.make_quantized(rows, cols, seed=seed, std=std, dist=dist)


def test_random_grouped_problems(cuda_device):
    from tritonbench_b200 import ops

    rng = random.Random(4101)
    for case in range(24):
        groups = rng.randint(1, 8)
        n = 16 * rng.randint(1, 60)
        k = 16 * rng.randint(1, 50)
        sizes = [rng.choice([0, 1, 5, 64, 128, 200, 300, 513]) for _ in range(groups)]
        spare = rng.choice([0, 0, 7])  # rows after the last group: never written
        m_total = sum(sizes) + spare
        if m_total == 0:
            continue
        xq, xs = _quantized(m_total, k, seed=case)
        wq, ws = _quantized(groups * n, k, seed=1000 + case, std=0.05)
        m_sizes = torch.tensor(sizes, dtype=torch.int32)
        out = torch.full((m_total, n), 3.0, dtype=torch.bfloat16, device="cuda")
        variant = rng.choice(["auto", "tc_1cta", "tc_2cta"])
        ops.fp8_gemm_rowwise_grouped(xq.cuda(), wq.cuda(), m_sizes.cuda(), xs.cuda(), ws.cuda(), out=out, variant=variant)
        ops.check_device_status()
        used = sum(sizes)
        if used:
            ref = orc.gemm_rowwise_grouped(xq[:used], wq, m_sizes, xs[:used], ws)
            _close(out[:used], ref, f"grouped {sizes} N={n} K={k} {variant}")
        assert bool((out[used:] == 3.0).all()), f"grouped {sizes}: rows beyond the groups were written"


def test_random_block_scaled_problems(cuda_device):
    from tritonbench_b200 import ops

    rng = random.Random(4102)
    gen = torch.Generator().manual_seed(4102)
    for case in range(16):
        m = rng.choice([1, 64, 128, 129, 300, 777, 1024])
        n = 16 * rng.randint(1, 80)
        k = 16 * rng.randint(1, 60)
        x = torch.randn(m, k, generator=gen)
        w = torch.randn(n, k, generator=gen) * 0.05
        xq, xs = orc.block_quantize_reference(x)
        wq, ws = orc.block_quantize_reference(w)
        ref = orc.gemm_blockwise(xq, wq, xs, ws)
        out_buf = torch.full((m, n + 16), 5.0, dtype=torch.bfloat16, device="cuda")
        y = ops.fp8_gemm_blockwise(xq.cuda(), wq.cuda(), xs.cuda(), ws.cuda(), out=out_buf[:, :n], tma_store=rng.random() < 0.75)
        ops.check_device_status()
        _close(y, ref, f"blockwise {m}x{n}x{k}")
        assert bool((out_buf[:, n:] == 5.0).all()), f"blockwise {m}x{n}x{k}: wrote past the row"


def test_random_host_pipeline_problems_and_panel_sizes(cuda_device):
    from tritonbench_b200 import ops

    rng = random.Random(4103)
    for case in range(10):
        m = rng.choice([1, 16, 300, 1024, 2048 + 37, 3000])
        n = 16 * rng.randint(1, 120)
        k = 16 * rng.randint(1, 40)
        xq, xs = _quantized(m, k, seed=case)
        wq, ws = _quantized(n, k, seed=2000 + case, std=0.05)
        bias = (torch.randn(n) * 0.5).bfloat16() if rng.random() < 0.5 else None
        panels = rng.choice([None, (1024, 1024), (512, 2048), (2048, 512), (256, 256)])
        ref = orc.gemm_rowwise(xq, wq, xs, ws, bias)
        gemm = ops.HostGemm(m, n, k, panels=panels)
        try:
            y = gemm(xq, wq, xs, ws, bias=bias).clone()
            y_resident = gemm(xq, None, xs, None).clone()  # W, w_scale and bias of the call above stay on the device
        finally:
            gemm.close()
        _close(y, ref, f"host {m}x{n}x{k} panels={panels}")
        _close(y_resident, ref, f"host, resident weights {m}x{n}x{k} panels={panels}")


def test_random_problems_stored_into_several_copies(cuda_device):
    from tritonbench_b200 import ops

    rng = random.Random(4104)
    for case in range(12):
        m = rng.choice([1, 100, 128, 256, 1000, 2048])
        n = 8 * rng.randint(1, 160)
        k = 16 * rng.randint(1, 50)
        copies = rng.randint(1, 8)
        xq, xs = _quantized(m, k, seed=case, dist="student_t3" if case % 3 == 0 else "normal")
        wq, ws = _quantized(n, k, seed=3000 + case, std=0.05)
        ref = orc.gemm_rowwise(xq, wq, xs, ws)
        bufs = [torch.full((m + 5, n), 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(copies)]
        variant = rng.choice(["auto", "tc_1cta", "tc_2cta"])
        ops.fp8_gemm_rowwise_gather(xq.cuda(), wq.cuda(), xs.cuda(), ws.cuda(), [b[2:2 + m].data_ptr() for b in bufs], n,
                                    variant=variant)
        ops.check_device_status()
        _close(bufs[0][2:2 + m], ref, f"gather {m}x{n}x{k} x{copies} {variant}")
        for b in bufs:
            assert torch.equal(b, bufs[0]), "the copies differ"
            assert bool((b[:2] == 9.0).all()) and bool((b[2 + m:] == 9.0).all()), "rows outside the call's slice were written"

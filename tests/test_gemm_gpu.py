"""Parity of the CUDA path against the oracle, through the C ABI (tritonbench_b200.ops is a thin
ctypes wrapper).  Tolerance everywhere: max |out - ref| <= 1 bf16 ulp of |ref| + 1e-2 * RMS(ref)
(oracle.fp8_rowwise_oracle.tolerance), the bound the benchmark specification states."""
import os

import numpy as np
import pytest
import torch

from oracle import fp8_rowwise_oracle as orc

pytestmark = pytest.mark.gpu

TC_VARIANTS = ("tc_1cta", "tc_2cta")


def _ops():
    from tritonbench_b200 import ops

    return ops


def _gpu(*ts):
    return [t.cuda() if t is not None else None for t in ts]


def _run(variant, xq, wq, xs, ws, bias=None, **kw):
    ops = _ops()
    y = ops.fp8_gemm_rowwise(*_gpu(xq, wq, xs, ws), bias=bias.cuda() if bias is not None else None, variant=variant, **kw)
    ops.check_device_status()
    return y


def _assert_close(y, ref, what=""):
    res = orc.compare(y, ref)
    assert res["ok"], f"{what}: {res}"
    return res


def _inputs(m, n, k, seed=0, dist="normal", w_std=1.0):
    from tritonbench_b200 import quantize

    return quantize.make_inputs(m, n, k, device="cpu", x_seed=seed, dist=dist, w_std=w_std)


def _bf16(bits):
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


# ------------------------------------------------------------------ golden fixtures
@pytest.mark.parametrize("variant", ["auto", "tc_1cta", "tc_2cta", "skinny", "simt"])
@pytest.mark.parametrize("fixture", ["config1_seed0_128x256x512.npz", "ref_quantizer_bf16_128x256x512.npz"])
def test_golden_fixture(cuda_device, golden_dir, variant, fixture):
    d = np.load(os.path.join(golden_dir, fixture))
    xq, wq = torch.from_numpy(d["xq"]).view(torch.float8_e4m3fn), torch.from_numpy(d["wq"]).view(torch.float8_e4m3fn)
    xs, ws = torch.from_numpy(d["x_scale"]), torch.from_numpy(d["w_scale"])
    y = _run(variant, xq, wq, xs, ws)
    _assert_close(y, _bf16(d["y_bf16"]), f"{variant} {fixture}")


# ------------------------------------------------------------------ ragged / tail shapes
TAIL_SHAPES = [
    (1, 8, 16), (129, 257, 144), (130, 264, 400), (255, 1001, 1040), (777, 1024, 2048), (300, 520, 3584),
    (513, 768, 128), (256, 512, 16), (1000, 5120, 512),
]


@pytest.mark.parametrize("variant", TC_VARIANTS)
@pytest.mark.parametrize("shape", TAIL_SHAPES)
def test_tile_tails_large_m_kernels(cuda_device, variant, shape):
    m, n, k = shape
    xq, wq, xs, ws = _inputs(m, n, k, seed=m + n + k)
    ref = orc.gemm_rowwise(xq, wq, xs, ws)
    _assert_close(_run(variant, xq, wq, xs, ws), ref, f"{variant} {shape}")
    _assert_close(_run(variant, xq, wq, xs, ws, tma_store=False), ref, f"{variant} {shape} plain stores")


SPLITK_SHAPES = [(777, 1024, 8192), (256, 512, 4096), (129, 257, 144), (300, 520, 400), (128, 256, 128), (1, 8, 16),
                 (512, 1024, 16384), (1000, 1001, 1040)]


@pytest.mark.parametrize("shape", SPLITK_SHAPES)
def test_cluster_split_k_kernel(cuda_device, shape):
    """K split across the CTAs of a cluster, partial sums exchanged over distributed shared memory."""
    m, n, k = shape
    xq, wq, xs, ws = _inputs(m, n, k, seed=3 * m + k)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(1)) * 10).to(torch.bfloat16)
    ref = orc.gemm_rowwise(xq, wq, xs, ws)
    y = _run("tc_splitk", xq, wq, xs, ws)
    _assert_close(y, ref, f"tc_splitk {shape}")
    assert torch.equal(_run("tc_splitk", xq, wq, xs, ws), y)  # fixed summation order: run-to-run identical
    _assert_close(_run("tc_splitk", xq, wq, xs, ws, tma_store=False), ref, f"tc_splitk {shape} plain stores")
    _assert_close(_run("tc_splitk", xq, wq, xs, ws, bias=bias), orc.gemm_rowwise(xq, wq, xs, ws, bias), "tc_splitk bias")
    _assert_close(_run("tc_splitk", xq, wq, xs, ws, out_dtype=torch.float16),
                  orc.gemm_rowwise(xq, wq, xs, ws, out_dtype=torch.float16), "tc_splitk fp16")


SPLIT_CONFIGS = [(256, 1), (256, 2), (256, 4), (256, 8), (128, 1), (128, 2), (128, 4), (128, 8), (64, 1), (64, 2), (64, 4),
                 (208, 1), (16, 1), (48, 1), (96, 2), (192, 4), (160, 2),
                 (320, 1), (384, 1), (448, 1)]  # wider than 256 columns: two MMA halves, one CTA, no K split


@pytest.mark.parametrize("config", SPLIT_CONFIGS)
def test_every_tile_width_and_cluster_size_of_the_one_tile_per_cluster_kernel(cuda_device, config):
    """B200FP8_FLAG_SPLITK_CONFIG: each (tile width, cluster size) on a decode shape (X stage of 8 rows, deep
    ring), a ragged mid-size shape (tails in M, N and K, several row tiles) and a K shorter than the split."""
    shapes = [(5, 1000, 2320), (300, 520, 1424), (64, 256, 128)]
    if config[0] > 256:
        shapes.append((260, 1500, 640))  # several wide tiles in both directions, ragged everywhere
    for m, n, k in shapes:
        xq, wq, xs, ws = _inputs(m, n, k, seed=m + n + k)
        ref = orc.gemm_rowwise(xq, wq, xs, ws)
        y = _run("tc_splitk", xq, wq, xs, ws, split_config=config)
        _assert_close(y, ref, f"tc_splitk {config} {(m, n, k)}")
        assert torch.equal(_run("tc_splitk", xq, wq, xs, ws, split_config=config, overlap=True), y)
        _assert_close(_run("tc_splitk", xq, wq, xs, ws, split_config=config, tma_store=False), ref,
                      f"tc_splitk {config} {(m, n, k)} plain stores")


def test_split_config_flag_rejects_impossible_combinations(cuda_device):
    ops = _ops()
    xq, wq, xs, ws = _gpu(*_inputs(16, 256, 512))
    # 64 / 8 < 16; 3 CTAs; a wide tile must be a multiple of 64 columns and cannot split K; 48 is not a multiple of 32
    for bad in [(64, 8), (128, 3), (272, 1), (288, 1), (320, 2), (48, 2)]:
        with pytest.raises(Exception):
            ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant="tc_splitk", split_config=bad)
    ops.check_device_status()


SKINNY_SHAPES = [
    (1, 8, 16), (1, 256, 512), (3, 1000, 1040), (8, 2304, 2304), (16, 1024, 1024), (17, 520, 400), (33, 4096, 2304),
    (64, 4096, 2048), (100, 1000, 4096), (128, 2304, 6656), (127, 129, 144),
]


@pytest.mark.parametrize("shape", SKINNY_SHAPES)
def test_skinny_kernel_shapes(cuda_device, shape):
    m, n, k = shape
    xq, wq, xs, ws = _inputs(m, n, k, seed=7 * m + n)
    ref = orc.gemm_rowwise(xq, wq, xs, ws)
    _assert_close(_run("skinny", xq, wq, xs, ws), ref, f"skinny {shape}")


GEMV_SHAPES = [(1, 8, 16), (1, 1000, 2320), (2, 520, 400), (3, 2304, 2304), (4, 4096, 6656), (1, 28672, 8192), (2, 9000, 8192),
               (4, 129, 144), (1, 5000, 16384)]


@pytest.mark.parametrize("shape", GEMV_SHAPES)
def test_gemv_kernel_for_one_to_four_tokens(cuda_device, shape):
    """The CUDA-core GEMV (128-bit loads of whole rows of W, fp32 accumulation, warp-shuffle reduction): ragged N, K tails
    of whole 16-byte chunks, bias, fp16 output, a pitched X, and overlapped launches that must not change a bit."""
    ops = _ops()
    m, n, k = shape
    xq, wq, xs, ws = _inputs(m, n, k, seed=11 * m + n, w_std=0.02)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(3)) * 0.5).to(torch.bfloat16)
    ref = orc.gemm_rowwise(xq, wq, xs, ws)
    y = _run("gemv", xq, wq, xs, ws)
    _assert_close(y, ref, f"gemv {shape}")
    _assert_close(_run("gemv", xq, wq, xs, ws, bias=bias), orc.gemm_rowwise(xq, wq, xs, ws, bias), f"gemv {shape} bias")
    _assert_close(_run("gemv", xq, wq, xs, ws, out_dtype=torch.float16), orc.gemm_rowwise(xq, wq, xs, ws, out_dtype=torch.float16),
                  f"gemv {shape} fp16")
    big_x = torch.zeros((m, k + 64), dtype=torch.uint8, device="cuda")
    big_x[:, :k] = xq.view(torch.uint8).cuda()
    out_big = torch.zeros((m, n + 8), dtype=torch.bfloat16, device="cuda")
    got = ops.fp8_gemm_rowwise(big_x[:, :k], wq.cuda(), xs.cuda(), ws.cuda(), out=out_big[:, :n], variant="gemv")
    assert torch.equal(got, y) and float(out_big[:, n:].abs().max()) == 0.0
    for _ in range(3):  # back to back with overlapped launches
        assert torch.equal(ops.fp8_gemm_rowwise(*_gpu(xq, wq, xs, ws), variant="gemv", overlap=True), y)
    ops.check_device_status()
    # the tensor-core decode kernel computes the same sums in another order: equal within the tolerance
    _assert_close(_run("tc_splitk", xq, wq, xs, ws), y.cpu(), f"gemv {shape} vs tc_splitk")


def test_gemv_kernel_refuses_what_it_cannot_take(cuda_device):
    ops = _ops()
    xq, wq, xs, ws = _gpu(*_inputs(5, 256, 256))
    with pytest.raises(Exception):
        ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant="gemv")  # five tokens
    xq, wq, xs, ws = _inputs(2, 64, 136)  # K is not a multiple of 16
    big_x = torch.zeros((2, 144), dtype=torch.uint8, device="cuda")
    big_w = torch.zeros((64, 144), dtype=torch.uint8, device="cuda")
    with pytest.raises((NotImplementedError, ValueError)):  # no plan: refused when the workspace is sized, or by the call
        ops.fp8_gemm_rowwise(big_x[:, :136], big_w[:, :136], xs.cuda(), ws.cuda(), variant="gemv")
    from tritonbench_b200 import lib

    ws256 = torch.zeros(256, dtype=torch.uint8, device="cuda")
    with pytest.raises(NotImplementedError):
        ops.fp8_gemm_rowwise(big_x[:, :136], big_w[:, :136], xs.cuda(), ws.cuda(), variant="gemv", workspace=ws256)

    assert lib.describe_plan(1, 28672, 8192).startswith("tc_splitk")  # auto never takes it: measured slower
    assert lib.describe_plan(1, 28672, 8192, lib.VARIANT_GEMV).startswith("gemv tokens=1 rows_per_warp=7 ctas=256")
    ops.check_device_status()


def test_skinny_workspace_survives_changes_of_geometry(cuda_device):
    """One workspace, problem sizes with different tile counts back to back: the counters a call
    leaves behind must still be zero where the next call looks for its own."""
    ops = _ops()
    from tritonbench_b200 import lib

    ws_bytes = max(ops.workspace_bytes(m, n, k, lib.VARIANT_SKINNY) for (m, n, k) in SKINNY_SHAPES)
    workspace = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    for rep in range(2):
        for (m, n, k) in [(64, 4096, 2048), (1, 8192, 4096), (100, 1000, 4096), (8, 2304, 2304), (16, 1024, 1024)]:
            xq, wq, xs, wsc = _inputs(m, n, k, seed=rep)
            y = ops.fp8_gemm_rowwise(*_gpu(xq, wq, xs, wsc), variant="skinny", workspace=workspace)
            _assert_close(y, orc.gemm_rowwise(xq, wq, xs, wsc), f"skinny {(m, n, k)} rep {rep}")
    torch.cuda.synchronize()
    assert int(workspace[: 256 + 262144].to(torch.int64).sum()) == 0  # status word and counters are zero again


# ------------------------------------------------------------------ benchmark configurations
@pytest.mark.parametrize("m", [1, 16, 64, 128])
def test_config3_decode_shapes(cuda_device, m):
    xq, wq, xs, ws = _inputs(m, 28672, 8192, seed=0, w_std=0.02)
    ref = orc.gemm_rowwise(xq, wq, xs, ws)
    res = _assert_close(_run("auto", xq, wq, xs, ws), ref, f"decode M={m}")
    assert res["max_ratio"] < 0.9


@pytest.mark.parametrize("shape", [(1000, 5120, 3584), (3000, 7168, 2048), (4096, 14336, 4096), (777, 1024, 8192)])
def test_config5_irregular_student_t(cuda_device, shape):
    m, n, k = shape
    xq, wq, xs, ws = _inputs(m, n, k, seed=0, dist="student_t3")
    ref32 = orc.gemm_rowwise(xq, wq, xs, ws, keep_fp32=True)
    ref = ref32.to(torch.bfloat16)
    for variant in ("auto",) + TC_VARIANTS:
        y = _run(variant, xq, wq, xs, ws)
        _assert_close(y, ref, f"{variant} {shape}")
        # stricter, per row: heavy rows must not hide errors in light rows behind the global RMS
        yf, rf = y.float().cpu(), ref.float()
        row_rms = ref32.pow(2).mean(dim=1, keepdim=True).sqrt()
        assert bool(((yf - rf).abs() <= orc.bf16_ulp(rf) + 1e-2 * row_rms).all()), f"{variant} {shape} per-row bound"


def test_config2_square_8192_against_oracle_rows_and_cuda_core_kernel(cuda_device):
    m = n = k = 8192
    from tritonbench_b200 import quantize

    xq, wq, xs, ws = quantize.make_inputs(m, n, k, device="cuda", x_seed=0)
    ops = _ops()
    y2 = ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant="tc_2cta")
    y1 = ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant="tc_1cta")
    ya = ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant="auto")
    ysimt = ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant="simt")
    ops.check_device_status()
    assert torch.equal(ya, y2)  # auto picks the CTA-pair kernel here
    # every element against the CUDA-core kernel (independent data path, fp32 FMA in ascending k)
    rms = ysimt.float().pow(2).mean().sqrt()
    for y in (y1, y2):
        diff = (y.float() - ysimt.float()).abs()
        ulp = torch.exp2(torch.floor(torch.log2(ysimt.float().abs().clamp(min=2.0 ** -126))) - 7.0)
        assert bool((diff <= ulp + 1e-2 * rms).all())
    # 512 rows against the CPU oracle (first tile, last tile, and a seeded sample)
    g = torch.Generator().manual_seed(0)
    rows = torch.cat([torch.arange(0, 128), torch.arange(m - 128, m), torch.randperm(m, generator=g)[:256]])
    ref = orc.gemm_rowwise(xq[rows.cuda()].cpu(), wq.cpu(), xs[rows.cuda()].cpu(), ws.cpu())
    for y in (y1, y2):
        _assert_close(y[rows.cuda()], ref, "8192^3 row sample")


def test_full_size_properties_permutation_and_power_of_two_scaling(cuda_device):
    """Size-independent properties at the full 8192^3 size: a row of Y depends only on its row of X
    (bit-exact under a permutation of rows), and multiplying a scale by a power of two multiplies
    the output by exactly that power."""
    m = n = k = 8192
    from tritonbench_b200 import quantize

    xq, wq, xs, ws = quantize.make_inputs(m, n, k, device="cuda", x_seed=1)
    ops = _ops()
    y = ops.fp8_gemm_rowwise(xq, wq, xs, ws)
    perm = torch.randperm(m, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    yp = ops.fp8_gemm_rowwise(xq.view(torch.uint8)[perm].view(torch.float8_e4m3fn), wq, xs[perm], ws)
    assert torch.equal(yp, y[perm])
    y4 = ops.fp8_gemm_rowwise(xq, wq, xs * 4.0, ws * 0.5)
    assert torch.equal(y4.float(), y.float() * 2.0)
    again = ops.fp8_gemm_rowwise(xq, wq, xs, ws)
    assert torch.equal(again, y)
    ops.check_device_status()


def test_config4_prefill_shards_as_the_ranks_compute_them(cuda_device):
    """The sharded run's unit of work: 8192-row shards of the M=65536 prefill problem (shard seeds of ranks
    0, 3 and 7, W from the common seed), each as its own GEMM, sampled rows against the oracle."""
    from tritonbench_b200 import dist, quantize

    n = k = 8192
    wq, ws = quantize.make_quantized(n, k, seed=dist.W_SEED, device="cuda")
    ops = _ops()
    for rank in (0, 3, 7):
        xq, xs = quantize.make_quantized(8192, k, seed=dist.shard_seed(rank), device="cuda")
        y = ops.fp8_gemm_rowwise(xq, wq, xs, ws)
        rows = torch.arange(rank * 16, 8192, 128, device="cuda")
        ref = orc.gemm_rowwise(xq[rows].cpu(), wq.cpu(), xs[rows].cpu(), ws.cpu())
        _assert_close(y[rows], ref, f"prefill shard {rank}")
    ops.check_device_status()


def test_config4_whole_prefill_problem_in_one_launch(cuda_device):
    """M=65536, N=K=8192 as ONE launch on one GPU (X 512 MiB, Y 1 GiB): 64 sampled rows of every 8192-row
    band against the oracle, first and last row of the problem included; the bands are also what the ranks of
    a sharded run produce, so each band must equal the separate GEMM of its rows bit for bit."""
    from tritonbench_b200 import dist, quantize

    m, n, k = 65536, 8192, 8192
    wq, ws = quantize.make_quantized(n, k, seed=dist.W_SEED, device="cuda")
    xq, xs = quantize.make_quantized(m, k, seed=dist.shard_seed(0), device="cuda")
    ops = _ops()
    y = ops.fp8_gemm_rowwise(xq, wq, xs, ws)
    ops.check_device_status()
    g = torch.Generator().manual_seed(4)
    rows = torch.cat([band * 8192 + torch.randperm(8192, generator=g)[:64] for band in range(8)])
    rows[0], rows[-1] = 0, m - 1
    rows_d = rows.cuda()
    ref = orc.gemm_rowwise(xq[rows_d].cpu(), wq.cpu(), xs[rows_d].cpu(), ws.cpu(), decode="cast")
    _assert_close(y[rows_d], ref, "M=65536 single launch, row sample")
    for band in (0, 5, 7):
        r0 = band * 8192
        one = ops.fp8_gemm_rowwise(xq[r0:r0 + 8192], wq, xs[r0:r0 + 8192], ws)
        assert torch.equal(y[r0:r0 + 8192], one), f"band {band}"
    ops.check_device_status()


@pytest.mark.parametrize("variant,shape,ranks", [("tc_2cta", (1024, 2048, 1024), 4), ("tc_1cta", (300, 520, 400), 3),
                                                 ("auto", (513, 1000, 256), 8), ("auto", (128, 256, 128), 2)])
def test_gather_fused_gemm_writes_every_copy_of_y(cuda_device, variant, shape, ranks):
    """The fused GEMM + all-gather on one GPU: `ranks` copies of the gathered [ranks*M, N] matrix stand in for the
    other GPUs' buffers.  The rows of 'rank 1' must arrive in every copy, equal to the plain GEMM bit for bit, and
    no other row of any copy may be touched."""
    ops = _ops()
    m, n, k = shape
    xq, wq, xs, ws = _gpu(*_inputs(m, n, k, seed=m + ranks))
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    want = ops.fp8_gemm_rowwise(xq, wq, xs, ws, bias=bias, variant=variant if variant != "auto" else "tc_1cta")
    _assert_close(want, orc.gemm_rowwise(xq.cpu(), wq.cpu(), xs.cpu(), ws.cpu(), bias.cpu()), "plain")
    rank = 1
    copies = [torch.full((ranks * m, n), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(ranks)]
    order = [rank] + [r for r in range(ranks) if r != rank]
    ptrs = [copies[r][rank * m:].data_ptr() for r in order]
    ops.fp8_gemm_rowwise_gather(xq, wq, xs, ws, ptrs, ldy=n, bias=bias, variant=variant)
    ops.check_device_status()
    for r in range(ranks):
        got = copies[r][rank * m:(rank + 1) * m]
        _assert_close(got, want, f"copy {r}")  # the same kernel arithmetic; the variants may differ in the last bit
        assert bool((copies[r][: rank * m] == 7.0).all()) and bool((copies[r][(rank + 1) * m:] == 7.0).all()), f"copy {r}"
    assert all(torch.equal(copies[r][rank * m:(rank + 1) * m], copies[0][rank * m:(rank + 1) * m]) for r in range(ranks))
    with pytest.raises(Exception):
        ops.fp8_gemm_rowwise_gather(xq, wq, xs, ws, ptrs + ptrs + ptrs + ptrs + ptrs, ldy=n)  # more than 8 copies
    with pytest.raises(NotImplementedError):
        ops.fp8_gemm_rowwise_gather(xq, wq, xs, ws, [ptrs[0] + 2], ldy=n)  # rows of Y must be 16-byte aligned


def test_shared_rows_buffer_on_one_rank(cuda_device):
    """The IPC-exportable buffer behaves like any tensor when there is a single rank."""
    from tritonbench_b200 import dist

    ops = _ops()
    m, n, k = 256, 512, 256
    xq, wq, xs, ws = _gpu(*_inputs(m, n, k, seed=5))
    rows = dist.SharedRows(m, n, 1, 0, torch.device("cuda", 0))
    assert tuple(rows.full.shape) == (m, n) and rows.full.dtype == torch.bfloat16 and rows.mine.data_ptr() == rows.full.data_ptr()
    ops.fp8_gemm_rowwise_gather(xq, wq, xs, ws, rows.my_rows_everywhere(), ldy=n)
    ops.check_device_status()
    _assert_close(rows.full, orc.gemm_rowwise(xq.cpu(), wq.cpu(), xs.cpu(), ws.cpu()), "shared rows, one rank")
    rows.close()


def test_plans_for_random_shapes_agree_with_scaled_mm(cuda_device):
    """Whatever the planner picks - pair kernel, wide tiles, K split over clusters, short rings under overlapped
    launches - the result must agree with cuBLASLt's on the same device tensors.  Sixty seeded shapes, with and
    without the overlap flag, ordinary and Student-t inputs."""
    import random

    from tritonbench_b200 import lib, quantize

    ops = _ops()
    rng = random.Random(20240611)
    seen = set()
    for i in range(60):
        m = rng.choice([1, 2, 5, 16, 33, 64, 100, 128, 129, 300, 777, 1000, 1500, 2048, 3000, 4100])
        n = 16 * rng.randint(1, 1400)
        k = 16 * rng.randint(1, 600)
        xq, wq, xs, ws = quantize.make_inputs(m, n, k, device="cuda", x_seed=i, dist="student_t3" if i % 3 == 0 else "normal",
                                              w_std=0.05)
        try:
            want = _scaled_mm_rowwise(xq, wq, xs, ws).float()
        except RuntimeError:
            continue
        tol = orc.bf16_ulp(want) + 1e-2 * want.double().pow(2).mean().sqrt().float()
        for overlap in (False, True):
            flags = lib.FLAG_PDL if overlap else 0
            seen.add(lib.describe_plan(m, n, k, flags).split(" ")[0] + ("+pdl" if overlap else ""))
            y = ops.fp8_gemm_rowwise(xq, wq, xs, ws, overlap=overlap).float()
            assert bool(torch.isfinite(y).all()) and bool(((y - want).abs() <= tol).all()), (m, n, k, overlap, lib.describe_plan(m, n, k, flags))
    ops.check_device_status()
    assert {"tc_2cta", "tc_splitk", "tc_splitk+pdl"} <= seen, seen


# ------------------------------------------------------------------ against the reference's own library call
def _scaled_mm_rowwise(xq, wq, xs, ws):
    """The torch baseline the operator itself names for this GEMM (tritonbench/operators/fp8_gemm_rowwise/
    operator.py:237-246) and the sibling operator runs (tritonbench/operators/fp8_gemm/fp8_gemm.py:88-101):
    cuBLASLt through torch._scaled_mm with one scale per row of X and per row of W."""
    return torch._scaled_mm(xq, wq.t(), scale_a=xs[:, None], scale_b=ws[None, :], use_fast_accum=True,
                            out_dtype=torch.bfloat16)


SCALED_MM_CASES = [
    ("config2", (8192, 8192, 8192), "normal", 1.0),
    ("config3_m1", (1, 28672, 8192), "normal", 0.02),
    ("config3_m16", (16, 28672, 8192), "normal", 0.02),
    ("config3_m64", (64, 28672, 8192), "normal", 0.02),
    ("config3_m128", (128, 28672, 8192), "normal", 0.02),
    ("config5_a", (1000, 5120, 3584), "student_t3", 1.0),
    ("config5_b", (3000, 7168, 2048), "student_t3", 1.0),
    ("config5_c", (4096, 14336, 4096), "student_t3", 1.0),
    ("config5_d", (777, 1024, 8192), "student_t3", 1.0),
]


@pytest.mark.parametrize("case", SCALED_MM_CASES, ids=[c[0] for c in SCALED_MM_CASES])
def test_against_torch_scaled_mm_the_call_the_reference_makes(cuda_device, case):
    """What pins the GEMM to code the reference itself calls: every output of the library against
    torch._scaled_mm with rowwise scales on the same device tensors, whole matrices, benchmark tolerance."""
    from tritonbench_b200 import quantize

    _, (m, n, k), dist_name, w_std = case
    xq, wq, xs, ws = quantize.make_inputs(m, n, k, device="cuda", x_seed=0, dist=dist_name, w_std=w_std)
    ops = _ops()
    try:
        want = _scaled_mm_rowwise(xq, wq, xs, ws)
    except RuntimeError as e:  # a torch build whose cuBLASLt refuses this shape cannot serve as the yardstick
        pytest.skip(f"torch._scaled_mm does not take this shape here: {e}")
    y = ops.fp8_gemm_rowwise(xq, wq, xs, ws)
    ops.check_device_status()
    ref = want.float()
    tol = orc.bf16_ulp(ref) + 1e-2 * ref.double().pow(2).mean().sqrt().float()
    diff = (y.float() - ref).abs()
    assert bool(torch.isfinite(y.float()).all())
    assert bool((diff <= tol).all()), f"{case[0]}: max ratio {float((diff / tol).max()):.3f}"
    if dist_name == "student_t3":  # per row as well: heavy rows must not hide light ones
        row_rms = ref.double().pow(2).mean(dim=1, keepdim=True).sqrt().float()
        assert bool((diff <= orc.bf16_ulp(ref) + 1e-2 * row_rms).all()), f"{case[0]} per-row bound"
    # the CPU oracle itself against the same reference-called output (64 sampled rows): this is what ties the
    # checker every other test uses to code the reference runs
    rows = torch.randperm(m, generator=torch.Generator().manual_seed(11))[: min(m, 64)].sort().values
    rows_d = rows.cuda()
    oracle_rows = orc.gemm_rowwise(xq[rows_d].cpu(), wq.cpu(), xs[rows_d].cpu(), ws.cpu(), decode="cast")
    res = orc.compare(oracle_rows, want[rows_d])
    assert res["ok"], f"{case[0]}: oracle vs torch._scaled_mm {res}"


def test_reference_builtin_decode_shapes(cuda_device, golden_dir):
    shapes = np.load(os.path.join(golden_dir, "ref_builtin_shapes.npz"))["shapes"]
    for (m, n, k) in shapes:
        if m > 128:
            continue
        xq, wq, xs, ws = _inputs(int(m), int(n), int(k), seed=int(m))
        _assert_close(_run("auto", xq, wq, xs, ws), orc.gemm_rowwise(xq, wq, xs, ws), f"builtin {(m, n, k)}")


# ------------------------------------------------------------------ options and edge cases
@pytest.mark.parametrize("variant,shape", [("tc_1cta", (300, 520, 400)), ("tc_2cta", (513, 1001, 256)), ("skinny", (17, 520, 400)), ("simt", (50, 70, 90))])
def test_bias(cuda_device, variant, shape):
    m, n, k = shape
    xq, wq, xs, ws = _inputs(m, n, k, seed=3)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(4)) * 30).to(torch.bfloat16)
    _assert_close(_run(variant, xq, wq, xs, ws, bias=bias), orc.gemm_rowwise(xq, wq, xs, ws, bias), f"{variant} bias")


def test_unaligned_k_falls_to_cuda_core_kernel_and_forced_variants_refuse(cuda_device):
    m, n, k = 70, 90, 130  # rows of 130 bytes cannot start on 16-byte boundaries
    xq, wq, xs, ws = _inputs(m, n, k, seed=8)
    _assert_close(_run("auto", xq, wq, xs, ws), orc.gemm_rowwise(xq, wq, xs, ws), "auto -> simt")
    for variant in TC_VARIANTS + ("skinny",):
        with pytest.raises(NotImplementedError):
            _run(variant, xq, wq, xs, ws)


def test_row_pitch_larger_than_k_and_strided_output(cuda_device):
    ops = _ops()
    m, n, k = 260, 520, 384
    xq, wq, xs, ws = _inputs(m, n, k, seed=2)
    ref = orc.gemm_rowwise(xq, wq, xs, ws)
    big_x = torch.zeros((m, k + 128), dtype=torch.uint8, device="cuda")
    big_w = torch.zeros((n, k + 256), dtype=torch.uint8, device="cuda")
    big_x[:, :k] = xq.view(torch.uint8).cuda()
    big_w[:, :k] = wq.view(torch.uint8).cuda()
    out_big = torch.zeros((m, n + 8), dtype=torch.bfloat16, device="cuda")
    for variant in TC_VARIANTS:
        out_big.zero_()
        y = ops.fp8_gemm_rowwise(big_x[:, :k], big_w[:, :k], xs.cuda(), ws.cuda(), out=out_big[:, :n], variant=variant)
        _assert_close(y, ref, f"{variant} pitched")
        assert float(out_big[:, n:].abs().max()) == 0.0  # nothing written past N
    ops.check_device_status()


def test_extreme_scales_and_zero_rows(cuda_device):
    m, n, k = 130, 264, 256
    xq, wq, xs, ws = _inputs(m, n, k, seed=6)
    xq = xq.clone()
    xq.view(torch.uint8)[5] = 0
    xs = xs.clone()
    xs[5] = 1e-12 / 448.0
    xs[6] = 3.0e4
    ws = ws.clone()
    ws[9] = 1e-20
    ref = orc.gemm_rowwise(xq, wq, xs, ws)
    for variant in TC_VARIANTS + ("simt",):
        y = _run(variant, xq, wq, xs, ws)
        _assert_close(y, ref, f"{variant} extreme scales")
        assert float(y[5].abs().max()) == 0.0


def test_saturated_operands_all_448(cuda_device):
    m, n, k = 128, 256, 4096
    xq = torch.full((m, k), 0x7E, dtype=torch.uint8).view(torch.float8_e4m3fn)
    wq = torch.full((n, k), 0xFE, dtype=torch.uint8).view(torch.float8_e4m3fn)
    xs = torch.ones(m)
    ws = torch.ones(n)
    ref = orc.gemm_rowwise(xq, wq, xs, ws)
    assert float(ref[0, 0]) == float(torch.tensor(-448.0 * 448.0 * k).to(torch.bfloat16))
    for variant in TC_VARIANTS + ("skinny",):
        assert torch.equal(_run(variant, xq, wq, xs, ws).cpu(), ref)


def test_status_codes_for_bad_calls(cuda_device):
    from tritonbench_b200 import lib

    ops = _ops()
    xq, wq, xs, ws = _gpu(*_inputs(16, 1024, 1024))
    tiny = torch.zeros(256, dtype=torch.uint8, device="cuda")
    with pytest.raises(lib.B200Fp8Error) as e:
        ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant="skinny", workspace=tiny)
    assert e.value.status == lib.WORKSPACE_TOO_SMALL
    x2, w2, xs2, ws2 = _gpu(*_inputs(200, 256, 256))
    with pytest.raises(ValueError):
        ops.workspace_bytes(200, 256, 256, lib.VARIANT_SKINNY)
    with pytest.raises(ValueError):
        ops.fp8_gemm_rowwise(x2, w2, xs2[:10], ws2)
    with pytest.raises(ValueError):
        ops.fp8_gemm_rowwise(x2.cpu(), w2, xs2, ws2)


def test_call_is_capturable_in_a_cuda_graph(cuda_device):
    """The reference times this operator by CUDA-graph replay; the call must allocate nothing and
    never synchronise.  Captured and replayed results equal the eager ones bit for bit."""
    ops = _ops()
    for variant, shape, overlap in (("tc_2cta", (512, 1024, 1024), False), ("tc_1cta", (300, 520, 400), False),
                                    ("skinny", (16, 4096, 2048), False), ("skinny", (16, 28672, 8192), True)):
        xq, wq, xs, ws = _gpu(*_inputs(*shape, seed=1))
        fn = ops.make_gemm_fn(xq, wq, xs, ws, variant=variant, reuse_out=True)
        eager = fn().clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn_side = ops.make_gemm_fn(xq, wq, xs, ws, variant=variant, reuse_out=True, overlap=overlap)
            fn_side()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(3 if overlap else 1):
                    out = fn_side()
        out.zero_()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager), variant
    ops.check_device_status()


@pytest.mark.parametrize("variant", ["auto", "tc_splitk", "skinny"])
def test_overlapped_launch_of_decode_kernels_back_to_back(cuda_device, variant):
    """B200FP8_FLAG_PDL: each kernel may start while the one before it still runs and reads only W that
    early.  A chain of decode GEMMs of different shapes, sharing one workspace and launched without any
    host synchronisation in between, must give the same bits as the ordinary launches."""
    ops = _ops()
    from tritonbench_b200 import lib
    shapes = [(16, 28672, 8192), (1, 4096, 2304), (16, 28672, 8192), (64, 4096, 2048), (8, 2304, 2304), (128, 2304, 6656)]
    cases = []
    for i, (m, n, k) in enumerate(shapes):
        xq, wq, xs, ws = _gpu(*_inputs(m, n, k, seed=20 + i, w_std=0.02))
        cases.append((xq, wq, xs, ws, ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant=variant)))
    ws_bytes = max(ops.workspace_bytes(m, n, k, lib.VARIANTS[variant]) for (m, n, k) in shapes)
    workspace = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    for rep in range(3):
        outs = [ops.fp8_gemm_rowwise(xq, wq, xs, ws, variant=variant, workspace=workspace, overlap=True)
                for (xq, wq, xs, ws, _) in cases]
        torch.cuda.synchronize()
        for out, case in zip(outs, cases):
            assert torch.equal(out, case[4]), f"rep {rep}"
    # a writer of X directly in front of the GEMM: X is read only after the writer has completed
    xq, wq, xs, ws, want = cases[0]
    x_bytes = xq.view(torch.uint8).clone()
    for rep in range(3):
        scratch = torch.zeros_like(x_bytes)
        scratch.copy_(x_bytes)  # the copy kernel is the immediate predecessor on the stream
        got = ops.fp8_gemm_rowwise(scratch.view(torch.float8_e4m3fn), wq, xs, ws, variant=variant, overlap=True)
        assert torch.equal(got, want)
    ops.check_device_status()


@pytest.mark.parametrize("producer", ["row_quantize", "rms_norm", "silu_mul"])
def test_decode_gemm_launched_behind_a_quantiser_of_x_starts_early_and_still_sees_its_output(cuda_device, producer):
    """The producer + quantiser kernels let a dependent launch start while they run (the plain row quantiser does not:
    it also serves weights).  A decode GEMM with the overlap flag directly behind a quantiser of X may prefetch W early
    but must read xq and x_scale only after the quantiser has completed:
    every iteration quantises a different activation into the same buffers, so a GEMM that read early would return the
    previous iteration's result."""
    ops = _ops()
    n, k = 2048, 4096
    gen = torch.Generator().manual_seed(77)
    w = (torch.randn(n, k, generator=gen) * 0.05).to(torch.bfloat16).cuda()
    wq, ws = ops.fp8_row_quantize(w)
    wd = torch.randn(k, generator=gen).to(torch.bfloat16).cuda()
    torch.cuda.synchronize()
    for m in (1, 16, 128):
        xs_in = [(torch.randn(m, k, generator=gen) * (1 + i)).to(torch.bfloat16).cuda() for i in range(4)]
        x2 = torch.randn(m, k, generator=gen).to(torch.bfloat16).cuda()

        def quantise(x):
            if producer == "row_quantize":
                return ops.fp8_row_quantize(x)
            if producer == "rms_norm":
                return ops.rms_norm_fp8_rowwise_quant(x, wd)
            return ops.silu_mul_fp8_rowwise_quant(x, x2)

        want = []
        for x in xs_in:  # ordinary launches, a synchronisation between the two kernels
            xq, xs = quantise(x)
            torch.cuda.synchronize()
            want.append(ops.fp8_gemm_rowwise(xq, wq, xs, ws).clone())
        torch.cuda.synchronize()
        for rep in range(12):
            x = xs_in[rep % 4]
            xq, xs = quantise(x)
            got = ops.fp8_gemm_rowwise(xq, wq, xs, ws, overlap=True)
            assert torch.equal(got, want[rep % 4]), (producer, m, rep)
            del xq, xs  # the next iteration's quantiser gets the same memory back from the caching allocator
    ops.check_device_status()


@pytest.mark.parametrize("variant,shape", [("tc_1cta", (300, 520, 400)), ("tc_2cta", (513, 1001, 256)), ("tc_2cta", (512, 1024, 1024)),
                                           ("skinny", (17, 520, 400)), ("skinny", (16, 4096, 2048)), ("simt", (50, 70, 90))])
def test_fp16_output(cuda_device, variant, shape):
    m, n, k = shape
    xq, wq, xs, ws = _inputs(m, n, k, seed=13)
    ref = orc.gemm_rowwise(xq, wq, xs, ws, out_dtype=torch.float16)
    y = _run(variant, xq, wq, xs, ws, out_dtype=torch.float16)
    assert y.dtype == torch.float16
    _assert_close(y, ref, f"{variant} fp16 out")
    y2 = _run(variant, xq, wq, xs, ws, out_dtype=torch.float16, tma_store=False)
    _assert_close(y2, ref, f"{variant} fp16 out, plain stores")


def test_fp8_gemm_call_with_per_tensor_and_unit_scales(cuda_device):
    """The sibling operator's call: a [M,K], b [K,N] column-major, per-tensor scales, fp16 out by default."""
    ops = _ops()
    g = torch.Generator().manual_seed(21)
    m, n, k = 384, 768, 1024
    a = torch.randn((m, k), generator=g).to(torch.float8_e4m3fn)
    b = torch.randn((k, n), generator=g).to(torch.float8_e4m3fn).T.contiguous().T  # the operator's own layout
    ones_m, ones_n = torch.ones(m), torch.ones(n)
    y = ops.fp8_gemm(a.cuda(), b.cuda())
    ops.check_device_status()
    assert y.dtype == torch.float16
    _assert_close(y, orc.gemm_rowwise(a, b.T, ones_m, ones_n, out_dtype=torch.float16), "fp8_gemm unit scales")
    y = ops.fp8_gemm(a.cuda(), b.cuda(), 0.5, torch.tensor(0.25), out_dtype=torch.bfloat16)
    _assert_close(y, orc.gemm_rowwise(a, b.T, ones_m * 0.5, ones_n * 0.25), "fp8_gemm per-tensor scales")
    y = ops.fp8_gemm(a.cuda(), b.cuda(), torch.full((m, 1), 2.0).cuda(), torch.full((1, n), 0.5).cuda(), out_dtype=torch.bfloat16)
    _assert_close(y, orc.gemm_rowwise(a, b.T, ones_m * 2.0, ones_n * 0.5), "fp8_gemm rowwise scales")
    with pytest.raises(ValueError):
        ops.fp8_gemm(a.cuda(), b.cuda().contiguous())


GROUPED_CASES = [
    # (m_sizes, N, K)
    ([512, 512], 1024, 1024),
    ([256, 256, 256, 256], 1024, 1024),
    ([100, 0, 333, 1, 130], 520, 400),     # ragged, an empty group, a one-row group, tails everywhere
    ([129, 127, 31, 33], 264, 144),
    ([2048, 2048, 2048, 2048], 4096, 4096),  # the operator's (8192, 4096, 4096) shape with 4 groups
]


@pytest.mark.parametrize("variant", ["auto", "tc_1cta", "tc_2cta"])
@pytest.mark.parametrize("case", GROUPED_CASES)
def test_grouped_gemm(cuda_device, case, variant):
    ops = _ops()
    sizes, n, k = case
    groups, m_total = len(sizes), sum(sizes)
    from tritonbench_b200 import quantize

    xq, xs = quantize.make_quantized(m_total, k, seed=31)
    wq, ws = quantize.make_quantized(groups * n, k, seed=32, std=0.05)
    m_sizes = torch.tensor(sizes, dtype=torch.int32)
    ref = orc.gemm_rowwise_grouped(xq, wq, m_sizes, xs, ws)
    y = ops.fp8_gemm_rowwise_grouped(*_gpu(xq, wq, m_sizes, xs, ws), variant=variant)
    ops.check_device_status()
    _assert_close(y, ref, f"grouped {case} {variant}")
    # no group may write into its neighbour's rows: equal to the per-group plain GEMMs bit for bit
    r0 = 0
    for g, rows in enumerate(sizes):
        if rows:
            one = ops.fp8_gemm_rowwise(*_gpu(xq[r0:r0 + rows], wq[g * n:(g + 1) * n], xs[r0:r0 + rows], ws[g * n:(g + 1) * n]),
                                       variant="tc_1cta")
            assert torch.equal(y[r0:r0 + rows], one), f"group {g}"
        r0 += rows


def test_grouped_gemm_leaves_rows_beyond_the_groups_untouched(cuda_device):
    ops = _ops()
    from tritonbench_b200 import quantize

    xq, xs = quantize.make_quantized(300, 256, seed=1)
    wq, ws = quantize.make_quantized(2 * 264, 256, seed=2)
    m_sizes = torch.tensor([100, 120], dtype=torch.int32)
    out = torch.full((300, 264), 7.0, dtype=torch.bfloat16, device="cuda")
    y = ops.fp8_gemm_rowwise_grouped(*_gpu(xq, wq, m_sizes, xs, ws), out=out)
    ref = orc.gemm_rowwise_grouped(xq, wq, m_sizes, xs, ws)
    _assert_close(y[:220], ref[:220], "grouped prefix")
    assert bool((y[220:] == 7.0).all())


def test_a_wait_that_runs_out_becomes_a_status_code_not_a_hang(cuda_device):
    """Failure detection without a fault: a CTA waits 2 ms on a barrier that nothing sets; the wait gives up,
    the kernel ends normally, the host reads DEVICE_TIMEOUT, and the GPU context is still good for the next GEMM."""
    import ctypes
    import time

    from tritonbench_b200 import lib

    ops = _ops()
    cdll = lib.load()
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    t0 = time.perf_counter()
    assert cdll.b200fp8_selftest_wait_timeout(ws.data_ptr(), 2000, torch.cuda.current_stream().cuda_stream) == lib.OK
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    word = ctypes.c_uint32(0)
    assert cdll.b200fp8_query_status(ws.data_ptr(), ctypes.byref(word)) == lib.DEVICE_TIMEOUT
    assert word.value >> 24 == 1 and (word.value & 0xFFFFFF) == 0x7E57
    with pytest.raises(lib.B200Fp8Error) as e:
        lib.check(lib.DEVICE_TIMEOUT, "selftest")
    assert e.value.status == lib.DEVICE_TIMEOUT
    ws.zero_()
    assert cdll.b200fp8_query_status(ws.data_ptr(), ctypes.byref(word)) == lib.OK
    xq, wq, xs, wsc = _inputs(128, 256, 512)
    _assert_close(_run("auto", xq, wq, xs, wsc), orc.gemm_rowwise(xq, wq, xs, wsc), "GEMM after the self-test")
    assert cdll.b200fp8_selftest_wait_timeout(ws.data_ptr(), 0, None) == lib.BAD_ARG


BLOCKWISE_SHAPES = [(128, 256, 128), (128, 256, 512), (200, 300, 400), (777, 1024, 2048), (1, 2304, 2048), (64, 4096, 2048),
                    (2048, 8192, 2048), (513, 1001, 1040), (4096, 2304, 4096)]


@pytest.mark.parametrize("shape", BLOCKWISE_SHAPES)
def test_block_scaled_gemm(cuda_device, shape):
    """128x128 block scales: per-k-block promotion in the kernel against dequantise-then-matmul in the oracle."""
    ops = _ops()
    from tritonbench_b200 import quantize

    m, n, k = shape
    g = torch.Generator().manual_seed(m + n)
    x = (torch.randn((m, k), generator=g) * (1 + 10 * torch.rand((m, 1), generator=g))).to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g) * 0.05).to(torch.bfloat16)
    xq, xs = quantize.fp8_block_quantize(x)
    wq, ws = quantize.fp8_block_quantize(w)
    ref = orc.gemm_blockwise(xq, wq, xs, ws)
    y = ops.fp8_gemm_blockwise(*_gpu(xq, wq, xs, ws))
    ops.check_device_status()
    _assert_close(y, ref, f"blockwise {shape}")
    assert torch.equal(ops.fp8_gemm_blockwise(*_gpu(xq, wq, xs, ws)), y)
    if n % 8 == 0:
        _assert_close(ops.fp8_gemm_blockwise(*_gpu(xq, wq, xs, ws), tma_store=False), ref, f"blockwise {shape} plain stores")


def test_host_buffer_entry_point(cuda_device):
    ops = _ops()
    for variant, shape in (("auto", (384, 768, 512)), ("auto", (16, 2304, 2048))):
        m, n, k = shape
        xq, wq, xs, ws = _inputs(m, n, k, seed=12)
        bias = torch.randn(n).to(torch.bfloat16)
        hg = ops.HostGemm(m, n, k, variant=variant)
        pinned = [t.contiguous().pin_memory() for t in (xq.view(torch.uint8), wq.view(torch.uint8), xs, ws)]
        y = hg(*pinned)
        _assert_close(y, orc.gemm_rowwise(xq, wq, xs, ws), f"host {shape}")
        yb = hg(*pinned, bias=bias.pin_memory())
        _assert_close(yb, orc.gemm_rowwise(xq, wq, xs, ws, bias), f"host bias {shape}")
        hg.close()


@pytest.mark.parametrize("shape,panels", [((2597, 1032, 640), None), ((2597, 1032, 640), (512, 256)), ((8192, 2048, 1024), None),
                                          ((4096 + 1, 520, 400), None), ((2100, 4352, 1536), None), ((300, 4096 + 8, 2048), (128, 1024))])
def test_host_buffer_entry_point_panel_pipeline(cuda_device, shape, panels):
    """Larger problems flow through the host-buffer call in panels over three streams (the form the end-to-end
    benchmark number is measured on): panels of X and of W uploaded alternately, every newly computable strip of Y
    multiplied and downloaded at once.  Several panels in both dimensions, ragged last panels (37 rows, one row,
    8 columns), bias on and off, pageable as well as pinned host memory, and the weights kept on the device."""
    ops = _ops()
    m, n, k = shape
    xq, wq, xs, ws = _inputs(m, n, k, seed=m)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(2)) * 20).to(torch.bfloat16)
    ref = orc.gemm_rowwise(xq, wq, xs, ws, decode="cast")
    ref_bias = orc.gemm_rowwise(xq, wq, xs, ws, bias, decode="cast")
    hg = ops.HostGemm(m, n, k, panels=panels)
    host = [t.contiguous() for t in (xq.view(torch.uint8), wq.view(torch.uint8), xs, ws)]
    pinned = [t.pin_memory() for t in host]
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16).pin_memory()
    y = hg(*pinned, out=out)
    assert y.data_ptr() == out.data_ptr()
    _assert_close(y, ref, f"host panels {shape}")
    _assert_close(hg(*pinned, bias=bias.pin_memory()), ref_bias, f"host panels {shape} bias")
    # W, w_scale and bias of the last upload stay on the device: wq=None sends X only
    out.fill_(float("nan"))
    _assert_close(hg(pinned[0], None, pinned[2], None, out=out), ref_bias, f"host panels {shape} resident weights + bias")
    hg.set_weights(pinned[1], pinned[3])
    out.fill_(float("nan"))
    _assert_close(hg(pinned[0], None, pinned[2], None, out=out), ref, f"host panels {shape} resident weights")
    out.fill_(float("nan"))
    _assert_close(hg(*host, out=out), ref, f"host panels {shape} pageable inputs")
    hg.set_weights(None, None)
    with pytest.raises(Exception):
        hg(pinned[0], None, pinned[2], None)
    # and against the device entry point on the whole problem (the blocks may be planned differently)
    _assert_close(out, ops.fp8_gemm_rowwise(*_gpu(xq, wq, xs, ws)).cpu(), f"host panels {shape} vs device call")
    hg.close()

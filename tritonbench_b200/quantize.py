"""Input side of the operator: rowwise e4m3 quantisation and the seeded synthetic inputs of the
benchmark configurations (input generation is untimed set-up in the reference as well:
tritonbench/operators/fp8_gemm_rowwise/operator.py:280-297).  CUDA tensors go through the library's
fused quantiser kernel (b200fp8_row_quantize); CPU tensors - fixtures, tests, the CPU benchmark legs -
through the torch expressions below, which produce the same bits.
"""
from typing import Optional, Tuple

import torch

E4M3_MAX = 448.0
EPS = 1e-12


def fp8_row_quantize(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same contract as the reference's `fp8_row_quantize` (operator.py:136-145): multiplier
    448 / clamp(rowmax, 1e-12) in x's dtype, clamp, cast to float8_e4m3fn, return (xq, 1/multiplier
    as float32)."""
    if x.is_cuda:
        from . import ops

        return ops.fp8_row_quantize(x, recipe="operator")  # one fused kernel, same bits
    row_max = x.abs().amax(dim=1)
    mult = E4M3_MAX / row_max.clamp(min=EPS)
    if x.dtype is torch.float16:
        mult = mult.clamp(max=torch.finfo(torch.float16).max)
    xq = (x * mult[:, None]).clamp(min=-E4M3_MAX, max=E4M3_MAX).to(torch.float8_e4m3fn)
    return xq, mult.reciprocal().to(torch.float32)


def fp8_row_quantize_fp32(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Benchmark recipe: scale = max(rowabsmax, 1e-12) / 448 in fp32; xq = e4m3(clamp(x / scale))."""
    x = x.to(torch.float32)
    if x.is_cuda:
        from . import ops

        return ops.fp8_row_quantize(x, recipe="fp32")
    scale = x.abs().amax(dim=1).clamp(min=EPS) / E4M3_MAX
    xq = (x / scale[:, None]).clamp(min=-E4M3_MAX, max=E4M3_MAX).to(torch.float8_e4m3fn)
    return xq, scale


def fp8_block_quantize(x: torch.Tensor, block_m: int = 128, block_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same contract as the reference's `fp8_block_quantize` (tritonbench/operators/fp8_gemm_blockwise/operator.py:87-120):
    one multiplier 448 / blockmax per block_m x block_k block (1.0 where that is infinite), no clamp before the
    e4m3 cast, returns (xq, 1 / multiplier as float32 [ceil(M/block_m), ceil(K/block_k)])."""
    if x.is_cuda and block_m == 128 and block_k == 128:
        from . import ops

        return ops.fp8_block_quantize(x)
    m, k = x.shape
    grid_m, grid_k = -(-m // block_m), -(-k // block_k)
    padded = torch.zeros(grid_m * block_m, grid_k * block_k, dtype=x.dtype, device=x.device)
    padded[:m, :k] = x
    block_max = padded.abs().reshape(grid_m, block_m, grid_k, block_k).amax(dim=(1, 3)).clamp(min=EPS)
    mult = E4M3_MAX / block_max.to(torch.float32)
    mult[mult == float("inf")] = 1.0
    xq = (padded * mult.repeat_interleave(block_m, dim=0).repeat_interleave(block_k, dim=1))[:m, :k]
    return xq.to(torch.float8_e4m3fn), 1 / mult


def _draw(rows: int, cols: int, dist: str, std: float, gen: torch.Generator, device) -> torch.Tensor:
    """Seeded fp32 draw, chunked by rows so that large matrices never hold more than ~1 GiB of fp32."""
    if dist == "normal":
        return torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * std
    if dist == "student_t3":
        # t(3) = z / sqrt(chi2_3 / 3) with chi2_3 the sum of three squared normals
        z = torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32)
        c = torch.randn((3, rows, cols), generator=gen, device=device, dtype=torch.float32).pow(2).sum(0)
        return z / (c / 3.0).sqrt() * std
    raise ValueError(f"unknown distribution {dist!r}")


def make_quantized(
    rows: int,
    cols: int,
    seed: int,
    device="cpu",
    dist: str = "normal",
    std: float = 1.0,
    chunk_rows: int = 8192,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Seeded [rows, cols] draw -> (e4m3 tensor, fp32 scale per row), generated in row chunks."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=device)
    s = torch.empty((rows,), dtype=torch.float32, device=device)
    for r0 in range(0, rows, chunk_rows):
        r1 = min(rows, r0 + chunk_rows)
        qc, sc = fp8_row_quantize_fp32(_draw(r1 - r0, cols, dist, std, gen, device))
        q[r0:r1] = qc
        s[r0:r1] = sc
    return q, s


def make_inputs(
    m: int,
    n: int,
    k: int,
    device="cpu",
    x_seed: int = 0,
    w_seed: Optional[int] = None,
    dist: str = "normal",
    x_std: float = 1.0,
    w_std: float = 1.0,
):
    """(xq, wq, x_scale, w_scale) for one benchmark shape.  With w_seed None, X then W come from one
    generator seeded x_seed (the single-GPU configurations); with w_seed given they are independent
    streams (the M-sharded configuration: W from a common seed on every rank, X from a per-shard seed)."""
    device = torch.device(device)
    if w_seed is None:
        gen = torch.Generator(device=device)
        gen.manual_seed(x_seed)
        if m * k <= (1 << 28) and n * k <= (1 << 28):
            xq, xs = fp8_row_quantize_fp32(_draw(m, k, dist, x_std, gen, device))
            wq, ws = fp8_row_quantize_fp32(_draw(n, k, dist, w_std, gen, device))
            return xq, wq, xs, ws
        w_seed = x_seed + 1_000_003
    xq, xs = make_quantized(m, k, x_seed, device, dist, x_std)
    wq, ws = make_quantized(n, k, w_seed, device, dist, w_std)
    return xq, wq, xs, ws

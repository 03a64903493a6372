"""CPU oracle for the FP8 rowwise-scaled GEMM path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference legs may import this
module, and only as the checker or the timed CPU baseline.  Nothing under tritonbench_b200/ uses it.

PARITY at the kernel boundary.  The arithmetic of the reference's backends lives in the third-party package
fbgemm_gpu (git submodule submodules/FBGEMM of the reference, .gitmodules:1-3, an empty directory in the mounted
tree with no recorded commit; not installed), and the reference's own tests skip this operator wholesale
(test/test_gpu/skip_tests_h100_pytorch.yaml:17-18), so the reference holds no golden vectors for the GEMM.  What
pins this oracle:
  * the GEMM (`gemm_rowwise`): on a GPU, against the output of the call the reference itself names as the operator's
    torch baseline and runs in the sibling operator - `torch._scaled_mm` with rowwise scales
    (tritonbench/operators/fp8_gemm_rowwise/operator.py:237-246, tritonbench/operators/fp8_gemm/fp8_gemm.py:88-101) -
    on every benchmark configuration (tests/test_gemm_gpu.py::test_against_torch_scaled_mm_the_call_the_reference_makes).
    That call runs on CUDA only (on CPU it rejects rowwise scales), so without a GPU the GEMM oracle is checked
    against the stored fixtures and its plain-C twin only: in a CPU-only run its parity is UNPINNED;
  * the row quantiser and the block quantiser: against the reference's own `fp8_row_quantize` and
    `fp8_block_quantize`, imported from the reference tree by tests/golden/make_golden.py (outputs committed as
    fixtures, rows with NaN and infinity included);
  * the e4m3 decode table: against torch.float8_e4m3fn for all 256 byte values.

What this restates:
  * `row_quantize_reference`  follows tritonbench/operators/fp8_gemm_rowwise/operator.py:130-145
  * `row_quantize`            the benchmark recipe: scale = max(rowabsmax, 1e-12) / 448 in fp32
  * `gemm_rowwise`            the fp32 dequantise-then-matmul torch form the operator keeps as its
                              (commented) torch baseline, operator.py:237-246, with the scales applied
                              to the operands in fp32 before the product, and the stock shims' bias
                              add (operator.py:207-213) done in fp32 before the single bf16 rounding
  * `flops`, `gbytes`         operator.py:248-271
  * `gemm_rowwise(out_dtype=float16)` with all-ones scales is the sibling operator `fp8_gemm`'s
    `torch._scaled_mm(a, b, 1.0, 1.0, out_dtype=float16)` (tritonbench/operators/fp8_gemm/fp8_gemm.py:88-101)
"""
import math
from typing import Optional, Tuple

import numpy as np
import torch

E4M3_MAX = 448.0
EPS = 1e-12


def e4m3_decode_table() -> np.ndarray:
    """float32 value of each of the 256 e4m3fn byte patterns, from the format definition:
    1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinities; S.1111.111 is NaN."""
    out = np.zeros(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = math.nan
        elif e == 0:
            v = sign * (m / 8.0) * 2.0 ** (-6)
        else:
            v = sign * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        out[b] = v
    return out


_TABLE = None


def decode_e4m3(q: torch.Tensor) -> torch.Tensor:
    """e4m3 bytes (float8_e4m3fn or uint8 tensor) -> float32 through the table above."""
    global _TABLE
    if _TABLE is None:
        _TABLE = torch.from_numpy(e4m3_decode_table())
    idx = q.view(torch.uint8).to(torch.int64)
    return _TABLE[idx]


def row_quantize_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """operator.py:136-145 — arithmetic in x's own dtype (bf16 in the reference's generator),
    multiplier 448 / clamp(rowmax, 1e-12), fp16 inputs clamp the multiplier to 65504, clamp to
    +-448, cast to e4m3 (round to nearest even), return the reciprocal multiplier as fp32."""
    row_max = torch.max(torch.abs(x), dim=1).values
    scale = E4M3_MAX / torch.clamp(row_max, EPS)
    if x.dtype is torch.float16:
        scale = torch.clamp(scale, max=torch.finfo(torch.float16).max)
    xq = torch.clamp(x * scale[:, None], min=-E4M3_MAX, max=E4M3_MAX).to(torch.float8_e4m3fn)
    return xq, scale.reciprocal().to(torch.float32)


def row_quantize(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Benchmark recipe: fp32 input, scale = max(rowabsmax, 1e-12) / 448 (fp32), q = e4m3(clamp(x / scale))."""
    x = x.to(torch.float32)
    scale = torch.clamp(x.abs().amax(dim=1), min=EPS) / E4M3_MAX
    xq = torch.clamp(x / scale[:, None], min=-E4M3_MAX, max=E4M3_MAX).to(torch.float8_e4m3fn)
    return xq, scale


def rms_norm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, round_bf16: bool = False) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * weight in fp32 on bf16 inputs: the producer of `rms_norm_fused` /
    `rms_norm_quant` (tritonbench/operators/fp8_fused_quant_gemm_rowwise/operator.py:86-107).  The producer
    kernels themselves are Meta-internal and absent from the reference tree: eps and the fp32 arithmetic are
    this build's definition, and parity for them is unpinned."""
    xf = x.to(torch.float32)
    inv = 1.0 / torch.sqrt(xf.pow(2).mean(dim=1, keepdim=True) + eps)
    y = (xf * inv) * weight.to(torch.float32)[None, :]
    return y.to(torch.bfloat16).to(torch.float32) if round_bf16 else y


def silu_mul_rows(x1: torch.Tensor, x2: torch.Tensor, round_bf16: bool = False) -> torch.Tensor:
    """y = x1 / (1 + exp(-x1)) * x2 in fp32 on bf16 inputs (`silu_mul_fused` / `silu_mul_quant`,
    tritonbench/operators/fp8_fused_quant_gemm_rowwise/operator.py:109-131); parity unpinned, as above."""
    a = x1.to(torch.float32)
    y = a / (1.0 + torch.exp(-a)) * x2.to(torch.float32)
    return y.to(torch.bfloat16).to(torch.float32) if round_bf16 else y


def gemm_rowwise(
    xq: torch.Tensor,
    wq: torch.Tensor,
    x_scale: torch.Tensor,
    w_scale: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    keep_fp32: bool = False,
    decode: str = "table",
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Y = bf16((float(xq) * x_scale[:, None]) @ (float(wq) * w_scale[:, None]).T (+ bias)) on CPU in fp32.

    decode="table" reads the operands through this module's own e4m3 table (the checker's default);
    decode="cast" uses torch's float8_e4m3fn -> float32 cast, i.e. literally `X.float()`, the form the
    benchmark specification times on the host cores.  The two are identical for all 256 byte values
    (tests/test_oracle.py), "cast" is several times faster on large operands."""
    if decode == "cast":
        x = xq.cpu().view(torch.float8_e4m3fn).to(torch.float32) * x_scale.cpu().to(torch.float32)[:, None]
        w = wq.cpu().view(torch.float8_e4m3fn).to(torch.float32) * w_scale.cpu().to(torch.float32)[:, None]
    else:
        x = decode_e4m3(xq.cpu()) * x_scale.cpu().to(torch.float32)[:, None]
        w = decode_e4m3(wq.cpu()) * w_scale.cpu().to(torch.float32)[:, None]
    y = x @ w.T
    if bias is not None:
        y = y + bias.cpu().to(torch.float32)[None, :]
    return y if keep_fp32 else y.to(out_dtype)


def gemm_rowwise_grouped(xq, wq, m_sizes, x_scale, w_scale) -> torch.Tensor:
    """Grouped form (tritonbench/operators/fp8_gemm_rowwise_grouped/operator.py:412-470, 547-580): rows of
    xq [M_total, K] split in order into groups of m_sizes[g] rows; group g uses rows [g*N, (g+1)*N) of the stacked
    wq [G*N, K].  Plain loop over the groups with `gemm_rowwise`; rows past the groups stay zero."""
    sizes = [int(v) for v in m_sizes.cpu().tolist()]
    groups = len(sizes)
    n = wq.shape[0] // groups
    y = torch.zeros((xq.shape[0], n), dtype=torch.bfloat16)
    r0 = 0
    for g, rows in enumerate(sizes):
        if rows > 0:
            y[r0 : r0 + rows] = gemm_rowwise(
                xq[r0 : r0 + rows], wq[g * n : (g + 1) * n], x_scale[r0 : r0 + rows], w_scale[g * n : (g + 1) * n]
            )
        r0 += rows
    return y


def block_quantize_reference(x: torch.Tensor, block_m: int = 128, block_k: int = 128):
    """tritonbench/operators/fp8_gemm_blockwise/operator.py:87-120: per 128x128 block, multiplier 448 / blockmax
    (blockmax clamped to 1e-12 in x's dtype, the division in fp32, infinite multipliers replaced by 1), the scaled
    values cast to e4m3 without a clamp; returns (xq, reciprocal multipliers [grid_m, grid_k] fp32)."""
    m, k = x.shape
    grid_m, grid_k = -(-m // block_m), -(-k // block_k)
    padded = torch.zeros(grid_m * block_m, grid_k * block_k, dtype=x.dtype)
    padded[:m, :k] = x
    block_max = torch.clamp(padded.abs().reshape(grid_m, block_m, grid_k, block_k).amax(dim=(1, 3)), min=EPS)
    scale = E4M3_MAX / block_max.to(torch.float32)
    scale[scale == float("inf")] = 1.0
    xq = (padded * scale.repeat_interleave(block_m, dim=0).repeat_interleave(block_k, dim=1))[:m, :k]
    return xq.to(torch.float8_e4m3fn), 1 / scale


def gemm_blockwise(xq, wq, x_scale, w_scale, keep_fp32: bool = False) -> torch.Tensor:
    """Block-scaled GEMM (operator.py:139-149 call sites): operands dequantised with their 128x128 block scales
    in fp32, fp32 matmul, bf16 result."""
    m, k = xq.shape
    n = wq.shape[0]
    xs = x_scale.cpu().to(torch.float32).repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)[:m, :k]
    ws = w_scale.cpu().to(torch.float32).repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)[:n, :k]
    y = (decode_e4m3(xq.cpu()) * xs) @ (decode_e4m3(wq.cpu()) * ws).T
    return y if keep_fp32 else y.to(torch.bfloat16)


def bf16_ulp(v: torch.Tensor) -> torch.Tensor:
    """Spacing of bf16 numbers at |v|: 2^(floor(log2|v|) - 7); the smallest normal's ulp below that."""
    a = v.abs().to(torch.float32).clamp(min=2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(a)) - 7.0)


def fp16_ulp(v: torch.Tensor) -> torch.Tensor:
    """Spacing of fp16 numbers at |v| (10 mantissa bits; subnormal spacing 2^-24 below 2^-14)."""
    a = v.abs().to(torch.float32).clamp(min=2.0 ** -14)
    return torch.exp2(torch.floor(torch.log2(a)) - 10.0)


def tolerance(ref_fp32: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Per-element bound: 1 ulp of the output type at |ref| + 1e-2 * RMS(ref)."""
    rms = ref_fp32.to(torch.float64).pow(2).mean().sqrt().to(torch.float32)
    ulp = fp16_ulp(ref_fp32) if out_dtype == torch.float16 else bf16_ulp(ref_fp32)
    return ulp + 1e-2 * rms


def compare(out_bf16: torch.Tensor, ref_bf16: torch.Tensor) -> dict:
    """max |out - ref| against the tolerance, everything as float32 on CPU."""
    out = out_bf16.detach().cpu().to(torch.float32)
    ref = ref_bf16.detach().cpu().to(torch.float32)
    tol = tolerance(ref, ref_bf16.dtype)
    diff = (out - ref).abs()
    ratio = diff / tol
    return {
        "max_abs_diff": float(diff.max()),
        "max_ratio": float(ratio.max()),
        "mismatched": int((diff > 0).sum()),
        "ok": bool((diff <= tol).all()) and bool(torch.isfinite(out).all()),
    }


def flops(m: int, n: int, k: int, bias: bool = False) -> int:
    """operator.py:248-259"""
    return 2 * m * n * k + (2 * m * n if bias else 0)


def gbytes(m: int, n: int, k: int) -> float:
    """operator.py:261-271: |a| + |b| + |c| in GB"""
    return (m * k + n * k + 2 * m * n) / 1e9

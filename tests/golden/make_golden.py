"""Generate the golden fixtures in this directory.  Run once, in a container where the reference
tree is mounted (it is not needed afterwards; the tests read only the .npz files):

    python tests/golden/make_golden.py /path/to/tritonbench-checkout

What it pins
  * quantiser: the reference's own `fp8_row_quantize`
    (tritonbench/operators/fp8_gemm_rowwise/operator.py:136-145) is imported and run on seeded
    inputs; its outputs are stored.  The operator module imports FBGEMM's `get_fp8_constants`
    at load time; FBGEMM is not vendored in the reference tree, so a one-function stand-in module
    that returns (torch.float8_e4m3fn, None, 448.0, 1e-12) is installed first.  Nothing else of
    FBGEMM is faked, and the stock backends stay disabled.
  * block quantiser: the sibling operator's `fp8_block_quantize`
    (tritonbench/operators/fp8_gemm_blockwise/operator.py:87-120), imported and run the same way.
  * non-finite inputs: both quantisers on rows / blocks that hold a NaN or an infinity.
  * GEMM: the reference has no runnable implementation and no test vectors for the GEMM itself
    (its kernels live in FBGEMM), so the stored Y is the fp32 dequantise-then-matmul result computed
    with plain torch CPU ops here, written out independently of oracle/ (no import of it).
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference_quantizer(ref_root: str):
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
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
        sys.modules[n] = mod
    sys.modules[names[-1]].get_fp8_constants = lambda: (torch.float8_e4m3fn, None, 448.0, 1e-12)
    import importlib

    op = importlib.import_module("tritonbench.operators.fp8_gemm_rowwise.operator")
    return op.fp8_row_quantize, op.BUILDIN_SHAPES


def dequant_matmul(xq, wq, xs, ws):
    x = xq.to(torch.float32) * xs[:, None]
    w = wq.to(torch.float32) * ws[:, None]
    return (x @ w.T).to(torch.bfloat16)


def u8(t):
    return t.view(torch.uint8).numpy()


def bf16_bits(t):
    return t.view(torch.int16).numpy()


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRITONBENCH_ROOT", "")
    if not os.path.isdir(os.path.join(ref_root, "tritonbench")):
        raise SystemExit("usage: make_golden.py <checkout of meta-pytorch/tritonbench>  (or set TRITONBENCH_ROOT)")
    quantize, shapes = import_reference_quantizer(ref_root)

    # (1) the reference's own input recipe (operator.py:280-297): bf16 randn under seed 1337
    torch.manual_seed(1337)
    m, n, k = 128, 256, 512
    x = torch.randn((m, k), dtype=torch.bfloat16)
    w = torch.randn((n, k), dtype=torch.bfloat16)
    xq, xs = quantize(x)
    wq, ws = quantize(w)
    np.savez_compressed(
        os.path.join(HERE, "ref_quantizer_bf16_128x256x512.npz"),
        x_bf16=bf16_bits(x), w_bf16=bf16_bits(w), xq=u8(xq), wq=u8(wq), x_scale=xs.numpy(), w_scale=ws.numpy(),
        y_bf16=bf16_bits(dequant_matmul(xq, wq, xs, ws)),
    )

    # (2) edge rows through the reference quantiser: zero row, one huge outlier, tiny values, +-max,
    #     in bf16, fp16 (the 65504 clamp branch) and fp32
    rows = torch.zeros((8, 64), dtype=torch.float32)
    g = torch.Generator().manual_seed(7)
    rows[1] = torch.randn(64, generator=g)
    rows[1, 3] = 3.0e4
    rows[2] = torch.randn(64, generator=g) * 1e-6
    rows[3] = torch.linspace(-448, 448, 64)
    rows[4] = torch.randn(64, generator=g) * 1e-30
    rows[5, 0] = 1.0
    rows[6] = torch.randn(64, generator=g) * 100
    rows[7] = -torch.ones(64)
    edge = {}
    for name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)):
        q, s = quantize(rows.to(dt))
        edge[f"q_{name}"] = u8(q)
        edge[f"s_{name}"] = s.numpy()
    np.savez_compressed(os.path.join(HERE, "ref_quantizer_edge_rows.npz"), rows=rows.numpy(), **edge)

    # (3) benchmark configuration 1: fp32 N(0,1), seed 0, scale = rowabsmax / 448 in fp32
    gen = torch.Generator().manual_seed(0)
    x = torch.randn((m, k), generator=gen, dtype=torch.float32)
    w = torch.randn((n, k), generator=gen, dtype=torch.float32)

    def q32(t):
        s = t.abs().amax(dim=1).clamp(min=1e-12) / 448.0
        return (t / s[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn), s

    xq, xs = q32(x)
    wq, ws = q32(w)
    np.savez_compressed(
        os.path.join(HERE, "config1_seed0_128x256x512.npz"),
        xq=u8(xq), wq=u8(wq), x_scale=xs.numpy(), w_scale=ws.numpy(), y_bf16=bf16_bits(dequant_matmul(xq, wq, xs, ws)),
    )

    # (4) the shape list the reference feeds the operator (operator.py:107-128)
    np.savez_compressed(os.path.join(HERE, "ref_builtin_shapes.npz"), shapes=np.array(shapes, dtype=np.int64))

    # (6) the block quantiser of the sibling operator fp8_gemm_blockwise (operator.py:87-120).  That module
    #     imports fbgemm_gpu.experimental.gen_ai for its side effects only; an empty stand-in lets it load.
    gen_ai = types.ModuleType("fbgemm_gpu.experimental.gen_ai")
    sys.modules["fbgemm_gpu.experimental.gen_ai"] = gen_ai
    sys.modules["fbgemm_gpu.experimental"].gen_ai = gen_ai
    import importlib

    blockwise = importlib.import_module("tritonbench.operators.fp8_gemm_blockwise.operator")
    torch.manual_seed(1337)
    xb = torch.randn((200, 300), dtype=torch.bfloat16)
    xb[130:140, 128:256] = 0.0
    xb[3, 5] = 1000.0
    qb, sb = blockwise.fp8_block_quantize(xb)
    np.savez_compressed(os.path.join(HERE, "ref_block_quantizer_200x300.npz"), x_bf16=bf16_bits(xb), q=u8(qb), scale=sb.numpy())

    # (7) rows (and blocks) that hold a NaN or an infinity, through the same two reference functions: torch's max,
    #     amax and clamp propagate NaN, so one NaN turns the whole row's (block's) scale and codes into NaN;
    #     an infinity gives a zero multiplier, zero codes for the finite elements and NaN for the infinite one
    nf = torch.randn((6, 64), generator=torch.Generator().manual_seed(11))
    nf[1, 5] = float("nan")
    nf[2, 7] = float("inf")
    nf[3, 1] = float("-inf")
    nf[3, 2] = float("nan")
    nf[5] = 0.0
    nonfinite = {}
    for name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)):
        q, s = quantize(nf.to(dt))
        nonfinite[f"q_{name}"] = u8(q)
        nonfinite[f"s_{name}"] = s.numpy()
    xb = torch.randn((130, 260), generator=torch.Generator().manual_seed(12)).to(torch.bfloat16)
    xb[5, 7] = float("nan")       # block (0, 0)
    xb[129, 200] = float("inf")   # block (1, 1)
    qb, sb = blockwise.fp8_block_quantize(xb)
    np.savez_compressed(os.path.join(HERE, "ref_quantizer_nonfinite.npz"), rows=nf.numpy(), **nonfinite,
                        block_x_bf16=bf16_bits(xb), block_q=u8(qb), block_scale=sb.numpy())

    # (5) all 256 e4m3 byte patterns as torch decodes them
    allb = torch.arange(256, dtype=torch.uint8)
    np.savez_compressed(os.path.join(HERE, "e4m3_all_bytes.npz"), values=allb.view(torch.float8_e4m3fn).to(torch.float32).numpy())
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()

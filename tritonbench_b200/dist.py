"""M-sharded (data-parallel over rows) runs of the operator: one process per GPU, W replicated.

The reference has no distributed code at all; this module is the row partition the sharded
benchmark configuration describes: rank r of G owns rows [r*M/G, (r+1)*M/G) of X, x_scale and Y,
every rank holds all of W and w_scale, and the GEMM itself needs no exchange.  The only collective
is the optional all-gather that assembles Y on every rank.
"""
import os
from typing import Optional, Tuple

import torch

W_SEED = 0  # W comes from the same seed on every rank (replicated weights)


def shard_seed(rank: int) -> int:
    """Seed of the X shard of `rank` (seed per shard: 1 + rank)."""
    return 1 + rank


def shard_rows(m_total: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[begin, end) rows of the global problem owned by `rank`; M must divide evenly."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} of {world_size}")
    if m_total % world_size != 0:
        raise ValueError(f"M={m_total} does not divide over {world_size} ranks")
    per = m_total // world_size
    return rank * per, (rank + 1) * per


def env_rank_world() -> Tuple[int, int, int]:
    """(rank, local_rank, world_size) from the torchrun environment; (0, 0, 1) outside it."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def init_process_group(backend: Optional[str] = None) -> bool:
    """Join the torchrun rendezvous if there is one.  Returns True if a group was created."""
    import torch.distributed as td

    rank, local_rank, world = env_rank_world()
    if world == 1:
        return False
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if backend == "nccl":
        torch.cuda.set_device(local_rank)
        td.init_process_group(backend, device_id=torch.device("cuda", local_rank))
    else:
        td.init_process_group(backend)
    return True


def make_shard_inputs(m_total: int, n: int, k: int, world_size: int, rank: int, device):
    """(xq, wq, x_scale, w_scale) of one rank: its X rows from the per-shard seed, W from W_SEED."""
    from . import quantize

    r0, r1 = shard_rows(m_total, world_size, rank)
    xq, xs = quantize.make_quantized(r1 - r0, k, seed=shard_seed(rank), device=device)
    wq, ws = quantize.make_quantized(n, k, seed=W_SEED, device=device)
    return xq, wq, xs, ws


def gathered_output(m_total: int, n: int, world_size: int, rank: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """([M, N] bf16 buffer for the gathered Y, this rank's [M/G, N] slice of it).  Writing the GEMM
    result straight into the slice makes the all-gather in-place: no staging copy."""
    full = torch.empty((m_total, n), dtype=torch.bfloat16, device=device)
    r0, r1 = shard_rows(m_total, world_size, rank)
    return full, full[r0:r1]


def all_gather_rows(full: torch.Tensor, world_size: int) -> None:
    """In-place all-gather of equal row slices of `full` (NCCL over NVLink on GPUs, gloo on CPU)."""
    import torch.distributed as td

    if world_size == 1:
        return
    td.all_gather_into_tensor(full, full[shard_slice(full.shape[0], world_size, td.get_rank())])


def shard_slice(m_total: int, world_size: int, rank: int) -> slice:
    r0, r1 = shard_rows(m_total, world_size, rank)
    return slice(r0, r1)

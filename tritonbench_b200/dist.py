"""M-sharded (data-parallel over rows) runs of the operator: one process per GPU, W replicated.

The reference has no distributed code at all; this module is the row partition the sharded
benchmark configuration describes: rank r of G owns rows [r*M/G, (r+1)*M/G) of X, x_scale and Y,
every rank holds all of W and w_scale, and the GEMM itself needs no exchange.  The only collective
is the optional all-gather that assembles Y on every rank: NCCL's (all_gather_rows), or fused into the GEMM's
epilogue, which then stores every tile into all ranks' copies of Y over NVLink (SharedRows +
ops.fp8_gemm_rowwise_gather).
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


def slice_byte_offset(m_total: int, n: int, world_size: int, rank: int, elem_bytes: int = 2) -> int:
    """Byte offset of rank's first row inside a row-major [m_total, n] matrix (the same in every copy of it)."""
    return shard_rows(m_total, world_size, rank)[0] * n * elem_bytes


def copy_order(world_size: int, rank: int):
    """Ranks in the order their copies are handed to the gather-fused GEMM: the caller's own copy first."""
    return [rank] + [r for r in range(world_size) if r != rank]


class _DeviceArray:
    """Presents library-owned device memory to torch through the CUDA array interface (int16 elements)."""

    def __init__(self, ptr: int, elements: int):
        self.__cuda_array_interface__ = {"shape": (elements,), "typestr": "<i2", "data": (ptr, False), "version": 3}


class SharedRows:
    """The gathered [m_total, n] bf16 matrix of a row-sharded run, one copy per rank, each copy mapped into every
    other rank's process (CUDA IPC through the library's b200fp8_shared_buffer_* calls; torch.distributed only
    carries the 64-byte handles).  `full` is this rank's copy, `mine` its own rows inside it, and `my_rows_everywhere()`
    the addresses of those same rows inside every copy - own copy first - which is what the gather-fused GEMM
    (ops.fp8_gemm_rowwise_gather) writes to.  With world_size 1 it is an ordinary buffer."""

    def __init__(self, m_total: int, n: int, world_size: int, rank: int, device, group=None):
        import ctypes

        import torch.distributed as td

        from . import lib as _lib

        self.m_total, self.n, self.world, self.rank = m_total, n, world_size, rank
        self._lib = _lib.load()
        self._ptr = ctypes.c_void_p()
        self._peers = {}
        handle = ctypes.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        nbytes = m_total * n * 2
        with torch.cuda.device(device):
            _lib.check(self._lib.b200fp8_shared_buffer_create(nbytes, ctypes.byref(self._ptr), handle, len(handle)),
                       "b200fp8_shared_buffer_create")
            self.full = torch.as_tensor(_DeviceArray(self._ptr.value, m_total * n), device=device).view(torch.bfloat16).view(m_total, n)
            self.mine = self.full[shard_slice(m_total, world_size, rank)]
            if world_size > 1:
                handles = [None] * world_size
                td.all_gather_object(handles, bytes(handle.raw), group=group)
                for r, h in enumerate(handles):
                    if r == rank:
                        continue
                    p = ctypes.c_void_p()
                    _lib.check(self._lib.b200fp8_shared_buffer_open(h, len(h), ctypes.byref(p)), f"b200fp8_shared_buffer_open(rank {r})")
                    self._peers[r] = p.value

    def my_rows_everywhere(self):
        off = slice_byte_offset(self.m_total, self.n, self.world, self.rank)
        return [(self._ptr.value if r == self.rank else self._peers[r]) + off for r in copy_order(self.world, self.rank)]

    def close(self) -> None:
        """Unmap the peers' copies and free this rank's.  Every rank must have finished using the others' memory
        (synchronise and pass a barrier first)."""
        for p in self._peers.values():
            self._lib.b200fp8_shared_buffer_close(p)
        self._peers = {}
        if self._ptr:
            self.full = self.mine = None
            self._lib.b200fp8_shared_buffer_destroy(self._ptr)
            self._ptr = None

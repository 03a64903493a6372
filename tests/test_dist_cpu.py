"""The M-sharded path with two CPU ranks over gloo: shard bounds, per-shard seeds, replicated W, and the
in-place all-gather layout, against the single-process oracle on the concatenated problem."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from oracle import fp8_rowwise_oracle as orc
from tritonbench_b200 import dist as shard
from tritonbench_b200 import quantize

M_TOTAL, N, K = 64, 48, 96


def test_shard_rows_cover_the_problem_without_overlap():
    for world in (1, 2, 4, 8):
        spans = [shard.shard_rows(65536, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 65536
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert len({b - a for a, b in spans}) == 1
    with pytest.raises(ValueError):
        shard.shard_rows(10, 3, 0)
    with pytest.raises(ValueError):
        shard.shard_rows(8, 2, 2)


def test_fused_gather_bookkeeping_every_rank_writes_its_rows_into_every_copy():
    """Host logic of the gather-fused GEMM: rank r writes rows [r*M/G, (r+1)*M/G) at the same byte offset of every
    copy, its own copy first.  Emulated on numpy buffers: after all ranks have 'stored', every copy is complete."""
    import numpy as np

    m_total, n = 64, 24
    for world in (1, 2, 4, 8):
        truth = np.arange(m_total * n, dtype=np.uint16).reshape(m_total, n)
        copies = [np.zeros(m_total * n * 2, dtype=np.uint8) for _ in range(world)]
        for rank in range(world):
            order = shard.copy_order(world, rank)
            assert order[0] == rank and sorted(order) == list(range(world))
            off = shard.slice_byte_offset(m_total, n, world, rank)
            r0, r1 = shard.shard_rows(m_total, world, rank)
            assert off == r0 * n * 2
            payload = truth[r0:r1].tobytes()
            for dest in order:
                copies[dest][off:off + len(payload)] = np.frombuffer(payload, dtype=np.uint8)
        for c in copies:
            assert np.array_equal(c.view(np.uint16).reshape(m_total, n), truth)


def test_shard_inputs_use_a_common_w_and_distinct_x():
    a = shard.make_shard_inputs(M_TOTAL, N, K, 2, 0, "cpu")
    b = shard.make_shard_inputs(M_TOTAL, N, K, 2, 1, "cpu")
    assert torch.equal(a[1].view(torch.uint8), b[1].view(torch.uint8)) and torch.equal(a[3], b[3])
    assert not torch.equal(a[0].view(torch.uint8), b[0].view(torch.uint8))
    assert a[0].shape == (M_TOTAL // 2, K)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world))
    assert shard.env_rank_world() == (rank, rank, world)
    assert shard.init_process_group("gloo")
    import torch.distributed as td

    xq, wq, xs, ws = shard.make_shard_inputs(M_TOTAL, N, K, world, rank, "cpu")
    full, mine = shard.gathered_output(M_TOTAL, N, world, rank, "cpu")
    full.zero_()
    mine.copy_(orc.gemm_rowwise(xq, wq, xs, ws))  # CPU stand-in for the rank's GEMM, written in place
    shard.all_gather_rows(full, world)
    # device-time style reduction: the slowest rank's time is what gets reported
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    td.all_reduce(t, op=td.ReduceOp.MAX)
    torch.save({"full": full, "tmax": float(t)}, os.path.join(out_dir, f"rank{rank}.pt"))
    td.barrier()
    td.destroy_process_group()


def test_two_gloo_ranks_assemble_the_global_result(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    xs_parts = [quantize.make_quantized(M_TOTAL // world, K, seed=shard.shard_seed(r)) for r in range(world)]
    xq = torch.cat([p[0].view(torch.uint8) for p in xs_parts]).view(torch.float8_e4m3fn)
    xs = torch.cat([p[1] for p in xs_parts])
    wq, ws = quantize.make_quantized(N, K, seed=shard.W_SEED)
    want = orc.gemm_rowwise(xq, wq, xs, ws)
    for r in range(world):
        got = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        assert torch.equal(got["full"], want)
        assert got["tmax"] == float(world)

"""Head sharding across ranks, exercised with two gloo ranks on CPU.

The hard path has no collective: every (batch, head) is independent, so a rank works on a
contiguous slice of heads and results are concatenated.  The CPU oracle stands in for the device
kernels here; what is tested is the partition, the per-rank slicing of every operand (vectors are
[B,N,H,C], labels [B,H,N], tau [H], hard [B,H]) and that gathering reproduces the unsharded result.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def worker(rank, world, port, result_path):
    sys.path.insert(0, ROOT)
    from dism_b200.sharding import head_range, shard_operands
    from oracle import dism_oracle as o
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    rng = np.random.default_rng(0)  # same data on every rank
    b, n, h, r, dv = 2, 256, 6, 32, 64
    operands = dict(
        sq=o.bf16_round(rng.standard_normal((b, n, h, r)).astype(np.float32) * .3),
        sk=o.bf16_round(rng.standard_normal((b, n, h, r)).astype(np.float32) * .3),
        v=o.bf16_round(rng.standard_normal((b, n, h, dv)).astype(np.float32)),
        iq=rng.integers(0, 6, (b, h, n), dtype=np.int32), ik=rng.integers(0, 6, (b, h, n), dtype=np.int32),
        hard=rng.random((b, h)) < .8, tau=np.linspace(-.5, .5, h).astype(np.float32))
    mine = shard_operands(operands, rank, world)
    lo, hi = head_range(h, rank, world)
    assert mine['sq'].shape[2] == hi - lo and mine['iq'].shape[1] == hi - lo and mine['tau'].shape[0] == hi - lo
    out, lse2 = o.forward(mine['sq'], mine['sk'], mine['v'], mine['iq'], mine['ik'], mine['hard'], mine['tau'])
    pieces = [None] * world
    dist.all_gather_object(pieces, (lo, hi, out, lse2))
    if rank == 0:
        full, full_lse2 = o.forward(*(operands[k] for k in ('sq', 'sk', 'v', 'iq', 'ik', 'hard', 'tau')))
        pieces.sort(key=lambda p: p[0])
        assert [p[0] for p in pieces] == [head_range(h, r_, world)[0] for r_ in range(world)]
        gathered = np.concatenate([p[2] for p in pieces], axis=2)
        gathered_lse2 = np.concatenate([p[3] for p in pieces], axis=1)
        np.save(result_path, np.array([np.array_equal(gathered, full), np.array_equal(gathered_lse2, full_lse2)]))
    dist.barrier()
    dist.destroy_process_group()


def free_port():
    import socket
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def test_two_rank_head_sharding(tmp_path):
    result = str(tmp_path / 'ok.npy')
    mp.spawn(worker, args=(2, free_port(), result), nprocs=2, join=True)
    assert np.load(result).all()


def test_head_ranges_cover_and_balance():
    sys.path.insert(0, ROOT)
    from dism_b200.sharding import head_range
    for heads in (1, 2, 6, 16, 32, 33):
        for world in (1, 2, 3, 4, 8):
            ranges = [head_range(heads, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == heads
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [hi - lo for lo, hi in ranges]
            assert max(sizes) - min(sizes) <= 1

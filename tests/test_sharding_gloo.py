"""CPU, world_size 2 over gloo: the host logic of the two multi-GPU modes.
The compute step is replaced by the oracle (there is no CPU product path), so
what is checked is the partitioning, the K/V exchange and the query windowing."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from baselinebenchmark_b200 import sharding
from oracle import moba_oracle as O


def test_unit_shard_partitions_every_unit_once():
    for nseq, hkv, world in [(16, 8, 8), (16, 8, 1), (3, 2, 4), (5, 1, 2), (2, 8, 3)]:
        seen = []
        for r in range(world):
            seen += sharding.unit_shard(nseq, hkv, world, r)
        assert sorted(seen) == [(s, h) for s in range(nseq) for h in range(hkv)]
        sizes = [len(sharding.unit_shard(nseq, hkv, world, r)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    # BASELINE.json configs[3]: 16 sequences x 8 KV-head groups on 8 GPUs = 16 units per GPU
    assert len(sharding.unit_shard(16, 8, 8, 5)) == 16


def test_context_windows_are_chunk_aligned_and_cover():
    for total, chunk, world in [(1048576, 4096, 8), (1000, 64, 3), (130, 64, 4), (4096, 512, 8)]:
        wins = [sharding.context_window(total, chunk, world, r) for r in range(world)]
        assert wins[0][0] == 0 and wins[-1][1] == total
        for (l0, h0), (l1, h1) in zip(wins, wins[1:]):
            assert h0 == l1
        for lo, hi in wins:
            if hi > lo:                                  # more ranks than chunks leaves empty windows
                assert lo % chunk == 0 and (hi % chunk == 0 or hi == total)
    assert sharding.context_window(1048576, 4096, 8, 3) == (3 * 131072, 4 * 131072)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_forward(q, k, v, cu, max_seqlen, chunk, topk, q_token_begin):
    """Oracle stand-in for the windowed operator: full evaluation, window rows returned."""
    n = k.shape[0]
    q_full = torch.zeros(n, q.shape[1], q.shape[2], dtype=q.dtype)
    q_full[q_token_begin:q_token_begin + q.shape[0]] = q
    out, _, _ = O.moba_forward(q_full, k, v, cu.numpy(), max_seqlen, chunk, topk)
    return out[q_token_begin:q_token_begin + q.shape[0]]


def _cp_worker(rank, world, port, total, chunk, topk, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, cu = O.make_inputs([total], 4, 2, 128, chunk, seed=77)
        lo, hi = sharding.context_window(total, chunk, world, rank)
        out = sharding.moba_context_parallel(q[lo:hi], k[lo:hi], v[lo:hi], total, chunk, topk,
                                             forward=_oracle_forward)
        ref, _, _ = O.moba_forward(q, k, v, cu, total, chunk, topk)
        result[rank] = float((out - ref[lo:hi]).abs().max()) if hi > lo else 0.0
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total,chunk,topk", [(1000, 64, 4), (640, 128, 3)])
def test_context_parallel_matches_single_process(total, chunk, topk):
    world = 2
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_cp_worker, args=(world, _free_port(), total, chunk, topk, result), nprocs=world, join=True)
        assert sorted(result.keys()) == [0, 1]
        assert max(result.values()) == 0.0          # same arithmetic on every rank: identical, not just close


def _unit_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens, hq, hkv, chunk, topk = [300, 200, 260], 4, 2, 64, 3
        q, k, v, cu = O.make_inputs(lens, hq, hkv, 128, chunk, seed=5)
        ref, _, _ = O.moba_forward(q, k, v, cu, max(lens), chunk, topk)
        units = sharding.unit_shard(len(lens), hkv, world, rank)
        worst = 0.0
        for tok, qh, kvh in sharding.shard_slices(units, cu, hq // hkv):
            n = tok.stop - tok.start
            out, _, _ = O.moba_forward(q[tok, qh], k[tok, kvh], v[tok, kvh], np.array([0, n]), n, chunk, topk)
            worst = max(worst, float((out - ref[tok, qh]).abs().max()))
        # the driver of a real job only exchanges timings: max over ranks
        t = torch.tensor([float(len(units))])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        result[rank] = (worst, len(units), float(t))
    finally:
        dist.destroy_process_group()


def test_unit_sharding_needs_no_exchange():
    world = 2
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_unit_worker, args=(world, _free_port(), result), nprocs=world, join=True)
        assert sum(r[1] for r in result.values()) == 6
        # a unit evaluated alone equals its slice of the whole-batch evaluation
        assert max(r[0] for r in result.values()) == 0.0
        assert all(r[2] == 3.0 for r in result.values())


def _bad_shape_worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        total, chunk = 640, 64
        q, k, v, _ = O.make_inputs([total], 4, 2, 128, chunk, seed=3)
        lo, hi = sharding.context_window(total, chunk, world, rank)
        if rank == 1:
            hi -= 5                                  # this rank passes too few rows
        try:
            sharding.moba_context_parallel(q[lo:hi], k[lo:hi], v[lo:hi], total, chunk, 3, forward=_oracle_forward)
            result[rank] = "returned"
        except ValueError as exc:
            result[rank] = str(exc)
    finally:
        dist.destroy_process_group()


def test_a_rank_with_a_bad_shape_makes_every_rank_raise():
    """Failure made on the host: rank 1 passes the wrong number of rows.  Every rank gets a
    ValueError from the agreement step instead of waiting in the exchange for a peer that
    never joins."""
    world = 2
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_bad_shape_worker, args=(world, _free_port(), result), nprocs=world, join=True)
        assert sorted(result.keys()) == [0, 1]
        assert "invalid" in result[0] and "this rank" not in result[0]
        assert "invalid" in result[1] and "this rank" in result[1]


def _absent_rank_worker(rank, world, port, result):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        if rank == 1:
            result[rank] = "left between steps"      # returns early: never enters the collective
            return
        try:
            sharding.agree(True, None)
            result[rank] = "returned"
        except Exception as exc:                     # noqa: BLE001  (gloo raises RuntimeError / DistBackendError)
            result[rank] = f"error: {type(exc).__name__}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:                            # noqa: BLE001
            pass


def test_a_rank_that_never_joins_ends_the_collective_with_an_error():
    """Rank 1 leaves before the step; rank 0's agreement collective ends with an error after the
    process group's (short) timeout instead of blocking."""
    world = 2
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_absent_rank_worker, args=(world, _free_port(), result), nprocs=world, join=True)
        assert result[1] == "left between steps"
        assert result[0].startswith("error")

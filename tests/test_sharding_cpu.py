"""The multi-rank orchestration on CPU: two gloo ranks, the oracle standing in for the
GPU arithmetic.  Checks the sharding ranges, which gradients are all-reduced, that the
replicated gradient ends up identical on both ranks, and that shards put back together
equal the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as ol
from primitiv_b200.sharding import ShardedMatmul, local_batch, shard_range


def test_shard_range_follows_batch_split():
    assert shard_range(8, 0, 2) == (0, 4) and shard_range(8, 1, 2) == (4, 4)
    assert shard_range(65536, 7, 8) == (57344, 8192)
    assert local_batch(1, 8) == 1 and local_batch(32, 8) == 4
    with pytest.raises(ValueError):
        shard_range(10, 0, 4)          # functions::batch::split refuses an indivisible batch
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


class OracleBackend:
    """numpy arrays + the CPU oracle in place of device memory + the CUDA kernels."""

    def matmul_fw(self, a, b, y, di, dj, dk, ba, bb):
        y[:] = ol.fw_naive(a, b, di, dj, dk, ba, bb)

    def matmul_bw(self, a, b, gy, ga, gb, di, dj, dk, ba, bb, acc_a=True, acc_b=True):
        # either gradient may be left out; acc_* False means the array holds garbage and is overwritten
        ga0 = np.zeros(di * dj * ba, np.float32) if (ga is None or not acc_a) else ga
        gb0 = np.zeros(dj * dk * bb, np.float32) if (gb is None or not acc_b) else gb
        ga2, gb2 = ol.bw_naive(a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
        if ga is not None:
            ga[:] = ga2
        if gb is not None:
            gb[:] = gb2

    def scratch_like(self, t):
        return np.full_like(t, np.nan)      # uninitialised memory: whoever reads it before writing fails the test

    def add_(self, dst, src):
        dst += src


CASES = [(6, 5, 4, 1, 4), (6, 5, 4, 4, 1), (6, 5, 4, 4, 4), (6, 5, 4, 1, 1)]


def _shard(x, vol, batch, rank, world):
    if batch == 1:
        return x.copy()
    first, count = shard_range(batch, rank, world)
    return x[first * vol:(first + count) * vol].copy()


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_reduce(arr):
        # asynchronous, as on the GPU: the handle is waited for only after the local gradient
        t = torch.from_numpy(arr)
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=True)

    sm = ShardedMatmul(OracleBackend(), world, rank, all_reduce)
    results = {}
    for ci, (di, dj, dk, ba, bb) in enumerate(CASES):
        bs = max(ba, bb)
        rng = np.random.default_rng(100 + ci)      # same global tensors on every rank
        a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
        b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
        gy = rng.standard_normal(di * dk * bs).astype(np.float32)
        la, lb, lg = _shard(a, di * dj, ba, rank, world), _shard(b, dj * dk, bb, rank, world), \
            _shard(gy, di * dk, bs, rank, world)
        y = np.empty(lg.size, np.float32)
        sm.forward(la, lb, y, di, dj, dk, ba, bb)
        ga = np.full(la.size, 0.5, np.float32)
        gb = np.full(lb.size, 0.5, np.float32)
        before = sm.collectives
        sm.backward(la, lb, lg, ga, gb, di, dj, dk, ba, bb)
        results["y%d" % ci], results["ga%d" % ci], results["gb%d" % ci] = y, ga, gb
        results["coll%d" % ci] = np.array([sm.collectives - before])
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **results)
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_result(tmp_path):
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    ranks = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    for ci, (di, dj, dk, ba, bb) in enumerate(CASES):
        bs = max(ba, bb)
        rng = np.random.default_rng(100 + ci)
        a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
        b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
        gy = rng.standard_normal(di * dk * bs).astype(np.float32)
        y = ol.fw_naive(a, b, di, dj, dk, ba, bb)
        ga, gb = ol.bw_naive(a, b, gy, np.full(a.size, 0.5, np.float32), np.full(b.size, 0.5, np.float32),
                             di, dj, dk, ba, bb)

        def joined(key, batch):
            if batch == 1:      # replicated: both ranks must hold the same bits
                assert np.array_equal(ranks[0][key], ranks[1][key]), key
                return ranks[0][key]
            return np.concatenate([ranks[r][key] for r in range(world)])

        if bs > 1:
            np.testing.assert_allclose(joined("y%d" % ci, bs), y, rtol=1e-6, atol=1e-6)
        else:
            np.testing.assert_allclose(ranks[0]["y%d" % ci], y, rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(joined("ga%d" % ci, ba), ga, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(joined("gb%d" % ci, bb), gb, rtol=1e-5, atol=1e-5)
        # exactly the cases with one broadcast operand need the exchange step
        expected = 1 if (ba == 1) != (bb == 1) else 0
        assert int(ranks[0]["coll%d" % ci][0]) == expected

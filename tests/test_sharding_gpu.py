"""Two GPUs, one process each, NCCL: a broadcast weight's gradient summed across ranks.

The MLP-layer shape (weights {256,192} broadcast over a batch of 64 vectors... kept small so
the CPU oracle can check it): each rank holds half the batch, computes its partial gW on
the tensor-core kernel, the partials are all-reduced over NCCL and added into the
replicated gradient.  Needs two GPUs; skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch

import oracle_lib as ol

pytestmark = pytest.mark.gpu

DI, DJ, DK, BA, BB = 256, 192, 8, 1, 64


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    import primitiv_b200 as pb
    from primitiv_b200.sharding import GpuBackend, ShardedMatmul, nccl_all_reduce, shard_range
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = pb.Context(rank)
    ctx.set_path_policy(2)
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, DI * DJ).astype(np.float32)
    b = rng.uniform(-1, 1, DJ * DK * BB).astype(np.float32)
    gy = rng.standard_normal(DI * DK * BB).astype(np.float32)
    first, count = shard_range(BB, rank, world)
    cu = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    la, lb = cu(a), cu(b[first * DJ * DK:(first + count) * DJ * DK])
    lgy = cu(gy[first * DI * DK:(first + count) * DI * DK])
    y = torch.empty(DI * DK * count, device="cuda")
    ga = torch.full((DI * DJ,), 0.5, device="cuda")
    gb = torch.full((DJ * DK * count,), 0.5, device="cuda")
    sm = ShardedMatmul(GpuBackend(ctx, pb.MODE_FP32_3XTF32), world, rank, nccl_all_reduce)
    sm.forward(la, lb, y, DI, DJ, DK, BA, BB)
    sm.backward(la, lb, lgy, ga, gb, DI, DJ, DK, BA, BB)
    torch.cuda.synchronize()
    assert ctx.status_poll() == 0 and sm.collectives == 1
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), y=y.cpu().numpy(), ga=ga.cpu().numpy(),
             gb=gb.cpu().numpy())
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_broadcast_weight_gradient_is_all_reduced(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % k)) for k in range(world)]
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, DI * DJ).astype(np.float32)
    b = rng.uniform(-1, 1, DJ * DK * BB).astype(np.float32)
    gy = rng.standard_normal(DI * DK * BB).astype(np.float32)
    y64 = ol.fw_f64(a, b, DI, DJ, DK, BA, BB)
    ga64, gb64 = ol.bw_f64(a, b, gy, np.full(a.size, 0.5, np.float32), np.full(b.size, 0.5, np.float32),
                           DI, DJ, DK, BA, BB)
    assert np.array_equal(r[0]["ga"], r[1]["ga"])          # replicas stay bit-identical
    assert ol.rel_err(r[0]["ga"], ga64) <= 1e-5
    assert ol.rel_err(np.concatenate([r[0]["y"], r[1]["y"]]), y64) <= 1e-5
    assert ol.rel_err(np.concatenate([r[0]["gb"], r[1]["gb"]]), gb64) <= 1e-5

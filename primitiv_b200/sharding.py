"""Batch sharding of matmul_fw / matmul_bw across ranks (one process per GPU).

The path shards by the minibatch: every product is independent per batch index, except
the batch sum into the gradient of a broadcast operand (batch 1), which is the single
exchange step.  Partitioning follows primitiv's ``functions::batch::split``
(primitiv/core/tensor_funcs.cc:366-384): equal contiguous chunks, an indivisible batch is
an error.  Tensors with batch N hold N / world elements per rank; tensors with batch 1
(weights and their gradients) are replicated and stay bit-identical on every rank because
each rank adds the same all-reduced partial.

The orchestration is independent of where the arithmetic runs: ``ShardedMatmul`` takes a
*backend* with four methods (``matmul_fw``, ``matmul_bw``, ``scratch_like``, ``add_``) and an
``all_reduce`` callable that may return a handle with ``wait()`` (an exchange still in
flight).  ``GpuBackend`` drives the C ABI on this rank's GPU; the CPU tests plug in the
oracle and a gloo process group to check the orchestration itself.
"""


def shard_range(total, rank, world):
    """(first, count) of this rank's contiguous share of a batch of `total`."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("invalid rank %r of %r" % (rank, world))
    span = total // world
    if span * world != total:
        raise ValueError("Could not split the batch with size %d into %d partitions." % (total, world))
    return rank * span, span


def local_batch(global_batch, world):
    """Batch size a rank holds for a tensor whose global batch is `global_batch` (1 = replicated)."""
    return 1 if global_batch == 1 else shard_range(global_batch, 0, world)[1]


class ShardedMatmul:
    """matmul_fw / matmul_bw of one rank over its batch shard.

    ba, bb below are the GLOBAL batch sizes of a and b (1 or N); the tensors passed in are
    this rank's shards (replicas for batch 1).
    """

    def __init__(self, backend, world, rank, all_reduce):
        self.backend, self.world, self.rank, self.all_reduce = backend, world, rank, all_reduce
        self.collectives = 0

    def forward(self, a, b, y, di, dj, dk, ba, bb):
        self.backend.matmul_fw(a, b, y, di, dj, dk, local_batch(ba, self.world), local_batch(bb, self.world))

    def backward(self, a, b, gy, ga, gb, di, dj, dk, ba, bb):
        la, lb = local_batch(ba, self.world), local_batch(bb, self.world)
        bk = self.backend
        a_summed = ba == 1 and bb > 1      # ga receives a sum over the (sharded) batch
        b_summed = bb == 1 and ba > 1
        if self.world == 1 or not (a_summed or b_summed):
            # every gradient is either local to the shard or (ba == bb == 1) replicated work
            bk.matmul_bw(a, b, gy, ga, gb, di, dj, dk, la, lb)
            return
        # The summed gradient's partial is computed first (stored, not added: the scratch needs
        # no zero-fill), its all-reduce is started, and the other gradient, which is local to the
        # shard, is computed while the partials cross the links.  Only then is the reduced sum
        # added into the replicated gradient: one `+=` of the same bits on every rank
        # (primitiv/devices/cuda/ops/matmul.cu:127-136 is the single-GPU form of the same sum).
        if a_summed:
            part = bk.scratch_like(ga)
            bk.matmul_bw(a, b, gy, part, None, di, dj, dk, la, lb, acc_a=False)
            pending = self.all_reduce(part)
            bk.matmul_bw(a, b, gy, None, gb, di, dj, dk, la, lb)      # gb is per batch element: local
            if pending is not None:
                pending.wait()
            bk.add_(ga, part)
        else:
            part = bk.scratch_like(gb)
            bk.matmul_bw(a, b, gy, None, part, di, dj, dk, la, lb, acc_b=False)
            pending = self.all_reduce(part)
            bk.matmul_bw(a, b, gy, ga, None, di, dj, dk, la, lb)
            if pending is not None:
                pending.wait()
            bk.add_(gb, part)
        self.collectives += 1


class GpuBackend:
    """The C ABI on this rank's GPU; tensors are torch CUDA tensors (device memory only)."""

    def __init__(self, ctx, mode):
        self.ctx, self.mode = ctx, mode
        self._scratch = {}

    def matmul_fw(self, a, b, y, di, dj, dk, ba, bb):
        self.ctx.matmul_fw(self.mode, a.data_ptr(), b.data_ptr(), y.data_ptr(), di, dj, dk, ba, bb)

    def matmul_bw(self, a, b, gy, ga, gb, di, dj, dk, ba, bb, acc_a=True, acc_b=True):
        """ga / gb may be None (that gradient is skipped); acc_* False stores instead of adding."""
        self.ctx.matmul_bw_ex(self.mode, a.data_ptr(), b.data_ptr(), gy.data_ptr(),
                              None if ga is None else ga.data_ptr(), None if gb is None else gb.data_ptr(),
                              di, dj, dk, ba, bb, acc_a, acc_b)

    def scratch_like(self, t):
        """Uninitialised device memory of t's size, kept for the next step (no allocation per step)."""
        import torch
        key = (t.numel(), t.dtype)
        if key not in self._scratch:
            self._scratch[key] = torch.empty_like(t)
        return self._scratch[key]

    def add_(self, dst, src):
        self.ctx.op("b200_inplace_add", self.mode, src.data_ptr(), dst.data_ptr(), dst.numel(), 1, 1, 1.0, None)


def nccl_all_reduce(t):
    """Starts the sum over ranks on NCCL's own stream (it first waits for the work queued so far
    on the current stream) and returns the handle; handle.wait() makes the current stream, not
    the host, wait for the result."""
    import torch.distributed as dist
    return dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=True)

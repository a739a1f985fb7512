"""Full-size workloads, checked through size-independent properties.

At these sizes the CPU oracle would take hours, so correctness is established by
the checksum identity of a matrix product, evaluated in fp64:
    u^T (A B) = (u^T A) B      and      (A B) v = A (B v)
for random +-1 vectors u, v.  A wrong tile, a dropped k-block, a missed batch or a
non-accumulating epilogue all break it.  Inputs are seeded synthetic tensors with
the shapes and value distributions of the named workloads.  torch is used here as
the fp64 checker and to hold device memory, not as the thing under test."""
import numpy as np
import pytest
import torch

import primitiv_b200 as pb
from gpu_util import TOL

pytestmark = pytest.mark.gpu


def _mat(t, rows, cols, n):
    """Flat column-major {rows, cols} x n device tensor -> (n, rows, cols) view."""
    return t.view(n, cols, rows).transpose(1, 2)


def _rel(x, ref):
    return float((x.double() - ref).norm() / ref.norm())


def _pm1(n, gen):
    return (torch.randint(0, 2, (n,), generator=gen, device="cuda").double() * 2 - 1)


def _combined(a, b, t, di, dj, dk, ba, bb):
    """With a broadcast `a`, b's (and y's / gy's) batches are adjacent columns of one matrix."""
    if ba == 1 and bb > 1:
        return dk * bb, 1
    return dk, bb


def check_fw(ctx, mode, a, b, di, dj, dk, ba, bb, tol, gen):
    bs = max(ba, bb)
    y = torch.full((di * dk * bs,), float("nan"), device="cuda", dtype=a.dtype)
    ctx.matmul_fw(mode, a.data_ptr(), b.data_ptr(), y.data_ptr(), di, dj, dk, ba, bb)
    torch.cuda.synchronize()
    assert ctx.status_poll() == 0
    dk, bb = _combined(a, b, y, di, dj, dk, ba, bb)
    bs = max(ba, bb)
    u, v = _pm1(di, gen), _pm1(dk, gen)
    A, B, Y = _mat(a, di, dj, ba), _mat(b, dj, dk, bb), _mat(y, di, dk, bs)
    for n in range(bs):
        An, Bn, Yn = A[n if ba > 1 else 0].double(), B[n if bb > 1 else 0].double(), Y[n].double()
        assert _rel(u @ Yn, (u @ An) @ Bn) <= tol
        assert _rel(Yn @ v, An @ (Bn @ v)) <= tol
    return y


def check_bw(ctx, mode, a, b, gy, di, dj, dk, ba, bb, tol, gen, prefill=0.5):
    ga = torch.full((di * dj * ba,), prefill, device="cuda", dtype=a.dtype)
    gb = torch.full((dj * dk * bb,), prefill, device="cuda", dtype=a.dtype)
    ctx.matmul_bw(mode, a.data_ptr(), b.data_ptr(), gy.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                  di, dj, dk, ba, bb)
    torch.cuda.synchronize()
    assert ctx.status_poll() == 0
    dk, bb = _combined(a, b, gy, di, dj, dk, ba, bb)
    bs = max(ba, bb)
    A, B, GY = _mat(a, di, dj, ba), _mat(b, dj, dk, bb), _mat(gy, di, dk, bs)
    GA, GB = _mat(ga, di, dj, ba), _mat(gb, dj, dk, bb)
    ui, uj, uk = _pm1(di, gen), _pm1(dj, gen), _pm1(dk, gen)
    # ga[n or 0] = prefill + sum gy[n] b[n or 0]^T : check  ui^T ga  and  ga uj  (same for gb)
    ref_l = [torch.zeros(dj, device="cuda", dtype=torch.float64) for _ in range(ba)]
    ref_r = [torch.zeros(di, device="cuda", dtype=torch.float64) for _ in range(ba)]
    rb_l = [torch.zeros(dk, device="cuda", dtype=torch.float64) for _ in range(bb)]
    rb_r = [torch.zeros(dj, device="cuda", dtype=torch.float64) for _ in range(bb)]
    for n in range(bs):
        An, Bn, Gn = A[n if ba > 1 else 0].double(), B[n if bb > 1 else 0].double(), GY[n].double()
        ia, ib = (n if ba > 1 else 0), (n if bb > 1 else 0)
        ref_l[ia] += (ui @ Gn) @ Bn.T
        ref_r[ia] += Gn @ (Bn.T @ uj)
        rb_l[ib] += (uj @ An.T) @ Gn
        rb_r[ib] += An.T @ (Gn @ uk)
    for n in range(ba):
        G = GA[n].double()
        assert _rel(ui @ G, ref_l[n] + prefill * ui.sum()) <= tol
        assert _rel(G @ uj, ref_r[n] + prefill * uj.sum()) <= tol
    for n in range(bb):
        G = GB[n].double()
        assert _rel(uj @ G, rb_l[n] + prefill * uj.sum()) <= tol
        assert _rel(G @ uk, rb_r[n] + prefill * uk.sum()) <= tol
    return ga, gb


def _gen(seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return g


def test_batched_square_gemm_workload_full_size(ctx):
    """A, B {4096,4096} x 8, N(0, 0.02); gy N(0,1); fp32 3xTF32: forward and both backward products."""
    g = _gen(0)
    n, bs = 4096, 8
    a = torch.randn(n * n * bs, generator=g, device="cuda") * 0.02
    b = torch.randn(n * n * bs, generator=g, device="cuda") * 0.02
    gy = torch.randn(n * n * bs, generator=g, device="cuda")
    check_fw(ctx, pb.MODE_FP32_3XTF32, a, b, n, n, n, bs, bs, TOL["3xtf32"], g)
    check_bw(ctx, pb.MODE_FP32_3XTF32, a, b, gy, n, n, n, bs, bs, TOL["3xtf32"], g, prefill=0.0)


def test_batched_square_gemm_workload_full_size_3xfp16(ctx):
    """The same workload in the second fp32-grade mode (row-scaled half planes, three fp16 passes):
    held to the same 1e-5 bound."""
    g = _gen(4)
    n, bs = 4096, 8
    a = torch.randn(n * n * bs, generator=g, device="cuda") * 0.02
    b = torch.randn(n * n * bs, generator=g, device="cuda") * 0.02
    gy = torch.randn(n * n * bs, generator=g, device="cuda")
    check_fw(ctx, pb.MODE_FP32_3XFP16, a, b, n, n, n, bs, bs, TOL["3xfp16"], g)
    check_bw(ctx, pb.MODE_FP32_3XFP16, a, b, gy, n, n, n, bs, bs, TOL["3xfp16"], g, prefill=0.5)


def test_mlp_layer_shapes_full_batch(ctx):
    """784 -> 1024 -> 1024 -> 10 with batch 65536 (> 65535: no grid.y batch index anywhere), broadcast weights."""
    g = _gen(1)
    bs = 65536
    for (rows, cols) in ((1024, 784), (1024, 1024), (10, 1024)):
        lim = (6.0 / (rows + cols)) ** 0.5
        w = (torch.rand(rows * cols, generator=g, device="cuda") * 2 - 1) * lim
        x = torch.rand(cols * bs, generator=g, device="cuda")
        gy = torch.randn(rows * bs, generator=g, device="cuda")
        check_fw(ctx, pb.MODE_FP32_3XTF32, w, x, rows, cols, 1, 1, bs, TOL["3xtf32"], g)
        check_bw(ctx, pb.MODE_FP32_3XTF32, w, x, gy, rows, cols, 1, 1, bs, TOL["3xtf32"], g)


def test_lstm_step_shapes_tf32(ctx):
    """Wx {4096,512}, Wh {4096,1024} broadcast over embeddings {512} x 64 and states {1024} x 64; TF32 fast mode."""
    g = _gen(2)
    for cols in (512, 1024):
        w = (torch.rand(4096 * cols, generator=g, device="cuda") * 2 - 1) * 0.1
        x = torch.randn(cols * 64, generator=g, device="cuda")
        gy = torch.randn(4096 * 64, generator=g, device="cuda")
        check_fw(ctx, pb.MODE_TF32, w, x, 4096, cols, 1, 1, 64, TOL["tf32"], g)
        check_bw(ctx, pb.MODE_TF32, w, x, gy, 4096, cols, 1, 1, 64, TOL["tf32"], g)


def test_fp16_workload_full_size(ctx):
    """A {8192,8192} broadcast, B {8192,2048} x 32, half storage, fp32 accumulation; gA summed over 32 batches."""
    g = _gen(3)
    a = (torch.randn(8192 * 8192, generator=g, device="cuda") * 0.05).half()
    b = (torch.randn(8192 * 2048 * 32, generator=g, device="cuda") * 0.05).half()
    check_fw(ctx, pb.MODE_FP16, a, b, 8192, 8192, 2048, 1, 32, TOL["fp16"], g)
    gy = torch.randn(8192 * 2048 * 32, generator=g, device="cuda").half()
    check_bw(ctx, pb.MODE_FP16, a, b, gy, 8192, 8192, 2048, 1, 32, TOL["fp16"], g, prefill=0.0)

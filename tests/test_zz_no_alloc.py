"""The allocation-free product, for hosts that must not allocate on the calling path
(an application that owns all device memory through its own allocator, or a request
loop that bans cudaMalloc / cudaFree because they synchronise the device).

b200_gemm_3xtf32_noalloc keeps its packing planes in a fixed array inside the
library instead of pool memory.  It is checked here against the ordinary entry
point (b200_gemm, 3xTF32, tensor-core kernel; same accuracy class, the last bits may differ
because b200_gemm may split a long contraction over k) on two calls in a row: the second
call is smaller and differently shaped than the first, so planes left behind by the
first call would show up as wrong results if the second call read anything it had
not written itself.  The file name sorts last on purpose: a run that stops at the
first failure has then already been through every other test."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
import primitiv_b200 as pb

pytestmark = pytest.mark.gpu

# normwise bound of the fp32 (3xTF32) mode, as in the other parity tests
TOL = 1e-5


def _run_pair(ctx, ta, tb, m, n, k, accumulate, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    A = torch.rand(m * k, generator=g, device="cuda") * 2 - 1
    B = torch.rand(n * k, generator=g, device="cuda") * 2 - 1
    C0 = torch.rand(m * n, generator=g, device="cuda")
    want, got = C0.clone(), C0.clone()
    ctx.gemm(pb.MODE_FP32_3XTF32, ta, tb, A.data_ptr(), B.data_ptr(), want.data_ptr(), m, n, k,
             accumulate=accumulate, force_path=2)
    before = ctx.pool_stats()
    ctx.gemm_3xtf32_noalloc(ta, tb, A.data_ptr(), B.data_ptr(), got.data_ptr(), m, n, k, accumulate)
    torch.cuda.synchronize()
    assert ctx.status_poll() == 0
    assert ctx.pool_stats() == before            # the pool was not touched
    err = float((got.double() - want.double()).norm() / want.double().norm())
    assert err <= TOL, err
    # and both agree with the fp64 oracle, not just with each other
    a_np, b_np = A.cpu().numpy(), B.cpu().numpy()
    Am = a_np.reshape(m, k) if ta else a_np.reshape(k, m).T
    Bm = b_np.reshape(k, n) if tb else b_np.reshape(n, k).T
    ref = Am.astype(np.float64) @ Bm.astype(np.float64)
    if accumulate:
        ref = ref + C0.cpu().numpy().astype(np.float64).reshape(n, m).T
    ref = np.ascontiguousarray(ref.T).reshape(-1)
    assert ol.rel_err(got.cpu().numpy(), ref) <= TOL
    return err


def test_matches_the_pool_backed_entry_point_on_two_calls_in_a_row(ctx):
    _run_pair(ctx, 0, 0, 512, 384, 1024, accumulate=False, seed=11)
    _run_pair(ctx, 1, 1, 200, 136, 72, accumulate=True, seed=12)


def test_a_product_that_fills_the_fixed_array_exactly(ctx):
    """1024 x 1024 x 2048: two planes of (m + n) * k floats are exactly the 8 Mi floats of the array,
    the largest case the entry point accepts.  An off-by-one in the plane layout would show here
    as a wrong last row or as a rejected call."""
    _run_pair(ctx, 0, 1, 1024, 1024, 2048, accumulate=False, seed=13)
    _run_pair(ctx, 1, 0, 1024, 1024, 2048, accumulate=True, seed=14)


def test_one_column_more_than_fits_is_rejected(ctx):
    x = torch.zeros(16, device="cuda")
    launches = ctx.launch_count()
    with pytest.raises(pb.B200Error) as e:
        ctx.gemm_3xtf32_noalloc(0, 0, x.data_ptr(), x.data_ptr(), x.data_ptr(), 1024, 1025, 2048)
    assert e.value.code == 1006
    assert ctx.launch_count() == launches    # nothing ran, so the small buffer was never read


def test_sizes_beyond_the_fixed_array_are_rejected(ctx):
    x = torch.zeros(16, device="cuda")
    launches = ctx.launch_count()
    with pytest.raises(pb.B200Error) as e:
        # (m + n) * k = 8 Mi elements: twice what the 32 MiB array holds.  Nothing is launched,
        # so the small buffer is never dereferenced.
        ctx.gemm_3xtf32_noalloc(0, 0, x.data_ptr(), x.data_ptr(), x.data_ptr(), 2048, 2048, 2048)
    assert e.value.code == 1006
    assert b"maximum" in pb.lib().b200_error_string(1006)
    assert ctx.launch_count() == launches

"""The caching pool on a real device: the behaviour the reference pins for its own
pool (test/cuda_memory_pool_test.cc: same pointers come back, round-up to the
size class, out-of-memory -> release the cache -> retry), restated with a soft
capacity so that the shared GPU's real memory is never exhausted."""
import pytest

import primitiv_b200 as pb

pytestmark = pytest.mark.gpu


@pytest.fixture()
def own_ctx():
    c = pb.Context(0)
    yield c
    c.close()


def test_blocks_are_reused_and_aligned(own_ctx):
    c = own_ctx
    p1, got1 = c.pool_alloc(1000)
    p2, got2 = c.pool_alloc(1000)
    assert got1 == 1024 and got2 == 1024 and p1 != p2
    assert p1 % 256 == 0 and p2 % 256 == 0
    c.pool_free(p1)
    c.pool_free(p2)
    q1, _ = c.pool_alloc(1024)   # same class: the cached blocks come back, last freed first
    q2, _ = c.pool_alloc(900)
    assert {q1, q2} == {p1, p2}
    s = c.pool_stats()
    assert s["mallocs"] == 2 and s["hits"] == 2 and s["in_use"] == 2048 and s["cached"] == 0
    c.pool_free(q1)
    c.pool_free(q2)
    assert c.pool_stats()["cached"] == 2048


def test_round_up_is_at_most_a_quarter(own_ctx):
    p, got = own_ctx.pool_alloc((1 << 20) + 1)
    assert got == (1 << 20) + (1 << 18)
    own_ctx.pool_free(p)


def test_out_of_memory_releases_cache_then_retries(own_ctx):
    c = own_ctx
    c.pool_set_limit(3 << 20)
    a, _ = c.pool_alloc(1 << 20)
    b, _ = c.pool_alloc(1 << 20)
    c.pool_free(a)
    c.pool_free(b)                      # 2 MiB cached, 0 in use
    big, got = c.pool_alloc(2 << 20)    # 2 cached + 2 new > limit -> cache is released, retry fits
    assert got == 2 << 20
    s = c.pool_stats()
    assert s["cached"] == 0 and s["in_use"] == 2 << 20
    with pytest.raises(pb.B200Error) as e:   # 2 in use + 2 > 3: fails even after the release
        c.pool_alloc(2 << 20)
    assert e.value.code == 1003
    c.pool_free(big)
    c.pool_set_limit(0)
    p, _ = c.pool_alloc(2 << 20)        # the context is still usable afterwards
    c.pool_free(p)


def test_free_of_unknown_pointer_is_an_error(own_ctx):
    with pytest.raises(pb.B200Error):
        own_ctx.pool_free(0x1000)


def test_invalid_device_id_is_rejected():
    with pytest.raises(pb.B200Error):
        pb.Context(9999)


def test_bounded_wait_reports_and_context_survives(own_ctx):
    """A device-side wait that runs out is reported through the status word, not by a fault."""
    import numpy as np
    import torch
    c = own_ctx
    assert c.status_poll() == 0
    c.op("b200_selftest_wait_timeout", None)
    assert c.status_poll() == 1004          # B200_ERR_KERNEL_TIMEOUT, read once ...
    assert c.status_poll() == 0             # ... and cleared
    # the same context still computes
    a = torch.eye(64, device="cuda").flatten()
    b = torch.arange(64 * 64, device="cuda", dtype=torch.float32)
    y = torch.empty(64 * 64, device="cuda")
    c.matmul_fw(pb.MODE_TF32, a.data_ptr(), b.data_ptr(), y.data_ptr(), 64, 64, 64, 1, 1)
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), b.cpu().numpy())


# ---- guard bands (debugging aid for out-of-bounds writes) ---------------------------------------
# Every write below stays inside memory the pool itself took from the driver (the bands are part of
# its allocations), so nothing here can fault.

def test_guard_bands_catch_a_write_past_either_end_and_rearm(own_ctx):
    c = own_ctx
    c.pool_set_guard(200)                       # rounded up to 256 bytes on each side
    p, got = c.pool_alloc(1000)
    q, _ = c.pool_alloc(5000)
    assert got == 1024 and p % 256 == 0
    fill = lambda ptr, n: c.op("b200_fill", pb.MODE_FP32_3XTF32, ptr, n, 1.0, None)
    fill(p, 256)                                # exactly the block
    assert c.pool_check_guards() == (0, None, 0)
    fill(p, 256 + 3)                            # three floats past the end
    assert c.pool_check_guards() == (1, p, 2)
    assert c.pool_check_guards() == (0, None, 0)    # the check restored the pattern
    fill(q - 8, 2)                              # two floats in front of the other block
    fill(p - 4, 1)
    n, first, side = c.pool_check_guards()
    assert n == 2 and first == min(p, q) and side == 1
    c.pool_free(p)
    fill(p + 1024, 1)                           # cached blocks are watched too
    assert c.pool_check_guards() == (1, p, 2)
    with pytest.raises(pb.B200Error):           # not while blocks are handed out
        c.pool_set_guard(0)
    c.pool_free(q)
    c.pool_set_guard(0)
    r, _ = c.pool_alloc(1000)
    assert c.pool_check_guards() == (0, None, 0)
    c.pool_free(r)


@pytest.mark.parametrize("mode", ["3XTF32", "TF32", "FP16", "3XFP16"])
def test_products_leave_the_guard_bands_alone(own_ctx, mode):
    """Ragged and skinny shapes through every kernel family, outputs and scratch in guarded pool
    blocks of exactly the needed size: no epilogue, pack or split-K kernel stores outside."""
    import numpy as np
    c = own_ctx
    m = {"3XTF32": pb.MODE_FP32_3XTF32, "TF32": pb.MODE_TF32, "FP16": pb.MODE_FP16, "3XFP16": pb.MODE_FP32_3XFP16}[mode]
    es = 2 if mode == "FP16" else 4
    c.pool_set_guard(256)
    rng = np.random.default_rng(5)
    shapes = [(130, 70, 50, 1, 3), (257, 129, 65, 3, 3), (10, 1024, 1, 1, 520), (64, 64, 64, 2, 1), (512, 264, 1000, 1, 1),
              (33, 4100, 17, 1, 2), (1, 1, 1, 1, 1), (128, 2048, 8, 1, 40)]
    for di, dj, dk, ba, bb in shapes:
        bs = max(ba, bb)
        sizes = [di * dj * ba, dj * dk * bb, di * dk * bs, di * dk * bs, di * dj * ba, dj * dk * bb]   # a b y gy ga gb
        ptrs = [c.pool_alloc(n * es)[0] for n in sizes]
        for ptr, n in zip(ptrs, sizes):
            v = rng.standard_normal(n).astype(np.float32)
            c.op("b200_upload", m, v.ctypes.data, ptr, n, None)
        a, b, y, gy, ga, gb = ptrs
        for policy in (0, 1, 2):
            c.set_path_policy(policy)
            c.matmul_fw(m, a, b, y, di, dj, dk, ba, bb)
            c.matmul_bw(m, a, b, gy, ga, gb, di, dj, dk, ba, bb)
        c.set_path_policy(0)
        assert c.pool_check_guards() == (0, None, 0), (di, dj, dk, ba, bb)
        for ptr in ptrs:
            c.pool_free(ptr)
    assert c.pool_check_guards() == (0, None, 0)
    c.pool_release_cached()
    c.pool_set_guard(0)


@pytest.mark.parametrize("n", [(8 << 20) // 4, (40 << 20) // 4 + 12345, (8 << 20) // 4 - 1])
@pytest.mark.parametrize("half", [False, True])
def test_large_uploads_arrive_intact(own_ctx, n, half):
    """Host arrays of 8 MiB and more are staged by several threads half a ring at a time; smaller ones
    slot by slot.  Whatever the route, interleaved with small uploads, the values arrive in order."""
    import numpy as np
    c = own_ctx
    m = pb.MODE_FP16 if half else pb.MODE_FP32_3XTF32
    rng = np.random.default_rng(n)
    big = rng.integers(-1000, 1000, n).astype(np.float32)      # exact in half precision too
    small = rng.integers(-1000, 1000, 300000).astype(np.float32)
    es = 2 if half else 4
    p_small, _ = c.pool_alloc(small.size * es)
    p_big, _ = c.pool_alloc(n * es)
    p_small2, _ = c.pool_alloc(small.size * es)
    c.op("b200_upload", m, small.ctypes.data, p_small, small.size, None)
    c.op("b200_upload", m, big.ctypes.data, p_big, n, None)
    c.op("b200_upload", m, small.ctypes.data, p_small2, small.size, None)
    for ptr, want in ((p_big, big), (p_small, small), (p_small2, small)):
        got = np.empty_like(want)
        c.op("b200_download", m, ptr, got.ctypes.data, want.size, None)
        assert np.array_equal(got, want)
        c.pool_free(ptr)

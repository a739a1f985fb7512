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

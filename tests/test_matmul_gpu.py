"""GPU parity tests of the hot path, through the C ABI, against the CPU oracle.

Tolerances: fp32 3xTF32 mode <= 1e-5 normwise relative error against the fp64
oracle; TF32 and fp16 modes <= 2e-3.  The reference's own known-answer vectors
are held to the reference's ULP bounds (4 ULP fp32; the CUDA16 bounds for fp16)."""
import json
import os

import numpy as np
import pytest
import torch

import oracle_lib as ol
import primitiv_b200 as pb
from gpu_util import MODES, TOL, dev, host, matmul_bw, matmul_fw

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

with open(os.path.join(GOLDEN, "matmul_known_answers.json")) as _f:
    KNOWN = json.load(_f)["cases"]


def _dims(case):
    di, dj = case["a_shape"]
    return di, dj, case["b_shape"][1], case["a_batch"], case["b_batch"]


@pytest.mark.parametrize("policy", [0, 2], ids=["auto", "tensorcore"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("case", KNOWN, ids=lambda c: c["name"])
def test_reference_known_answers(ctx, case, mode, policy):
    """test/tensor_forward_test.cc:1798-1905, test/tensor_backward_test.cc:1599-1668,
    test/operator_impl_test.cc:1132-1144 of the reference, on this backend."""
    m = MODES[mode]
    di, dj, dk, ba, bb = _dims(case)
    ulps = case["ulps_fp16"] if mode == "fp16" else case["ulps"]
    a, b = np.array(case["a"], np.float32), np.array(case["b"], np.float32)
    ctx.set_path_policy(policy)
    try:
        if case["kind"] == "fw":
            y = matmul_fw(ctx, m, a, b, di, dj, dk, ba, bb)
            assert ol.ulp_diff(y, np.array(case["y"], np.float32)).max() <= ulps
        else:
            gy = np.array(case["gy"], np.float32)
            ga0 = np.full(di * dj * ba, case["prefill"], np.float32)
            gb0 = np.full(dj * dk * bb, case["prefill"], np.float32)
            ga, gb = matmul_bw(ctx, m, a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
            assert ol.ulp_diff(ga, np.array(case["ga"], np.float32)).max() <= ulps
            assert ol.ulp_diff(gb, np.array(case["gb"], np.float32)).max() <= ulps
    finally:
        ctx.set_path_policy(0)


def _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb, prefill=0.5):
    m = MODES[mode]
    if mode == "fp16":  # the oracle sees the values the device stores
        a, b, gy = ol.round_to_half(a), ol.round_to_half(b), ol.round_to_half(gy)
    ga0 = np.full(di * dj * ba, prefill, np.float32)
    gb0 = np.full(dj * dk * bb, prefill, np.float32)
    y = matmul_fw(ctx, m, a, b, di, dj, dk, ba, bb)
    ga, gb = matmul_bw(ctx, m, a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
    y64 = ol.fw_f64(a, b, di, dj, dk, ba, bb)
    ga64, gb64 = ol.bw_f64(a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
    errs = (ol.rel_err(y, y64), ol.rel_err(ga, ga64), ol.rel_err(gb, gb64))
    assert max(errs) <= TOL[mode], errs
    return y, ga, gb


_REF = np.load(os.path.join(GOLDEN, "matmul_ref_naive_cases.npz"))


@pytest.mark.parametrize("policy", [0, 2], ids=["auto", "tensorcore"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("idx", range(len(_REF["cases"])))
def test_against_reference_naive_fixtures(ctx, idx, mode, policy):
    di, dj, dk, ba, bb = [int(v) for v in _REF["cases"][idx]]
    a, b, gy = _REF["a_%d" % idx], _REF["b_%d" % idx], _REF["gy_%d" % idx]
    ctx.set_path_policy(policy)
    try:
        y, ga, gb = _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb)
    finally:
        ctx.set_path_policy(0)
    if mode in ("3xtf32", "3xfp16"):  # directly against what the reference's Naive device produced
        for got, key in ((y, "y"), (ga, "ga"), (gb, "gb")):
            want = _REF["%s_%d" % (key, idx)]
            assert np.linalg.norm(got - want) <= 1e-5 * np.linalg.norm(want)


# (di, dj, dk, ba, bb): every broadcast combination, tile-edge and ragged extents, a long
# contraction, a batch-summed gradient with many batches.  Sized for the CPU oracle.
SHAPES = [
    (512, 384, 256, 1, 4), (384, 512, 320, 4, 4), (256, 768, 128, 3, 1), (1024, 1024, 1024, 1, 1),
    (260, 132, 72, 2, 2), (128, 128, 128, 1, 1), (129, 257, 65, 1, 3), (130, 36, 520, 5, 1),
    (64, 4096, 64, 1, 2), (256, 256, 64, 1, 16), (4096, 512, 64, 1, 1), (96, 200, 40, 7, 1),
    (100, 1000, 8, 1, 64),
]


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_random_shapes_against_fp64_oracle(ctx, shape, mode):
    di, dj, dk, ba, bb = shape
    rng = np.random.default_rng(hash(shape) % (2 ** 32))
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * max(ba, bb)).astype(np.float32)
    _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb)


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_fp32_mode_with_tf32_planes_throughout(ctx, shape):
    """The fp32 mode runs its two correction passes on bf16 planes by default (every other test of
    mode 3xtf32 in this file); b200_set_correction_policy(1) keeps all three passes on TF32 planes.
    Same shapes, same 1e-5 bound, tensor-core kernel forced."""
    di, dj, dk, ba, bb = shape
    rng = np.random.default_rng(hash(shape) % (2 ** 32))
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * max(ba, bb)).astype(np.float32)
    ctx.set_correction_policy(1)
    ctx.set_path_policy(2)
    try:
        _check_all(ctx, "3xtf32", a, b, gy, di, dj, dk, ba, bb)
    finally:
        ctx.set_correction_policy(0)
        ctx.set_path_policy(0)


def test_correction_policies_per_product_error(ctx):
    """What the two policies differ in: with positive operands (no cancellation) and a contraction of
    only 8 terms, every element's relative error is bounded by the per-product error of the
    split: about 2^-19 with bf16 correction operands, 2^-22 with TF32 ones."""
    di, dj, dk = 256, 8, 256
    rng = np.random.default_rng(21)
    a = rng.uniform(1, 2, di * dj).astype(np.float32)
    b = rng.uniform(1, 2, dj * dk).astype(np.float32)
    y64 = ol.fw_f64(a, b, di, dj, dk, 1, 1)
    worst = {}
    ctx.set_path_policy(2)
    try:
        for policy in (0, 1):
            ctx.set_correction_policy(policy)
            y = matmul_fw(ctx, pb.MODE_FP32_3XTF32, a, b, di, dj, dk, 1, 1)
            worst[policy] = float(np.max(np.abs(y - y64) / np.abs(y64)))
    finally:
        ctx.set_correction_policy(0)
        ctx.set_path_policy(0)
    assert worst[0] <= 4e-6 and worst[1] <= 1e-6, worst
    assert worst[1] < worst[0], worst


def _cuda(x):
    return torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda()


@pytest.mark.parametrize("di", [384, 1664])
@pytest.mark.parametrize("batches", [(1, 4), (4, 4), (4, 1), (1, 1)], ids=lambda b: "ba%d_bb%d" % b)
def test_operand_cache_shares_planes_between_forward_and_backward(ctx, batches, di):
    """With the cache on, a step packs each of a, b, gy once in the array's own layout (three
    misses) and the second use of each finds those planes (three hits).  b's second use is as an
    MN-major B operand, whose TF32 plane the kernel reads slowly: with few output rows (di = 384)
    that product still takes all of b's cached planes (transposing b would cost more than the slower
    main loop; a b of under a million elements does the same whatever di), with many (di = 1664, b of
    a million elements) it takes the cached bf16 planes and transposes the TF32 plane alone into
    scratch.  The results are the oracle's."""
    dj, dk = (256, 512) if di == 384 else (1024, 1024)
    ba, bb = batches
    bs = max(ba, bb)
    rng = np.random.default_rng(31 + ba * 10 + bb)
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * bs).astype(np.float32)
    da, db, dgy = _cuda(a), _cuda(b), _cuda(gy)
    y = torch.empty(di * dk * bs, device="cuda")
    ga, gb = torch.full((di * dj * ba,), 0.5, device="cuda"), torch.full((dj * dk * bb,), 0.5, device="cuda")
    M = pb.MODE_FP32_3XTF32
    ctx.set_path_policy(2)
    ctx.operand_cache_enable(1 << 30)
    try:
        s0 = ctx.operand_cache_stats()
        ctx.matmul_fw(M, da.data_ptr(), db.data_ptr(), y.data_ptr(), di, dj, dk, ba, bb)
        ctx.matmul_bw(M, da.data_ptr(), db.data_ptr(), dgy.data_ptr(), ga.data_ptr(), gb.data_ptr(), di, dj, dk, ba, bb)
        torch.cuda.synchronize()
        s1 = ctx.operand_cache_stats()
        assert (s1["misses"] - s0["misses"], s1["hits"] - s0["hits"]) == (3, 3), (s0, s1)
        assert s1["entries"] == 3 and s1["bytes"] >= 2 * 4 * (a.size + b.size + gy.size)
    finally:
        ctx.operand_cache_enable(0)
        ctx.set_path_policy(0)
    assert ctx.operand_cache_stats()["entries"] == 0
    half = np.full
    ga64, gb64 = ol.bw_f64(a, b, gy, half(a.size, 0.5, np.float32), half(b.size, 0.5, np.float32), di, dj, dk, ba, bb)
    assert ol.rel_err(y.cpu().numpy(), ol.fw_f64(a, b, di, dj, dk, ba, bb)) <= 1e-5
    assert ol.rel_err(ga.cpu().numpy(), ga64) <= 1e-5 and ol.rel_err(gb.cpu().numpy(), gb64) <= 1e-5


def test_operand_cache_forgets_what_is_written(ctx):
    """Planes go stale in three ways, and each is handled: the caller writes an operand and says so
    (invalidate), a product of this library overwrites an array that was an operand before, and a
    block goes back to the pool."""
    n = 256
    rng = np.random.default_rng(41)
    a, b, c, a2 = (rng.uniform(-1, 1, n * n).astype(np.float32) for _ in range(4))
    da, db, dc = _cuda(a), _cuda(b), _cuda(c)
    y, z = torch.empty(n * n, device="cuda"), torch.empty(n * n, device="cuda")
    M = pb.MODE_FP32_3XTF32
    fw = lambda p, q, r: ctx.matmul_fw(M, p.data_ptr(), q.data_ptr(), r.data_ptr(), n, n, n, 1, 1)
    ref = lambda p, q: ol.fw_f64(p, q, n, n, n, 1, 1)
    ctx.set_path_policy(2)
    ctx.operand_cache_enable(1 << 30)
    try:
        fw(da, db, y)                                   # y = a.b, planes of a and b kept
        fw(y, dc, z)                                    # z = y.c, planes of y kept
        da.copy_(_cuda(a2))                             # the caller rewrites a ...
        ctx.operand_cache_invalidate(da.data_ptr(), da.numel() * 4)   # ... and says so
        fw(da, db, y)                                   # y = a2.b: writes y, so y's planes are dropped here
        fw(y, dc, z)
        torch.cuda.synchronize()
        y2 = ref(a2, b)
        assert ol.rel_err(y.cpu().numpy(), y2) <= 1e-5
        assert ol.rel_err(z.cpu().numpy(), ref(y2.astype(np.float32), c)) <= 1e-5
        # a pool block used as an operand, freed, handed out again with other contents
        p1, _ = ctx.pool_alloc(n * n * 4)
        ctx.op("b200_upload", M, a.ctypes.data, p1, n * n, None)
        ctx.matmul_fw(M, p1, db.data_ptr(), y.data_ptr(), n, n, n, 1, 1)
        ctx.pool_free(p1)
        p2, _ = ctx.pool_alloc(n * n * 4)
        assert p2 == p1                                 # same block, as the pool promises
        ctx.op("b200_upload", M, c.ctypes.data, p2, n * n, None)
        ctx.matmul_fw(M, p2, db.data_ptr(), y.data_ptr(), n, n, n, 1, 1)
        torch.cuda.synchronize()
        ctx.pool_free(p2)
        assert ol.rel_err(y.cpu().numpy(), ref(c, b)) <= 1e-5
    finally:
        ctx.operand_cache_enable(0)
        ctx.set_path_policy(0)


def test_backward_call_packs_the_upstream_gradient_once(ctx):
    """Without the cache: inside one b200_matmul_bw call gy still serves both products from one set of
    planes (one hit), and nothing is kept afterwards."""
    di = dj = dk = 256
    rng = np.random.default_rng(43)
    a, b, gy = (rng.uniform(-1, 1, di * dj).astype(np.float32) for _ in range(3))
    ctx.set_path_policy(2)
    try:
        s0 = ctx.operand_cache_stats()
        ga, gb = matmul_bw(ctx, pb.MODE_FP32_3XTF32, a, b, gy, np.zeros(di * dj, np.float32), np.zeros(dj * dk, np.float32),
                           di, dj, dk, 1, 1)
        s1 = ctx.operand_cache_stats()
    finally:
        ctx.set_path_policy(0)
    # gy and a are packed flat (two misses) and gy is found again by the second product (one hit);
    # b is an MN-major B operand in ga = gy . b^T and is repacked for that product alone
    assert s1["hits"] - s0["hits"] == 1 and s1["misses"] - s0["misses"] == 2 and s1["entries"] == 0, (s0, s1)
    ga64, gb64 = ol.bw_f64(a, b, gy, np.zeros(di * dj, np.float32), np.zeros(dj * dk, np.float32), di, dj, dk, 1, 1)
    assert ol.rel_err(ga, ga64) <= 1e-5 and ol.rel_err(gb, gb64) <= 1e-5


@pytest.mark.parametrize("dependent", [True, False], ids=["pdl", "no_pdl"])
@pytest.mark.parametrize("mode", list(MODES))
def test_launch_policy_does_not_change_results(ctx, mode, dependent):
    """Launches issued by the worker thread, with and without programmatic dependent launch: the
    same bits as launches from the calling thread, on a chain of products that reuses buffers
    (forward, both gradients, a second backward call that accumulates, split-k and skinny shapes)."""
    shapes = [(384, 256, 512, 1, 4), (260, 132, 72, 2, 2), (10, 1024, 1, 1, 4096), (4096, 512, 64, 1, 1)]
    results = {}
    for queued in (False, True):
        ctx.set_async_launch(queued)
        ctx.set_dependent_launch(dependent if queued else True)
        try:
            outs = []
            for di, dj, dk, ba, bb in shapes:
                rng = np.random.default_rng(di + dj)
                a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
                b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
                gy = rng.standard_normal(di * dk * max(ba, bb)).astype(np.float32)
                y, ga, gb = _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb)
                outs += [y, ga, gb]
            results[queued] = outs
        finally:
            ctx.set_async_launch(False)
            ctx.set_dependent_launch(True)
    for x, z in zip(results[False], results[True]):
        assert np.array_equal(x, z)


@pytest.mark.parametrize("mode", list(MODES))
def test_plumbing_workload(ctx, mode):
    """W {256,256} broadcast, X {256,64}x16, gy N(0,1), all from one mt19937(0); gradients pre-filled 0.5."""
    c = ol.config1_inputs()
    args = (c["di"], c["dj"], c["dk"], c["ba"], c["bb"])
    y, ga, gb = _check_all(ctx, mode, c["a"], c["b"], c["gy"], *args, prefill=0.5)
    if mode in ("3xtf32", "3xfp16") and ol.have_ref():
        y_ref, _ = ol.ref_fw(c["a"], c["b"], *args)
        ga_ref, gb_ref, _ = ol.ref_bw(c["a"], c["b"], c["gy"], c["ga0"], c["gb0"], *args)
        for got, want in ((y, y_ref), (ga, ga_ref), (gb, gb_ref)):
            assert np.linalg.norm(got - want) <= 1e-5 * np.linalg.norm(want)


def test_accumulation_really_accumulates(ctx):
    """Two backward calls into the same gradient add twice (beta = 1), and the forward overwrites."""
    di, dj, dk, ba, bb = 192, 160, 96, 1, 3
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, di * dj).astype(np.float32)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * bb).astype(np.float32)
    m = pb.MODE_FP32_3XTF32
    da, db, dgy = [torch.from_numpy(x).cuda() for x in (a, b, gy)]
    ga = torch.full((di * dj,), 0.25, device="cuda")
    gb = torch.full((dj * dk * bb,), -1.0, device="cuda")
    for _ in range(2):
        ctx.matmul_bw(m, da.data_ptr(), db.data_ptr(), dgy.data_ptr(), ga.data_ptr(), gb.data_ptr(),
                      di, dj, dk, ba, bb)
    z = np.zeros
    ga64, gb64 = ol.bw_f64(a, b, gy, z(di * dj, np.float32), z(dj * dk * bb, np.float32), di, dj, dk, ba, bb)
    assert ol.rel_err(ga.cpu().numpy(), 0.25 + 2 * ga64) < 1e-5
    assert ol.rel_err(gb.cpu().numpy(), -1.0 + 2 * gb64) < 1e-5
    y = torch.full((di * dk * bb,), 1e30, device="cuda")  # must be overwritten, not added to
    ctx.matmul_fw(m, da.data_ptr(), db.data_ptr(), y.data_ptr(), di, dj, dk, ba, bb)
    assert ol.rel_err(y.cpu().numpy(), ol.fw_f64(a, b, di, dj, dk, ba, bb)) < 1e-5


def test_null_gradient_skips_that_product(ctx):
    di, dj, dk = 64, 64, 64
    rng = np.random.default_rng(6)
    a, b, gy = [torch.from_numpy(rng.standard_normal(di * dj).astype(np.float32)).cuda() for _ in range(3)]
    ga = torch.zeros(di * dj, device="cuda")
    ctx.matmul_bw(pb.MODE_TF32, a.data_ptr(), b.data_ptr(), gy.data_ptr(), ga.data_ptr(), None, di, dj, dk, 1, 1)
    torch.cuda.synchronize()
    assert float(ga.abs().sum()) > 0


@pytest.mark.parametrize("mode", list(MODES))
def test_bitwise_deterministic(ctx, mode):
    """No atomics anywhere on the path: the batch-summed gradient is the same bits every run."""
    di, dj, dk, ba, bb = 256, 192, 128, 6, 1
    rng = np.random.default_rng(7)
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * ba).astype(np.float32)
    z = np.zeros
    runs = [matmul_bw(ctx, MODES[mode], a, b, gy, z(di * dj * ba, np.float32), z(dj * dk, np.float32),
                      di, dj, dk, ba, bb) for _ in range(3)]
    for ga, gb in runs[1:]:
        assert np.array_equal(ga, runs[0][0]) and np.array_equal(gb, runs[0][1])


def test_invalid_arguments_are_rejected(ctx):
    x = torch.zeros(64, device="cuda")
    p = x.data_ptr()
    with pytest.raises(pb.B200Error):  # incompatible batches (Shape::has_compatible_batch)
        ctx.matmul_fw(pb.MODE_TF32, p, p, p, 2, 2, 2, 2, 3)
    with pytest.raises(pb.B200Error):
        ctx.matmul_fw(7, p, p, p, 2, 2, 2, 1, 1)
    with pytest.raises(pb.B200Error):
        ctx.matmul_fw(pb.MODE_TF32, None, p, p, 2, 2, 2, 1, 1)


def test_host_buffer_entry_points(ctx):
    c = ol.config1_inputs()
    args = (c["di"], c["dj"], c["dk"], c["ba"], c["bb"])
    y = np.empty(c["di"] * c["dk"] * c["bb"], np.float32)
    ctx.matmul_fw_host(pb.MODE_FP32_3XTF32, c["a"].ctypes.data, c["b"].ctypes.data, y.ctypes.data, *args)
    assert ol.rel_err(y, ol.fw_f64(c["a"], c["b"], *args)) < 1e-5
    ga, gb = c["ga0"].copy(), c["gb0"].copy()
    ctx.matmul_bw_host(pb.MODE_FP32_3XTF32, c["a"].ctypes.data, c["b"].ctypes.data, c["gy"].ctypes.data,
                       ga.ctypes.data, gb.ctypes.data, *args)
    ga64, gb64 = ol.bw_f64(c["a"], c["b"], c["gy"], c["ga0"], c["gb0"], *args)
    assert ol.rel_err(ga, ga64) < 1e-5 and ol.rel_err(gb, gb64) < 1e-5


@pytest.mark.parametrize("batches", [(6, 6), (1, 6), (6, 1)], ids=lambda b: "ba%d_bb%d" % b)
@pytest.mark.parametrize("mode", ["3xtf32", "fp16"])
def test_host_buffer_entry_points_pipeline_over_batch_chunks(ctx, mode, batches):
    """Large enough that the host-buffer calls split the batch into several ragged chunks
    (6 items in 4 chunks) and overlap upload, products and download; gradients pre-filled 0.5,
    so a chunk added twice, skipped, or downloaded before its product finished would show."""
    di = dj = dk = 512
    ba, bb = batches
    bs = max(ba, bb)
    rng = np.random.default_rng(100 + 10 * ba + bb)
    half = mode == "fp16"
    dt = np.float16 if half else np.float32
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32).astype(dt)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32).astype(dt)
    gy = rng.standard_normal(di * dk * bs).astype(np.float32).astype(dt)
    a32, b32, gy32 = (x.astype(np.float32) for x in (a, b, gy))
    args = (di, dj, dk, ba, bb)
    tol = 2e-3 if half else 1e-5
    y = np.full(di * dk * bs, 7.0, dt)
    ctx.matmul_fw_host(MODES[mode], a.ctypes.data, b.ctypes.data, y.ctypes.data, *args)
    assert ol.rel_err(y.astype(np.float32), ol.fw_f64(a32, b32, *args)) < tol
    ga, gb = np.full(di * dj * ba, 0.5, dt), np.full(dj * dk * bb, 0.5, dt)
    ctx.matmul_bw_host(MODES[mode], a.ctypes.data, b.ctypes.data, gy.ctypes.data, ga.ctypes.data, gb.ctypes.data, *args)
    ga64, gb64 = ol.bw_f64(a32, b32, gy32, np.full(di * dj * ba, 0.5, np.float32),
                           np.full(dj * dk * bb, 0.5, np.float32), *args)
    assert ol.rel_err(ga.astype(np.float32), ga64) < tol and ol.rel_err(gb.astype(np.float32), gb64) < tol


@pytest.mark.parametrize("accumulate", [True, False], ids=["prefill_0.5", "known_zero"])
@pytest.mark.parametrize("batches", [(6, 6), (1, 6), (6, 1), (1, 1)], ids=lambda b: "ba%d_bb%d" % b)
@pytest.mark.parametrize("mode", ["3xtf32", "fp16"])
def test_fused_host_entry_point(ctx, mode, batches, accumulate):
    """b200_matmul_fw_bw_host: y, ga and gb of one call against the fp64 oracle.  With the
    accumulate flags set the gradients start from 0.5 (the reference's `+=`); with them clear the
    host arrays hold a poison value that must not reach the result (the gradient is declared to
    start from zeros and is never uploaded)."""
    di = dj = dk = 512
    ba, bb = batches
    bs = max(ba, bb)
    rng = np.random.default_rng(200 + 10 * ba + bb)
    half = mode == "fp16"
    dt = np.float16 if half else np.float32
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32).astype(dt)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32).astype(dt)
    gy = rng.standard_normal(di * dk * bs).astype(np.float32).astype(dt)
    a32, b32, gy32 = (x.astype(np.float32) for x in (a, b, gy))
    args = (di, dj, dk, ba, bb)
    tol = 2e-3 if half else 1e-5
    start = 0.5 if accumulate else 0.0
    y = np.full(di * dk * bs, 7.0, dt)
    ga = np.full(di * dj * ba, 0.5 if accumulate else 1e4, dt)
    gb = np.full(dj * dk * bb, 0.5 if accumulate else 1e4, dt)
    ctx.matmul_fw_bw_host(MODES[mode], a.ctypes.data, b.ctypes.data, gy.ctypes.data, y.ctypes.data,
                          ga.ctypes.data, gb.ctypes.data, *args, accumulate_a=accumulate, accumulate_b=accumulate)
    ga64, gb64 = ol.bw_f64(a32, b32, gy32, np.full(di * dj * ba, start, np.float32),
                           np.full(dj * dk * bb, start, np.float32), *args)
    assert ol.rel_err(y.astype(np.float32), ol.fw_f64(a32, b32, *args)) < tol
    assert ol.rel_err(ga.astype(np.float32), ga64) < tol and ol.rel_err(gb.astype(np.float32), gb64) < tol


@pytest.mark.parametrize("accumulate", [True, False], ids=["prefill_0.5", "known_zero"])
@pytest.mark.parametrize("mode", ["3xtf32", "fp16"])
@pytest.mark.parametrize("outputs", ["all", "no_y", "no_gb", "no_ga"])
def test_fused_host_entry_point_large_items(ctx, mode, accumulate, outputs):
    """Items large enough that the call's pipeline runs one batch item per chunk (8 MiB and more per
    operand item), pinned host buffers: same results as the oracle, whichever outputs are asked for."""
    di, dj, dk, ba, bb = 1024, 1024, 2048, 3, 3
    rng = np.random.default_rng(77)
    half = mode == "fp16"
    dt = np.float16 if half else np.float32
    mk = lambda n, normal=False: (rng.standard_normal(n) if normal else rng.uniform(-1, 1, n)).astype(np.float32).astype(dt)
    a, b, gy = mk(di * dj * ba), mk(dj * dk * bb), mk(di * dk * bb, True)
    a32, b32, gy32 = (x.astype(np.float32) for x in (a, b, gy))
    pin = lambda x: torch.from_numpy(x.copy()).pin_memory()
    ta, tb, tgy = pin(a), pin(b), pin(gy)
    ty = pin(np.full(di * dk * bb, 7.0, dt))
    tga = pin(np.full(di * dj * ba, 0.5 if accumulate else 1e4, dt))
    tgb = pin(np.full(dj * dk * bb, 0.5 if accumulate else 1e4, dt))
    P = lambda t: t.data_ptr()
    ctx.matmul_fw_bw_host(MODES[mode], P(ta), P(tb), P(tgy), None if outputs == "no_y" else P(ty),
                          None if outputs == "no_ga" else P(tga), None if outputs == "no_gb" else P(tgb),
                          di, dj, dk, ba, bb, accumulate_a=accumulate, accumulate_b=accumulate)
    tol = 2e-3 if half else 1e-5
    start = 0.5 if accumulate else 0.0
    ga64, gb64 = ol.bw_f64(a32, b32, gy32, np.full(di * dj * ba, start, np.float32), np.full(dj * dk * bb, start, np.float32),
                           di, dj, dk, ba, bb)
    if outputs != "no_y":
        assert ol.rel_err(ty.numpy().astype(np.float32), ol.fw_f64(a32, b32, di, dj, dk, ba, bb)) < tol
    if outputs != "no_ga":
        assert ol.rel_err(tga.numpy().astype(np.float32), ga64) < tol
    if outputs != "no_gb":
        assert ol.rel_err(tgb.numpy().astype(np.float32), gb64) < tol


def test_fused_host_entry_point_optional_outputs(ctx):
    """Any of y / ga / gb may be left out; the plumbing workload with pinned host buffers."""
    c = ol.config1_inputs()
    args = (c["di"], c["dj"], c["dk"], c["ba"], c["bb"])
    M = pb.MODE_FP32_3XTF32
    pin = lambda x: torch.from_numpy(x.copy()).pin_memory()
    a, b, gy = pin(c["a"]), pin(c["b"]), pin(c["gy"])
    y = torch.empty(c["di"] * c["dk"] * c["bb"]).pin_memory()
    ga, gb = pin(c["ga0"]), pin(c["gb0"])
    P = lambda t: t.data_ptr()
    ctx.matmul_fw_bw_host(M, P(a), P(b), None, P(y), None, None, *args)               # forward only
    assert ol.rel_err(y.numpy(), ol.fw_f64(c["a"], c["b"], *args)) < 1e-5
    ctx.matmul_fw_bw_host(M, P(a), P(b), P(gy), None, P(ga), None, *args)             # ga only, +=
    ctx.matmul_fw_bw_host(M, P(a), P(b), P(gy), None, None, P(gb), *args)             # gb only, +=
    ga64, gb64 = ol.bw_f64(c["a"], c["b"], c["gy"], c["ga0"], c["gb0"], *args)
    assert ol.rel_err(ga.numpy(), ga64) < 1e-5 and ol.rel_err(gb.numpy(), gb64) < 1e-5
    with pytest.raises(pb.B200Error):   # gradients asked for without an upstream gradient
        ctx.matmul_fw_bw_host(M, P(a), P(b), None, None, P(ga), None, *args)


# Few output tiles against a long contraction: the tensor-core path cuts k into slices for the
# idle SMs and adds the slices in a fixed order.  (di, dj, dk, ba, bb)
SPLIT_K_SHAPES = [
    (384, 320, 1, 1, 4096),    # gradient of a broadcast weight: 384 x 320 output, k = 4096 batch items
    (10, 1024, 1, 1, 8192),    # a 10-row weight (classifier layer): a few rows, long k
    (4096, 512, 1, 1, 64),     # recurrent step: gb is 512 x 64 with k = 4096
    (200, 136, 8, 1, 700),     # ragged extents, slices that do not divide k
]


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("shape", SPLIT_K_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_split_k_products(ctx, shape, mode):
    di, dj, dk, ba, bb = shape
    rng = np.random.default_rng(hash(shape) % (2 ** 32))
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * max(ba, bb)).astype(np.float32)
    if mode == "fp16":   # keep the batch-summed gradients inside half's range
        gy *= 0.05
    for policy in (0, 2):
        ctx.set_path_policy(policy)
        try:
            first = _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb)
            again = _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb)
        finally:
            ctx.set_path_policy(0)
        for x, y in zip(first, again):   # slices are added in a fixed order: same bits every run
            assert np.array_equal(x, y)


# Extents of 1 in every position (scalars, dot products, outer products, matrix-vector), alone
# and batched / broadcast: the shapes the reference's own small tests are made of.
DEGENERATE = [
    (1, 1, 1, 1, 1), (1, 1, 1, 4, 4), (1, 37, 1, 1, 3), (29, 1, 31, 3, 1), (1, 64, 40, 2, 2),
    (48, 64, 1, 1, 5), (1, 4096, 1, 1, 1), (8, 8, 8, 1, 300),
]


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("shape", DEGENERATE, ids=lambda s: "x".join(map(str, s)))
def test_degenerate_extents(ctx, shape, mode):
    di, dj, dk, ba, bb = shape
    rng = np.random.default_rng(hash(shape) % (2 ** 32))
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * max(ba, bb)).astype(np.float32)
    for policy in (0, 2):
        ctx.set_path_policy(policy)
        try:
            _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb)
        finally:
            ctx.set_path_policy(0)


def test_zero_extent_is_a_no_op(ctx):
    """An empty output launches nothing and touches nothing (the C ABI accepts what primitiv's
    Shape can never produce, so that callers need not special-case it)."""
    x = torch.full((16,), 3.0, device="cuda")
    before = ctx.launch_count()
    ctx.matmul_fw(pb.MODE_FP32_3XTF32, x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, 4, 4, 1, 1)
    ctx.matmul_bw(pb.MODE_FP32_3XTF32, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                  4, 4, 0, 1, 1)
    torch.cuda.synchronize()
    assert ctx.launch_count() == before and float(x.sum()) == 48.0


def test_3xfp16_rows_of_very_different_magnitude(ctx):
    """The fp16-pipe mode scales every operand row by its own power of two: rows (and columns)
    whose magnitudes differ by 2^60 each keep fp32-grade accuracy, measured per output row and per
    output column, not just over the whole matrix."""
    di, dj, dk = 192, 640, 160
    rng = np.random.default_rng(77)
    a = rng.uniform(-1, 1, (di, dj)) * np.exp2(rng.integers(-30, 31, (di, 1)))
    b = rng.uniform(-1, 1, (dj, dk)) * np.exp2(rng.integers(-30, 31, (1, dk)))
    a32 = np.ascontiguousarray(a.T, np.float32).ravel()      # column-major {di, dj}
    b32 = np.ascontiguousarray(b.T, np.float32).ravel()      # column-major {dj, dk}
    ctx.set_path_policy(2)
    try:
        y = matmul_fw(ctx, pb.MODE_FP32_3XFP16, a32, b32, di, dj, dk, 1, 1).reshape(dk, di).T
    finally:
        ctx.set_path_policy(0)
    want = a32.reshape(dj, di).T.astype(np.float64) @ b32.reshape(dk, dj).T.astype(np.float64)
    row_err = np.linalg.norm(y - want, axis=1) / np.linalg.norm(want, axis=1)
    col_err = np.linalg.norm(y - want, axis=0) / np.linalg.norm(want, axis=0)
    assert row_err.max() < 1e-5 and col_err.max() < 1e-5, (row_err.max(), col_err.max())


# One tiny extent against large ones (a 10-row classifier layer over a large minibatch and its two
# gradients): in the fp32-grade modes these go to the CUDA-core kernels of gemm_skinny.cu, which
# stream the large operand once and compute in plain fp32.  (di, dj, dk, ba, bb)
SKINNY_SHAPES = [
    (10, 1024, 1, 1, 8192),    # rows / reduce / outer with the layouts matmul_fw / matmul_bw produce
    (7, 1000, 1, 1, 9001),     # nothing divides anything
    (3, 64, 1, 1, 8193),       # the smallest staging width
    (16, 300, 1, 1, 8500),     # the largest tiny extent
]


@pytest.mark.parametrize("mode", ["3xtf32", "3xfp16"])
@pytest.mark.parametrize("shape", SKINNY_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_skinny_products_run_on_cuda_cores_in_fp32(ctx, shape, mode):
    di, dj, dk, ba, bb = shape
    rng = np.random.default_rng(hash(shape) % (2 ** 32))
    a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
    b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * max(ba, bb)).astype(np.float32)
    ctx.profile_read()
    ctx.profile_enable(True)
    try:
        y, ga, gb = _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb)
    finally:
        ctx.profile_enable(False)
    prof = ctx.profile_read()
    assert prof["gemm_tc"][1] == 0 and prof["pack"][1] == 0 and prof["gemm_simt"][1] == 3, prof
    # plain fp32 arithmetic: an order of magnitude inside the bound of the tensor-core modes
    y64 = ol.fw_f64(a, b, di, dj, dk, ba, bb)
    assert ol.rel_err(y, y64) <= 1e-6
    again = _check_all(ctx, mode, a, b, gy, di, dj, dk, ba, bb)
    for x, z in zip((y, ga, gb), again):   # fixed summation order: same bits every run
        assert np.array_equal(x, z)


@pytest.mark.parametrize("mode", list(MODES))
def test_skinny_kernels_forced_in_every_mode(ctx, mode):
    """force_path = 3 through b200_gemm: the three kernels in every storage type, overwrite and +=;
    a shape that is none of theirs is refused."""
    m_, k_, n_ = 10, 512, 4099
    rng = np.random.default_rng(11)
    w = rng.uniform(-1, 1, (k_, m_)).astype(np.float32)      # {m, k} column-major
    x = rng.uniform(-1, 1, (n_, k_)).astype(np.float32)      # {k, n} column-major
    gy = (0.05 * rng.standard_normal((n_, m_))).astype(np.float32)
    if mode == "fp16":
        w, x, gy = ol.round_to_half(w), ol.round_to_half(x), ol.round_to_half(gy)
    M = MODES[mode]
    dw, dx, dgy = dev(w, M), dev(x, M), dev(gy, M)
    for accumulate, fill in ((False, 3.0), (True, 0.25)):
        base = fill if accumulate else 0.0
        y = dev(np.full((n_, m_), fill, np.float32), M)
        gx = dev(np.full((n_, k_), fill, np.float32), M)
        ctx.gemm(M, 0, 0, dw.data_ptr(), dx.data_ptr(), y.data_ptr(), m_, n_, k_, accumulate=accumulate, force_path=3)
        ctx.gemm(M, 1, 0, dw.data_ptr(), dgy.data_ptr(), gx.data_ptr(), k_, n_, m_, accumulate=accumulate, force_path=3)
        torch.cuda.synchronize()
        assert ctx.status_poll() == 0
        tol = TOL[mode] if mode == "fp16" else 1e-6
        assert ol.rel_err(host(y).reshape(n_, m_), base + x.astype(np.float64) @ w.astype(np.float64)) <= tol
        assert ol.rel_err(host(gx).reshape(n_, k_), base + gy.astype(np.float64) @ w.astype(np.float64).T) <= tol
        # reduce: C {m, n2} (+)= A {m, k2} . B {n2, k2}^T over a long k2
        n2, k2 = 300, 9001
        a2 = (0.05 * rng.standard_normal((k2, m_))).astype(np.float32)
        b2 = rng.uniform(-1, 1, (k2, n2)).astype(np.float32)
        if mode == "fp16":
            a2, b2 = ol.round_to_half(a2), ol.round_to_half(b2)
        c2 = dev(np.full((n2, m_), fill, np.float32), M)
        da2, db2 = dev(a2, M), dev(b2, M)
        ctx.gemm(M, 0, 1, da2.data_ptr(), db2.data_ptr(), c2.data_ptr(), m_, n2, k2, accumulate=accumulate, force_path=3)
        torch.cuda.synchronize()
        assert ctx.status_poll() == 0
        assert ol.rel_err(host(c2).reshape(n2, m_), base + b2.astype(np.float64).T @ a2.astype(np.float64)) <= tol
    with pytest.raises(pb.B200Error):
        ctx.gemm(M, 0, 0, dw.data_ptr(), dx.data_ptr(), y.data_ptr(), 64, 64, 64, force_path=3)


def test_l2_ingest_measurement_is_sane(ctx):
    """The measurement aid streams L2-resident data into every SM and reports the rate: a few tens of bytes
    per SM clock on this GPU generation, and its bounded waits must not have run out."""
    per_clk, gbs = ctx.measure_l2_ingest()
    assert 16.0 < per_clk < 200.0 and 20.0 < gbs < 400.0, (per_clk, gbs)
    assert ctx.status_poll() == 0


@pytest.mark.parametrize("dims", [(300, 200, 1100, 1, 1), (512, 264, 520, 1, 3), (260, 72, 2048, 2, 2), (1024, 136, 512, 1, 1)])
def test_half_precision_wide_tile_matches_the_regular_tile(ctx, dims):
    """Half storage, 256 x 512 tiles per CTA pair (pair policy 3 forces them wherever the product has 512
    columns; by default only large products take them) against 256 x 256 tiles (policy 2): all three
    products, ragged edges in every dimension, every operand major-ness.  An overwriting product gives the
    same bits (same instructions in the same order per output element); an accumulating one rounds the
    product to half before adding the old value, so it may differ from the regular tile by one rounding."""
    di, dj, dk, ba, bb = dims
    rng = np.random.default_rng(sum(dims))
    bs = max(ba, bb)
    a = ol.round_to_half(rng.standard_normal(di * dj * ba).astype(np.float32))
    b = ol.round_to_half(rng.standard_normal(dj * dk * bb).astype(np.float32))
    gy = ol.round_to_half(rng.standard_normal(di * dk * bs).astype(np.float32))
    m = MODES["fp16"]
    out = {}
    ctx.set_path_policy(2)
    try:
        for pair in (2, 3):
            ctx.set_pair_policy(pair)
            y = matmul_fw(ctx, m, a, b, di, dj, dk, ba, bb)
            ga0 = np.full(di * dj * ba, 0.5, np.float32)
            gb0 = np.full(dj * dk * bb, 0.5, np.float32)
            ga, gb = matmul_bw(ctx, m, a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
            out[pair] = (y, ga, gb)
    finally:
        ctx.set_pair_policy(0)
        ctx.set_path_policy(0)
    assert np.array_equal(out[2][0], out[3][0])
    y64 = ol.fw_f64(a, b, di, dj, dk, ba, bb)
    ga64, gb64 = ol.bw_f64(a, b, gy, np.full(di * dj * ba, 0.5, np.float32), np.full(dj * dk * bb, 0.5, np.float32),
                           di, dj, dk, ba, bb)
    for got, want in zip(out[3], (y64, ga64, gb64)):
        assert ol.rel_err(got, want) <= TOL["fp16"]
    for i in (1, 2):
        assert ol.rel_err(out[3][i], out[2][i].astype(np.float64)) <= 1e-3

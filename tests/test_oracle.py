"""Pins the CPU oracle: against the reference's own known-answer vectors, against
outputs of the reference's Naive device (committed fixtures, and live where the
reference was compiled into oracle/_ref), and fp64 against fp32."""
import json
import os

import numpy as np
import pytest

import oracle_lib as ol

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def known_answers():
    with open(os.path.join(GOLDEN, "matmul_known_answers.json")) as f:
        return json.load(f)["cases"]


def dims(case):
    di, dj = case["a_shape"]
    dk = case["b_shape"][1]
    assert case["b_shape"][0] == dj
    return di, dj, dk, case["a_batch"], case["b_batch"]


@pytest.mark.parametrize("case", known_answers(), ids=lambda c: c["name"])
def test_oracle_matches_reference_known_answers(case):
    di, dj, dk, ba, bb = dims(case)
    a = np.array(case["a"], np.float32)
    b = np.array(case["b"], np.float32)
    if case["kind"] == "fw":
        want = np.array(case["y"], np.float32)
        got = ol.fw_naive(a, b, di, dj, dk, ba, bb)
        assert ol.ulp_diff(got, want).max() <= case["ulps"]
        got64 = ol.fw_f64(a, b, di, dj, dk, ba, bb)
        assert ol.ulp_diff(got64.astype(np.float32), want).max() <= case["ulps"]
    else:
        gy = np.array(case["gy"], np.float32)
        ga0 = np.full(di * dj * ba, case["prefill"], np.float32)
        gb0 = np.full(dj * dk * bb, case["prefill"], np.float32)
        ga, gb = ol.bw_naive(a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
        assert ol.ulp_diff(ga, np.array(case["ga"], np.float32)).max() <= case["ulps"]
        assert ol.ulp_diff(gb, np.array(case["gb"], np.float32)).max() <= case["ulps"]
        ga64, gb64 = ol.bw_f64(a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
        assert ol.ulp_diff(ga64.astype(np.float32), np.array(case["ga"], np.float32)).max() <= case["ulps"]
        assert ol.ulp_diff(gb64.astype(np.float32), np.array(case["gb"], np.float32)).max() <= case["ulps"]


def ref_cases():
    d = np.load(os.path.join(GOLDEN, "matmul_ref_naive_cases.npz"))
    out = []
    for idx, (di, dj, dk, ba, bb) in enumerate(d["cases"].tolist()):
        out.append((idx, di, dj, dk, ba, bb, d))
    return out


@pytest.mark.parametrize("idx,di,dj,dk,ba,bb,d", ref_cases(),
                         ids=lambda v: str(v) if isinstance(v, int) else "")
def test_oracle_bit_exact_against_reference_naive_fixtures(idx, di, dj, dk, ba, bb, d):
    a, b, gy = d["a_%d" % idx], d["b_%d" % idx], d["gy_%d" % idx]
    y = ol.fw_naive(a, b, di, dj, dk, ba, bb)
    assert np.array_equal(y, d["y_%d" % idx])
    ga0 = np.full(di * dj * ba, 0.5, np.float32)
    gb0 = np.full(dj * dk * bb, 0.5, np.float32)
    ga, gb = ol.bw_naive(a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
    assert np.array_equal(ga, d["ga_%d" % idx])
    assert np.array_equal(gb, d["gb_%d" % idx])
    # the fp64 arbiter agrees with the reference to fp32 rounding noise
    assert ol.rel_err(d["y_%d" % idx], ol.fw_f64(a, b, di, dj, dk, ba, bb)) < 1e-6
    ga64, gb64 = ol.bw_f64(a, b, gy, ga0, gb0, di, dj, dk, ba, bb)
    assert ol.rel_err(d["ga_%d" % idx], ga64) < 1e-6
    assert ol.rel_err(d["gb_%d" % idx], gb64) < 1e-6


@pytest.mark.skipif(not ol.have_ref(), reason="reference not compiled into oracle/_ref on this machine")
def test_oracle_bit_exact_against_live_reference_on_config1():
    c = ol.config1_inputs()
    args = (c["di"], c["dj"], c["dk"], c["ba"], c["bb"])
    y_ref, _ = ol.ref_fw(c["a"], c["b"], *args)
    assert np.array_equal(ol.fw_naive(c["a"], c["b"], *args), y_ref)
    ga_ref, gb_ref, _ = ol.ref_bw(c["a"], c["b"], c["gy"], c["ga0"], c["gb0"], *args)
    ga, gb = ol.bw_naive(c["a"], c["b"], c["gy"], c["ga0"], c["gb0"], *args)
    assert np.array_equal(ga, ga_ref) and np.array_equal(gb, gb_ref)
    # the two oracle tiers agree to 1e-6 on the plumbing workload
    assert ol.rel_err(y_ref, ol.fw_f64(c["a"], c["b"], *args)) < 1e-6
    ga64, gb64 = ol.bw_f64(c["a"], c["b"], c["gy"], c["ga0"], c["gb0"], *args)
    assert ol.rel_err(ga_ref, ga64) < 1e-6 and ol.rel_err(gb_ref, gb64) < 1e-6


def test_input_generator_is_deterministic_and_distributed():
    c1, c2 = ol.config1_inputs(), ol.config1_inputs()
    for k in ("a", "b", "gy"):
        assert np.array_equal(c1[k], c2[k])
    assert -1 <= c1["a"].min() and c1["a"].max() < 1 and abs(c1["a"].mean()) < 0.02
    assert abs(c1["gy"].mean()) < 0.01 and abs(c1["gy"].std() - 1) < 0.01


def test_round_to_half_matches_numpy():
    rng = np.random.default_rng(3)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 0.05,
        rng.uniform(-70000, 70000, 2000).astype(np.float32),
        rng.uniform(-1e-6, 1e-6, 2000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 6.1e-5, 5.96e-8, 2.98e-8, 2.9e-8, np.inf, -np.inf],
                 np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(ol.round_to_half(x), want)


def test_empty_and_degenerate_shapes():
    # 1x1x1, and a contraction shorter than the 8-wide run
    a = np.array([3.0], np.float32)
    b = np.array([-2.0], np.float32)
    assert ol.fw_naive(a, b, 1, 1, 1, 1, 1)[0] == -6.0
    ga, gb = ol.bw_naive(a, b, np.array([1.0], np.float32), np.zeros(1, np.float32), np.zeros(1, np.float32),
                         1, 1, 1, 1, 1)
    assert ga[0] == -2.0 and gb[0] == 3.0

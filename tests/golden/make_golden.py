#!/usr/bin/env python3
"""Regenerates the committed matmul fixtures from the reference tree.

Run where the reference sources are mounted and `make -C oracle ref` has been run:

    python tests/golden/make_golden.py --ref <primitiv source tree>

Writes, next to this script:

* matmul_known_answers.json -- the known-answer vectors of the reference's own
  matmul tests, read out of the test sources as text:
    test/tensor_forward_test.cc   CheckMatMulAA / AB / BatchBroadcast1N / BatchBroadcastN1 / Large
    test/tensor_backward_test.cc  CheckMatMul11 / NN / 1N / N1
    test/operator_impl_test.cc    CheckMatrixMultiply (inputs from setup_2args, gy = ones)
  CheckMatMulLarge builds its 123x123 data from closed forms (i/16, j/16, N*i*j/256,
  sum(i^2)/256); the same closed forms are evaluated here and stored as the vectors.
* matmul_ref_naive_cases.npz -- outputs of the reference's own Naive device
  (oracle/_ref/libref_shim.so, compiled from the unmodified reference sources) on
  seeded random inputs: every broadcast combination at several ragged shapes,
  gradients pre-filled with 0.5 so that accumulation is visible.

Neither file is read from the reference at test time: the tests only use what is
committed here.
"""
import argparse
import ctypes
import json
import os
import re

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _block(src, fixture, name):
    m = re.search(r"TEST_F\(%s, %s\) \{" % (fixture, name), src)
    assert m, name
    end = src.find("\nTEST_F(", m.end())
    return src[m.end():end if end > 0 else len(src)]


def _nums(text):
    return [float(t) for t in re.split(r"[,\s]+", text.strip()) if t]


def _shape(text):
    """'Shape({2, 2}, 3)' or '{2, 2}' -> ([2, 2], 3)."""
    m = re.match(r"Shape\(\{([\d, ]*)\},\s*(\d+)\)", text.strip())
    if m:
        return [int(v) for v in _nums(m.group(1))], int(m.group(2))
    m = re.match(r"\{([\d, ]*)\}", text.strip())
    return [int(v) for v in _nums(m.group(1))], 1


def forward_cases(src):
    out = []
    shapes = {
        "CheckMatMulAA": (([2, 2], 3), ([2, 2], 3)),
        "CheckMatMulAB": (([3, 4], 1), ([4, 6], 1)),
        "CheckMatMulBatchBroadcast1N": (([2, 2], 1), ([2, 2], 2)),
        "CheckMatMulBatchBroadcastN1": (([2, 2], 2), ([2, 2], 1)),
    }
    for name, (sa, sb) in shapes.items():
        blk = _block(src, "TensorForwardTest", name)
        vecs = {k: _nums(v) for k, v in re.findall(r"(\w+_data)\s*\{([^}]*)\}", blk)}
        # the shapes in the table above must be the ones the test constructs
        made = re.findall(r"new_tensor_by_vector\(\s*(Shape\(\{[\d, ]*\},\s*\d+\)|\{[\d, ]*\})", blk)
        made = [_shape(t) for t in made]
        if name == "CheckMatMulAA":
            assert made == [tuple(sa)] or made == [sa], made
            a = b = vecs["x_data"]
        else:
            assert [tuple(x) for x in made] == [tuple(sa), tuple(sb)], (name, made)
            a, b = vecs["a_data"], vecs["b_data"]
        ulps = 4
        ulps16 = 4096
        m = re.search(r"CUDA16 \? (\d+)", blk)
        if m:
            ulps16 = int(m.group(1))
        out.append(dict(name=name, kind="fw", a_shape=sa[0], a_batch=sa[1],
                        b_shape=sb[0], b_batch=sb[1], a=a, b=b, y=vecs["y_data"],
                        ulps=ulps, ulps_fp16=ulps16))
    # CheckMatMulLarge: closed forms (test/tensor_forward_test.cc:1872-1905)
    blk = _block(src, "TensorForwardTest", "CheckMatMulLarge")
    n = int(re.search(r"N = (\d+);", blk).group(1))
    ulps16 = int(re.search(r"CUDA16 \? (\d+)", blk).group(1))
    ksum = sum(i * i for i in range(n))
    a = np.zeros(n * n, np.float32)
    b = np.zeros(n * n, np.float32)
    y1 = np.zeros(n * n, np.float32)
    y2 = np.zeros(n * n, np.float32)
    for i in range(n):
        for j in range(n):
            a[i + j * n] = i / 16.0
            b[i + j * n] = j / 16.0
            y1[i + j * n] = n * i * j / 256.0
            y2[i + j * n] = ksum / 256.0
    out.append(dict(name="CheckMatMulLarge_ab", kind="fw", a_shape=[n, n], a_batch=1,
                    b_shape=[n, n], b_batch=1, a=a.tolist(), b=b.tolist(), y=y1.tolist(),
                    ulps=4, ulps_fp16=ulps16))
    out.append(dict(name="CheckMatMulLarge_ba", kind="fw", a_shape=[n, n], a_batch=1,
                    b_shape=[n, n], b_batch=1, a=b.tolist(), b=a.tolist(), y=y2.tolist(),
                    ulps=4, ulps_fp16=ulps16))
    return out


def backward_cases(src):
    out = []
    for name in ("CheckMatMul11", "CheckMatMulNN", "CheckMatMul1N", "CheckMatMulN1"):
        blk = _block(src, "TensorBackwardTest", name)
        made = re.findall(
            r"new_tensor_by_vector\(\s*(Shape\(\{[\d, ]*\},\s*\d+\)|\{[\d, ]*\}),\s*\{([^}]*)\}\)", blk)
        assert len(made) == 3, (name, made)
        (sa, a), (sb, b), (sg, gy) = [(_shape(s), _nums(v)) for s, v in made]
        prefill = float(re.search(r"new_tensor_by_constant\(a\.shape\(\), ([-\d.]+)\)", blk).group(1))
        vals = {k: _nums(v) for k, v in re.findall(r"(g[ab]_val)\s*\{([^}]*)\}", blk)}
        out.append(dict(name=name, kind="bw", a_shape=sa[0], a_batch=sa[1],
                        b_shape=sb[0], b_batch=sb[1], a=a, b=b, gy=gy, prefill=prefill,
                        ga=vals["ga_val"], gb=vals["gb_val"], ulps=4, ulps_fp16=4096))
    return out


def operator_case(src):
    setup = re.search(r"void setup_2args\(\) \{(.*?)\n  \}", src, re.S).group(1)
    lists = re.findall(r"\*arg_shapes\[\d\], \{([^}]*)\}", setup)
    a, b = _nums(lists[0]), _nums(lists[1])
    blk = _block(src, "OperatorImplTest", "CheckMatrixMultiply")
    ret = _nums(re.search(r"ret_data \{([^}]*)\}", blk).group(1))
    grads = re.search(r"bw_grads \{\s*\{([^}]*)\},\s*\{([^}]*)\},", blk)
    return [
        dict(name="OperatorMatrixMultiply_fw", kind="fw", a_shape=[2, 2], a_batch=3,
             b_shape=[2, 2], b_batch=3, a=a, b=b, y=ret, ulps=4, ulps_fp16=4096),
        dict(name="OperatorMatrixMultiply_bw", kind="bw", a_shape=[2, 2], a_batch=3,
             b_shape=[2, 2], b_batch=3, a=a, b=b, gy=[1.0] * 12, prefill=0.0,
             ga=_nums(grads.group(1)), gb=_nums(grads.group(2)), ulps=4, ulps_fp16=4096),
    ]


# (di, dj, dk, ba, bb): ragged, prime and tile-edge shapes, all broadcast combinations.
REF_CASES = [
    (1, 1, 1, 1, 1), (2, 3, 4, 1, 1), (7, 5, 3, 3, 3), (7, 5, 3, 1, 3), (7, 5, 3, 3, 1),
    (16, 16, 16, 2, 2), (33, 17, 9, 1, 4), (33, 17, 9, 4, 1), (64, 40, 24, 2, 2),
    (129, 65, 31, 1, 2), (129, 65, 31, 2, 1), (128, 128, 128, 1, 1), (100, 260, 12, 2, 2),
    (10, 1024, 1, 1, 8), (64, 96, 32, 1, 4),
]


def ref_naive_cases():
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_shim.so"))
    fp = ctypes.POINTER(ctypes.c_float)
    u32 = ctypes.c_uint32
    lib.ref_naive_matmul_fw.argtypes = [fp, fp, fp, u32, u32, u32, u32, u32, ctypes.c_void_p]
    lib.ref_naive_matmul_bw.argtypes = [fp, fp, fp, fp, fp, u32, u32, u32, u32, u32, ctypes.c_void_p]
    store = {"cases": np.array(REF_CASES, np.uint32)}
    for idx, (di, dj, dk, ba, bb) in enumerate(REF_CASES):
        rng = np.random.default_rng(1000 + idx)
        bs = max(ba, bb)
        a = rng.uniform(-1, 1, di * dj * ba).astype(np.float32)
        b = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
        gy = rng.standard_normal(di * dk * bs).astype(np.float32)
        y = np.zeros(di * dk * bs, np.float32)
        ga = np.full(di * dj * ba, 0.5, np.float32)
        gb = np.full(dj * dk * bb, 0.5, np.float32)
        p = lambda x: x.ctypes.data_as(fp)
        assert lib.ref_naive_matmul_fw(p(a), p(b), p(y), di, dj, dk, ba, bb, None) == 0
        assert lib.ref_naive_matmul_bw(p(a), p(b), p(gy), p(ga), p(gb), di, dj, dk, ba, bb, None) == 0
        for k, v in dict(a=a, b=b, gy=gy, y=y, ga=ga, gb=gb).items():
            store["%s_%d" % (k, idx)] = v
    return store


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="the primitiv source tree the vectors are taken from")
    args = ap.parse_args()
    rd = lambda p: open(os.path.join(args.ref, p)).read()
    cases = forward_cases(rd("test/tensor_forward_test.cc"))
    cases += backward_cases(rd("test/tensor_backward_test.cc"))
    cases += operator_case(rd("test/operator_impl_test.cc"))
    with open(os.path.join(HERE, "matmul_known_answers.json"), "w") as f:
        json.dump(dict(source="reference test sources, read as text", cases=cases), f)
    np.savez_compressed(os.path.join(HERE, "matmul_ref_naive_cases.npz"), **ref_naive_cases())
    print("wrote", len(cases), "known-answer cases and", len(REF_CASES), "reference-run cases")


if __name__ == "__main__":
    main()

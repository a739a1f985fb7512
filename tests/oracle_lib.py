"""ctypes access to the CPU checkers under oracle/ (test infrastructure only).

* ``oracle/_build/libmatmul_oracle.so``  -- the plain-C restatement + seeded input generator
* ``oracle/_ref/libref_shim.so``         -- the reference's own Naive device (optional: only
  present where it was compiled from the reference sources)
"""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "_build", "libmatmul_oracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libref_shim.so")

_fp = ctypes.POINTER(ctypes.c_float)
_dp = ctypes.POINTER(ctypes.c_double)
_u32 = ctypes.c_uint32
_u64 = ctypes.c_uint64

_oracle = None
_ref = None


def build_oracle():
    subprocess.check_call(["make", "-s", "-C", ORACLE_DIR, "oracle"])


def oracle():
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            build_oracle()
        lib = ctypes.CDLL(ORACLE_SO)
        lib.oracle_matmul_fw_naive_f32.argtypes = [_fp, _fp, _fp, _u32, _u32, _u32, _u32, _u32]
        lib.oracle_matmul_bw_naive_f32.argtypes = [_fp, _fp, _fp, _fp, _fp, _u32, _u32, _u32, _u32, _u32]
        lib.oracle_matmul_fw_f64.argtypes = [_fp, _fp, _dp, _u32, _u32, _u32, _u32, _u32]
        lib.oracle_matmul_bw_f64.argtypes = [_fp, _fp, _fp, _dp, _dp, _u32, _u32, _u32, _u32, _u32]
        lib.oracle_normwise_rel_err_f32.argtypes = [_fp, _dp, _u64]
        lib.oracle_normwise_rel_err_f32.restype = ctypes.c_double
        lib.oracle_round_to_half.argtypes = [_fp, _fp, _u64]
        lib.oracle_mt19937_draw.argtypes = [_u32, ctypes.c_int, ctypes.POINTER(ctypes.c_int), _fp, _fp,
                                            ctypes.POINTER(_u64), ctypes.POINTER(_fp)]
        _oracle = lib
    return _oracle


def have_ref():
    return os.path.exists(REF_SO)


def ref():
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(REF_SO)
        lib.ref_naive_matmul_fw.argtypes = [_fp, _fp, _fp, _u32, _u32, _u32, _u32, _u32, _dp]
        lib.ref_naive_matmul_bw.argtypes = [_fp, _fp, _fp, _fp, _fp, _u32, _u32, _u32, _u32, _u32, _dp]
        _ref = lib
    return _ref


def _f(x):
    assert x.dtype == np.float32 and x.flags.c_contiguous
    return x.ctypes.data_as(_fp)


def _d(x):
    assert x.dtype == np.float64 and x.flags.c_contiguous
    return x.ctypes.data_as(_dp)


def fw_naive(a, b, di, dj, dk, ba, bb):
    y = np.empty(di * dk * max(ba, bb), np.float32)
    oracle().oracle_matmul_fw_naive_f32(_f(a), _f(b), _f(y), di, dj, dk, ba, bb)
    return y


def bw_naive(a, b, gy, ga0, gb0, di, dj, dk, ba, bb):
    ga, gb = ga0.copy(), gb0.copy()
    oracle().oracle_matmul_bw_naive_f32(_f(a), _f(b), _f(gy), _f(ga), _f(gb), di, dj, dk, ba, bb)
    return ga, gb


def fw_f64(a, b, di, dj, dk, ba, bb):
    y = np.empty(di * dk * max(ba, bb), np.float64)
    oracle().oracle_matmul_fw_f64(_f(a), _f(b), _d(y), di, dj, dk, ba, bb)
    return y


def bw_f64(a, b, gy, ga0, gb0, di, dj, dk, ba, bb):
    ga, gb = ga0.astype(np.float64), gb0.astype(np.float64)
    oracle().oracle_matmul_bw_f64(_f(a), _f(b), _f(gy), _d(ga), _d(gb), di, dj, dk, ba, bb)
    return ga, gb


def rel_err(x, ref64):
    x = np.ascontiguousarray(x, np.float32)
    return oracle().oracle_normwise_rel_err_f32(_f(x), _d(ref64), x.size)


def round_to_half(x):
    y = np.empty_like(x)
    oracle().oracle_round_to_half(_f(x), _f(y), x.size)
    return y


def ref_fw(a, b, di, dj, dk, ba, bb):
    y = np.empty(di * dk * max(ba, bb), np.float32)
    sec = ctypes.c_double()
    assert ref().ref_naive_matmul_fw(_f(a), _f(b), _f(y), di, dj, dk, ba, bb, ctypes.byref(sec)) == 0
    return y, sec.value


def ref_bw(a, b, gy, ga0, gb0, di, dj, dk, ba, bb):
    ga, gb = ga0.copy(), gb0.copy()
    sec = ctypes.c_double()
    assert ref().ref_naive_matmul_bw(_f(a), _f(b), _f(gy), _f(ga), _f(gb), di, dj, dk, ba, bb,
                                     ctypes.byref(sec)) == 0
    return ga, gb, sec.value


def mt19937_draw(seed, specs):
    """specs: list of (kind, p0, p1, count) with kind 'uniform' | 'normal'.  One generator, in order."""
    n = len(specs)
    kinds = (ctypes.c_int * n)(*[0 if s[0] == "uniform" else 1 for s in specs])
    p0 = np.array([s[1] for s in specs], np.float32)
    p1 = np.array([s[2] for s in specs], np.float32)
    counts = (_u64 * n)(*[int(s[3]) for s in specs])
    outs = [np.empty(int(s[3]), np.float32) for s in specs]
    ptrs = (_fp * n)(*[_f(o) for o in outs])
    oracle().oracle_mt19937_draw(seed, n, kinds, _f(p0), _f(p1), counts, ptrs)
    return outs


def ulp_diff(a, b):
    """Elementwise ULP distance, as test/test_utils.h:26-35 of the reference computes it."""
    ai = np.ascontiguousarray(a, np.float32).view(np.int32).astype(np.int64)
    bi = np.ascontiguousarray(b, np.float32).view(np.int32).astype(np.int64)
    ai = np.where(ai < 0, -(2 ** 31) - ai, ai)
    bi = np.where(bi < 0, -(2 ** 31) - bi, bi)
    return np.abs(ai - bi)


def config1_inputs():
    """The plumbing workload: W {256,256} U(-1,1); X {256,64}x16 U(-1,1); gy {256,64}x16 N(0,1); seed 0."""
    di, dj, dk, ba, bb = 256, 256, 64, 1, 16
    w, x, gy = mt19937_draw(0, [("uniform", -1, 1, di * dj), ("uniform", -1, 1, dj * dk * bb),
                                ("normal", 0, 1, di * dk * bb)])
    return dict(di=di, dj=dj, dk=dk, ba=ba, bb=bb, a=w, b=x, gy=gy,
                ga0=np.full(di * dj, 0.5, np.float32), gb0=np.full(dj * dk * bb, 0.5, np.float32))

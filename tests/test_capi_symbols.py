"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol
include/*.h declares, fails loudly without a GPU, and its pure host logic is right."""
import ctypes
import glob
import os
import re

import pytest

import primitiv_b200 as pb
from primitiv_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for h in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"B200_API\s+[\w\s\*]+?\b(b200_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_hot_path():
    names = declared_symbols()
    for must in ("b200_matmul_fw", "b200_matmul_bw", "b200_gemm", "b200_ctx_create", "b200_pool_alloc"):
        assert must in names


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(pb.library_path())
    missing = [n for n in declared_symbols() if not hasattr(handle, n)]
    assert not missing, missing


def test_python_binding_covers_every_declared_symbol():
    assert sorted(capi.SIGNATURES) == declared_symbols()


def test_error_strings():
    lib = pb.lib()
    assert lib.b200_error_string(0) == b"ok"
    assert b"no CPU fallback" in lib.b200_error_string(1002)
    assert b"bounded" in lib.b200_error_string(1004)


def test_no_gpu_means_loud_failure_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pb.B200Error) as e:
        pb.Context(0)
    assert e.value.code == 1002


def test_pool_size_classes():
    f = pb.lib().b200_pool_size_class
    assert f(0) == 256 and f(1) == 256 and f(256) == 256 and f(257) == 512 and f(1024) == 1024
    prev = 0
    for req in [1025, 4096, 4097, 5000, 1 << 20, (1 << 20) + 1, 205520896, 1 << 29, (1 << 30) + 5, 3 << 30]:
        c = f(req)
        assert c >= req and c % 256 == 0
        assert c <= req * 1.25 + 256          # four classes per octave: at most 25% round-up
        assert f(c) == c                      # classes are fixed points
        assert c >= prev
        prev = c
    # the 205 MB activation of the MLP workload takes a 224 MiB block, not 256 MiB
    assert f(784 * 65536 * 4) == 224 << 20


def test_every_kernel_takes_part_in_dependent_launch():
    """Kernels are launched with the programmatic-serialization attribute, which lets a grid start
    before the one in front of it has finished: each kernel must therefore wait for its predecessor
    (pdl_enter, or pdl_wait_previous after a set-up that touches no global memory) before anything
    else.  A kernel without the wait would race; this keeps one from slipping in."""
    csrc = os.path.join(ROOT, "primitiv_b200", "csrc")
    missing, raw = [], []
    for name in sorted(os.listdir(csrc)):
        if not name.endswith((".cu", ".cuh")):
            continue
        text = open(os.path.join(csrc, name)).read()
        if "<<<" in text:
            raw.append(name)          # every launch goes through b200::launch
        for m in re.finditer(r"__global__", text):
            brace = text.index("{", m.end())      # no brace occurs inside a kernel's signature
            body = text[brace:brace + 4000]
            if "pdl_enter();" not in body[:200] and "pdl_wait_previous();" not in body:
                missing.append((name, text[m.start():m.start() + 120].split("(")[0][-60:]))
    assert not raw, raw
    assert not missing, missing

"""primitiv::devices::B200 through primitiv's own C++ API.

The parity runner (tests/cpp/device_parity.cc) is a C++ program because the interface
under test is a C++ class: it drives every Device operation, the copy-on-write Tensor
logic, and a Graph + SGD training loop on the B200 device and on the reference's Naive
device from the same seeded inputs, and compares.  It is built where the reference
headers are available (primitiv_b200/device/Makefile) and travels as a binary."""
import ctypes
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNER = os.path.join(ROOT, "tests", "cpp", "_build", "device_parity")
PLUGIN = os.path.join(ROOT, "primitiv_b200", "device", "libprimitiv_b200_device.so")

needs_plugin = pytest.mark.skipif(not os.path.exists(PLUGIN),
                                  reason="device plugin not built (needs the primitiv headers)")


@needs_plugin
def test_plugin_exports_the_c_api_constructors():
    lib = ctypes.CDLL(PLUGIN)
    for name in ("primitivCreateB200Device", "primitivCreateB200DeviceWithSeed",
                 "primitivCreateB200DeviceWithSeedAndMode", "primitivGetNumB200Devices"):
        assert hasattr(lib, name), name


@needs_plugin
def test_plugin_fails_loudly_without_a_gpu():
    import sys
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    # In a fresh interpreter: primitiv's C API reports errors by throwing and catching C++
    # exceptions inside its shared library, and that unwinding does not survive in a process
    # that has already loaded torch's bundled runtime libraries.
    code = ("import ctypes; lib = ctypes.CDLL(%r); dev = ctypes.c_void_p(); "
            "rc = lib.primitivCreateB200Device(0, ctypes.byref(dev)); print(rc, dev.value)" % PLUGIN)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    # PRIMITIV_C_ERROR (-1): the constructor threw primitiv::Error, no fallback device is made
    assert r.stdout.split() == ["-1", "None"], r.stdout + r.stderr


@pytest.mark.gpu
@needs_plugin
@pytest.mark.parametrize("mode", ["3xtf32", "tf32", "fp16"])
def test_device_parity_against_reference_naive(mode):
    assert os.path.exists(RUNNER), "tests/cpp/_build/device_parity is not built"
    r = subprocess.run([RUNNER, mode], capture_output=True, text=True, timeout=600)
    tail = (r.stdout + r.stderr)[-4000:]
    assert r.returncode == 0, tail
    assert "0 failures" in r.stdout, tail


@pytest.mark.gpu
@needs_plugin
def test_primitiv_c_api_runs_matmul_on_b200():
    """primitiv's unmodified C API (primitivApplyTensorMatmul) on a device made by the new constructor."""
    capi = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libprimitiv_c.so"), mode=ctypes.RTLD_GLOBAL)
    plug = ctypes.CDLL(PLUGIN, mode=ctypes.RTLD_GLOBAL)
    vp = ctypes.c_void_p
    dev = vp()
    assert plug.primitivCreateB200DeviceWithSeedAndMode(0, 1, 0, ctypes.byref(dev)) == 0
    u32 = ctypes.c_uint32

    def shape(dims, batch):
        s = vp()
        arr = (u32 * len(dims))(*dims)
        assert capi.primitivCreateShapeWithDims(arr, ctypes.c_size_t(len(dims)), u32(batch), ctypes.byref(s)) == 0
        return s

    def tensor(dims, batch, values):
        t = vp()
        buf = (ctypes.c_float * len(values))(*values)
        assert capi.primitivApplyTensorInput(shape(dims, batch), buf, ctypes.c_size_t(len(values)), dev,
                                             ctypes.byref(t)) == 0
        return t

    # test/tensor_forward_test.cc:1840-1850 (CheckMatMulBatchBroadcast1N) through the C API
    a = tensor([2, 2], 1, [10, 1000, 1, 100])
    b = tensor([2, 2], 2, [1, 2, 3, 4, 5, 6, 7, 8])
    y = vp()
    assert capi.primitivApplyTensorMatmul(a, b, ctypes.byref(y)) == 0
    n = ctypes.c_size_t(0)
    assert capi.primitivEvaluateTensorAsArray(y, None, ctypes.byref(n)) == 0
    out = (ctypes.c_float * n.value)()
    assert capi.primitivEvaluateTensorAsArray(y, out, ctypes.byref(n)) == 0
    assert list(out) == [12, 1200, 34, 3400, 56, 5600, 78, 7800]
    for t in (a, b, y):
        capi.primitivDeleteTensor(t)
    capi.primitivDeleteDevice(dev)

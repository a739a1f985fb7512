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
                 "primitivCreateB200DeviceWithSeedAndMode", "primitivGetNumB200Devices",
                 "primitivCreateB200GroupDevice", "primitivCreateB200GroupDeviceWithSeedAndMode"):
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
@pytest.mark.parametrize("mode", ["3xtf32", "tf32", "fp16", "3xfp16"])
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
    capi = ctypes.CDLL(os.path.join(ROOT, "baseline", "_ref", "framework", "libprimitiv_c.so"), mode=ctypes.RTLD_GLOBAL)
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


def _run_json(binary, *args):
    import json
    path = os.path.join(ROOT, "tests", "cpp", "_build", binary)
    assert os.path.exists(path), "%s is not built" % path
    r = subprocess.run([path] + [str(a) for a in args], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


@pytest.mark.gpu
@needs_plugin
@pytest.mark.parametrize("mode,tol", [("3xtf32", 2e-5), ("tf32", 4e-3)])
def test_recurrent_step_loop_matches_reference_naive(mode, tol):
    """An LSTM step loop through primitiv's Graph (forward and backward through time): the loss
    and the weight gradients of a 3-step prefix agree with the reference's Naive device."""
    out = _run_json("lstm_steps", mode, 6, 1, 3)
    assert out["loss_rel_diff"] < tol and out["grad_wx_rel_diff"] < tol and out["grad_wh_rel_diff"] < tol, out
    assert out["launches_per_loop"]["gemm_tc"] > 0     # the products ran on the tensor-core kernel


@pytest.mark.gpu
@needs_plugin
@pytest.mark.parametrize("mode,tol", [("3xtf32", 1e-5), ("tf32", 2e-3), ("3xfp16", 1e-5)])
def test_perceptron_training_step_matches_reference_naive(mode, tol):
    """Two SGD steps of the 784-1024-1024-10 perceptron (softmax cross entropy) at batch 256 on
    both devices: loss and updated weights agree; then one step at a batch above 65535."""
    out = _run_json("mlp_step", mode, 65600, 1, 256)
    assert out["loss_rel_diff"] < tol and out["w1_rel_diff"] < tol and out["w3_rel_diff"] < tol, out
    assert 2.0 < out["loss"] < 2.6                      # ln(10) = 2.30 for an untrained 10-way classifier


REF_SUITE = os.path.join(ROOT, "tests", "cpp", "_build", "ref_tensor_tests")


@pytest.mark.gpu
@needs_plugin
@pytest.mark.parametrize("policy", ["0", "2"], ids=["auto", "tensorcore"])
@pytest.mark.parametrize("mode", ["3xtf32", "tf32", "fp16", "3xfp16"])
def test_primitiv_own_tensor_tests_pass_on_b200(mode, policy):
    """The reference's own test/tensor_forward_test.cc, tensor_backward_test.cc and tensor_test.cc
    (compiled from the reference tree, unmodified; 372 cases, each looping over every device in
    the list) with two devices::B200 objects next to Naive in that list, at the reference's own
    tolerances (4 ULPs for fp32 storage, the CUDA16 bound for half storage)."""
    assert os.path.exists(REF_SUITE), "tests/cpp/_build/ref_tensor_tests is not built"
    # policy 2: even the tests' tiny products go through the tensor-core kernel where eligible
    env = dict(os.environ, PRIMITIV_B200_PATH_POLICY=policy)
    r = subprocess.run([REF_SUITE, mode], capture_output=True, text=True, timeout=900, env=env)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    summary = [l for l in r.stdout.splitlines() if l.startswith("[==========]")][-1]
    ran, passed, failed = [int(w) for w in summary.replace(",", "").split() if w.isdigit()]
    assert ran >= 370 and passed == ran and failed == 0, summary
    assert r.stderr.count("Type: B200") >= 6   # two B200 objects in each of the three suites' lists


@pytest.mark.gpu
@needs_plugin
@pytest.mark.parametrize("program", ["device_parity", "ref_tensor_tests"])
@pytest.mark.parametrize("mode", ["3xtf32", "fp16"])
def test_no_operation_writes_outside_its_tensor(mode, program):
    """Both suites again with guard bands round every block of the memory pool, checked before
    every operation (PRIMITIV_B200_POOL_GUARD=2): a kernel that stored past either end of a tensor
    or of its scratch would make the next operation throw."""
    path = os.path.join(ROOT, "tests", "cpp", "_build", program)
    assert os.path.exists(path), "%s is not built" % path
    env = dict(os.environ, PRIMITIV_B200_POOL_GUARD="2", PRIMITIV_B200_PATH_POLICY="2" if program == "ref_tensor_tests" else "0")
    r = subprocess.run([path, mode], capture_output=True, text=True, timeout=1200, env=env)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "guard band" not in r.stdout + r.stderr, tail
    if program == "device_parity":
        assert "0 failures" in r.stdout, tail
    else:
        summary = [l for l in r.stdout.splitlines() if l.startswith("[==========]")][-1]
        ran, passed, failed = [int(w) for w in summary.replace(",", "").split() if w.isdigit()]
        assert ran >= 370 and passed == ran and failed == 0, summary


@pytest.mark.gpu
@needs_plugin
def test_reference_xor_example_trains_on_b200():
    """examples/xor/xor.cc of the reference, compiled from the reference tree with only its device
    line swapped (a forced include turns `devices::Naive dev;` into a B200 on GPU 0): Graph,
    Parameter, XavierUniform (device RNG), SGD and the matmul path, ten epochs, loss must fall."""
    path = os.path.join(ROOT, "primitiv_b200", "device", "_build", "example_xor")
    assert os.path.exists(path), "example_xor is not built"
    r = subprocess.run([path], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout + r.stderr)[-2000:]
    losses = [float(l.split(":")[1]) for l in r.stdout.splitlines() if l.strip().startswith("loss:")]
    assert len(losses) == 10 and losses[-1] < losses[0], losses


# ---- devices::B200Group: one primitiv Device over several shards -------------------------------
#
# "0,0,0" puts three shards on GPU 0: every line of the sharding logic (uneven cuts, minibatches
# smaller than the group, sums over shards, items moving between shards) runs on a single GPU;
# "0,1" is the same over two GPUs, where the sums and copies cross NVLink.

GROUP_RUNNER = os.path.join(ROOT, "tests", "cpp", "_build", "group_parity")


def _gpu_count():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _group_lists():
    lists = ["0,0", "0,0,0"]
    n = _gpu_count()
    if n >= 2:
        lists.append("0,1")
    if n >= 4:
        lists.append("0,1,2,3")
    return lists


@pytest.mark.gpu
@needs_plugin
@pytest.mark.parametrize("mode", ["3xtf32", "tf32", "fp16", "3xfp16"])
def test_group_parity_against_reference_naive(mode):
    """tests/cpp/group_parity.cc: matmul fw / bw in all broadcast combinations, sums over the
    batch, batch_pick / slice / concat and three training steps through primitiv's Graph on a
    B200Group against Naive; replicas of unbatched tensors must hold identical bits."""
    import json
    assert os.path.exists(GROUP_RUNNER), "tests/cpp/_build/group_parity is not built"
    for ids in _group_lists():
        r = subprocess.run([GROUP_RUNNER, mode, ids], capture_output=True, text=True, timeout=600)
        tail = (r.stdout + r.stderr)[-4000:]
        assert r.returncode == 0, "%s: %s" % (ids, tail)
        out = json.loads(r.stdout.strip().splitlines()[-1])
        assert out["failures"] == 0 and out["checks"] > 200 and out["cross_gpu_sums"] > 50, out
        assert out["shards"] == len(ids.split(","))


@pytest.mark.gpu
@needs_plugin
@pytest.mark.parametrize("mode", ["3xtf32", "fp16"])
def test_primitiv_own_tensor_tests_pass_on_a_group(mode):
    """The reference's own tensor tests again, with a B200Group as the first GPU device of the list
    (next to Naive and a plain B200, so tensors are also copied between all three kinds)."""
    assert os.path.exists(REF_SUITE), "tests/cpp/_build/ref_tensor_tests is not built"
    for ids in _group_lists()[1:3]:
        env = dict(os.environ, PRIMITIV_B200_GROUP=ids)
        r = subprocess.run([REF_SUITE, mode], capture_output=True, text=True, timeout=900, env=env)
        tail = (r.stdout + r.stderr)[-3000:]
        assert r.returncode == 0, "%s: %s" % (ids, tail)
        summary = [l for l in r.stdout.splitlines() if l.startswith("[==========]")][-1]
        ran, passed, failed = [int(w) for w in summary.replace(",", "").split() if w.isdigit()]
        assert ran >= 370 and passed == ran and failed == 0, summary
        assert r.stderr.count("Type: B200Group") >= 3


@pytest.mark.gpu
@needs_plugin
def test_perceptron_step_on_a_group_of_gpus():
    """mlp_step unchanged on a B200Group over two GPUs: same loss and weights as Naive at batch 256."""
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    out = _run_json("mlp_step", "3xtf32", 8192, 1, 256, 2)
    assert out["gpus"] == 2
    assert out["loss_rel_diff"] < 1e-5 and out["w1_rel_diff"] < 1e-5 and out["w3_rel_diff"] < 1e-5, out


@pytest.mark.gpu
@needs_plugin
def test_reference_xor_example_trains_on_a_group():
    """examples/xor/xor.cc of the reference again, its device line swapped for a B200Group: the batch of
    four samples is cut over the shards and the parameter gradients are summed between them."""
    path = os.path.join(ROOT, "primitiv_b200", "device", "_build", "example_xor_group")
    assert os.path.exists(path), "example_xor_group is not built"
    for ids in _group_lists()[:3]:
        env = dict(os.environ, PRIMITIV_B200_GROUP=ids)
        r = subprocess.run([path], capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, "%s: %s" % (ids, (r.stdout + r.stderr)[-2000:])
        losses = [float(l.split(":")[1]) for l in r.stdout.splitlines() if l.strip().startswith("loss:")]
        assert len(losses) == 10 and losses[-1] < losses[0], (ids, losses)

"""In-tree build of libprimitiv_b200.so (CUDA kernels + C ABI) for sm_100a.

    python -m primitiv_b200.build [--verbose] [--force]

nvcc cross-compiles without a GPU.  Objects and the library stay inside the
package directory so that a snapshot of the tree carries them to a GPU machine.
The CUDA runtime is linked statically, so the library does not depend on which
libcudart another component of the process (e.g. PyTorch) has loaded.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(PKG, "libprimitiv_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False, dev_knobs=False):
    """dev_knobs=True compiles the development switches of the tensor-core kernel in
    (-DPRIMITIV_B200_DEV_KNOBS: environment variables that disable parts of it for
    experiments).  The flag set is recorded beside the objects, so a product build after a
    development build recompiles."""
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    flags = NVCC_FLAGS + (["-DPRIMITIV_B200_DEV_KNOBS"] if dev_knobs else [])
    stamp = os.path.join(OBJ, "flags.txt")
    old_flags = open(stamp).read() if os.path.exists(stamp) else None
    if old_flags != " ".join(flags):
        force = True
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(PKG), "include", "primitiv_b200.h"))
    headers.append(os.path.join(os.path.dirname(PKG), "include", "primitiv_b200_ops.h"))
    headers.append(os.path.abspath(__file__))
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=8) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed: " + cmd[-3])
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                      "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    with open(stamp, "w") as f:
        f.write(" ".join(flags))
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv, dev_knobs="--dev-knobs" in sys.argv))

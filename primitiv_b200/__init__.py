"""primitiv_b200: Blackwell (sm_100a) backend for primitiv's matmul_fw / matmul_bw path.

The product is the native library ``libprimitiv_b200.so`` (CUDA kernels behind the
C ABI declared in ``include/primitiv_b200.h``) and the C++ class
``primitiv::devices::B200`` built on it (``primitiv_b200/device``).  This Python
package is a thin ctypes binding of the C ABI for tests, the benchmark and the
multi-GPU harness.  There is no Python or CPU implementation behind it: if the
library is missing, or no sm_100 GPU is visible, the calls raise.
"""
from .capi import (  # noqa: F401
    MODE_FP32_3XTF32, MODE_TF32, MODE_FP16, MODE_FP32_3XFP16, B200Error, Context, lib, library_path,
)

"""ctypes binding of include/primitiv_b200.h.

Device memory and streams come from the caller (raw integer addresses, e.g.
``torch.Tensor.data_ptr()``); this module never allocates through torch and has
no compute of its own.
"""
import ctypes
import os

MODE_FP32_3XTF32 = 0
MODE_TF32 = 1
MODE_FP16 = 2
MODE_FP32_3XFP16 = 3

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_u32 = ctypes.c_uint32
_u64 = ctypes.c_uint64
_vp = ctypes.c_void_p
_int = ctypes.c_int

# name -> (restype, argtypes); every symbol include/primitiv_b200.h declares
SIGNATURES = {
    "b200_error_string": (ctypes.c_char_p, [_int]),
    "b200_ctx_create": (_int, [_int, ctypes.POINTER(_vp)]),
    "b200_ctx_destroy": (_int, [_vp]),
    "b200_ctx_device": (_int, [_vp, ctypes.POINTER(_int), ctypes.POINTER(_int)]),
    "b200_status_poll": (_int, [_vp, _vp, ctypes.POINTER(_int)]),
    "b200_status_peek": (_int, [_vp, ctypes.POINTER(_int)]),
    "b200_selftest_wait_timeout": (_int, [_vp, _vp]),
    "b200_pool_alloc": (_int, [_vp, ctypes.c_size_t, ctypes.POINTER(_vp), ctypes.POINTER(ctypes.c_size_t)]),
    "b200_pool_free": (_int, [_vp, _vp]),
    "b200_pool_release_cached": (_int, [_vp]),
    "b200_pool_stats": (_int, [_vp, ctypes.POINTER(_u64)]),
    "b200_pool_set_limit": (_int, [_vp, ctypes.c_size_t]),
    "b200_pool_size_class": (ctypes.c_size_t, [ctypes.c_size_t]),
    "b200_measure_l2_ingest": (_int, [_vp, _vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]),
    "b200_pool_set_guard": (_int, [_vp, ctypes.c_size_t]),
    "b200_pool_check_guards": (_int, [_vp, _vp, ctypes.POINTER(_u64), ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int)]),
    "b200_matmul_fw": (_int, [_vp, _int, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp]),
    "b200_matmul_bw": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp]),
    "b200_matmul_bw_ex": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _int, _int, _vp]),
    "b200_matmul_fw_host": (_int, [_vp, _int, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32]),
    "b200_matmul_bw_host": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32]),
    "b200_matmul_fw_bw_host": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _int, _int]),
    "b200_gemm": (_int, [_vp, _int, _int, _int, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32,
                         _u64, _u64, _u64, _u64, _u64, _int, _int, _vp]),
    "b200_gemm_3xtf32_noalloc": (_int, [_vp, _int, _int, _vp, _vp, _vp, _u32, _u32, _u32, _int, _vp]),
    "b200_set_path_policy": (_int, [_vp, _int]),
    "b200_set_pair_policy": (_int, [_vp, _int]),
    "b200_set_correction_policy": (_int, [_vp, _int]),
    "b200_set_async_launch": (_int, [_vp, _int]),
    "b200_set_dependent_launch": (_int, [_vp, _int]),
    "b200_launch_flush": (_int, [_vp]),
    "b200_operand_cache_enable": (_int, [_vp, ctypes.c_size_t]),
    "b200_operand_cache_invalidate": (_int, [_vp, _vp, ctypes.c_size_t]),
    "b200_operand_cache_stats": (_int, [_vp, ctypes.POINTER(_u64)]),
    "b200_profile_enable": (_int, [_vp, _int]),
    "b200_profile_read": (_int, [_vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_u64)]),
    "b200_launch_count": (_int, [_vp, ctypes.POINTER(_u64)]),
    # ---- include/primitiv_b200_ops.h ----
    "b200_unary_fw": (_int, [_vp, _int, _int, _vp, _vp, _u64, ctypes.c_float, ctypes.c_int32, _vp]),
    "b200_unary_bw": (_int, [_vp, _int, _int, _vp, _vp, _vp, _vp, _u64, ctypes.c_float, ctypes.c_int32, _int, _vp]),
    "b200_scalar_fw": (_int, [_vp, _int, _int, _vp, _vp, _vp, _u64, _u32, _int, _int, _vp]),
    "b200_binary_fw": (_int, [_vp, _int, _int, _vp, _vp, _vp, _u64, _u32, _int, _int, _vp]),
    "b200_binary_bw": (_int, [_vp, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _u32, _int, _int, _int, _int, _vp]),
    "b200_inplace_add": (_int, [_vp, _int, _vp, _vp, _u64, _u32, _u32, ctypes.c_float, _vp]),
    "b200_inplace_add_ex": (_int, [_vp, _int, _vp, _vp, _u64, _u32, _u32, ctypes.c_float, _int, _vp]),
    "b200_inplace_multiply_const": (_int, [_vp, _int, _vp, _u64, ctypes.c_float, _vp]),
    "b200_fill": (_int, [_vp, _int, _vp, _u64, ctypes.c_float, _vp]),
    "b200_identity": (_int, [_vp, _int, _vp, _u32, _vp]),
    "b200_im2col": (_int, [_vp, _int, _vp, _vp] + [_u32] * 14 + [_int, _vp]),
    "b200_col2im": (_int, [_vp, _int, _vp, _vp] + [_u32] * 14 + [_vp]),
    "b200_max_pool2d_fw": (_int, [_vp, _int, _vp, _vp] + [_u32] * 10 + [_u64, _vp]),
    "b200_max_pool2d_bw": (_int, [_vp, _int, _vp, _vp, _vp, _vp] + [_u32] * 10 + [_u64, _vp]),
    "b200_upload": (_int, [_vp, _int, _vp, _vp, _u64, _vp]),
    "b200_download": (_int, [_vp, _int, _vp, _vp, _u64, _vp]),
    "b200_copy": (_int, [_vp, _int, _vp, _int, _vp, _u64, _vp]),
    "b200_slice_fw": (_int, [_vp, _int, _vp, _vp, _u64, _u32, _u32, _u32, _u64, _vp]),
    "b200_slice_bw": (_int, [_vp, _int, _vp, _vp, _u64, _u32, _u32, _u32, _u64, _u32, _u32, _vp]),
    "b200_slice_bw_ex": (_int, [_vp, _int, _vp, _vp, _u64, _u32, _u32, _u32, _u64, _u32, _u32, _int, _vp]),
    "b200_concat_part": (_int, [_vp, _int, _vp, _vp, _u64, _u32, _u32, _u32, _u64, _u32, _int, _vp]),
    "b200_pick_fw": (_int, [_vp, _int, _vp, _vp, _u32, _vp, _u64, _u32, _u64, _u32, _int, _vp]),
    "b200_pick_bw": (_int, [_vp, _int, _vp, _vp, _u32, _vp, _u64, _u32, _u64, _u32, _int, _vp]),
    "b200_broadcast_fw": (_int, [_vp, _int, _vp, _vp, _u64, _u64, _u32, _vp]),
    "b200_batch_pick_fw": (_int, [_vp, _int, _vp, _vp, _u32, _vp, _u64, _vp]),
    "b200_batch_pick_bw": (_int, [_vp, _int, _vp, _vp, _u32, _vp, _u64, _vp]),
    "b200_transpose": (_int, [_vp, _int, _vp, _vp, _u32, _u32, _u32, _int, _vp]),
    "b200_permute_dims": (_int, [_vp, _int, _vp, _vp, _u32, _vp, _vp, _u32, _int, _vp]),
    "b200_flip": (_int, [_vp, _int, _vp, _vp, _u64, _u32, _u64, _int, _vp]),
    "b200_reduce_fw": (_int, [_vp, _int, _int, _vp, _vp, _u32, _u64, _u64, _vp]),
    "b200_minmax_bw": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _u32, _u64, _u64, _vp]),
    "b200_argminmax": (_int, [_vp, _int, _int, _vp, _vp, _u32, _u64, _u64, _vp]),
    "b200_batch_sum_fw": (_int, [_vp, _int, _vp, _vp, _u64, _u32, _vp]),
    "b200_seed": (_int, [_vp, _u64]),
    "b200_random": (_int, [_vp, _int, _int, ctypes.c_float, ctypes.c_float, _vp, _u64, _vp]),
    "b200_peer_enable": (_int, [_vp, _vp]),
    "b200_stream_barrier": (_int, [ctypes.POINTER(_vp), _int]),
    "b200_peer_sum": (_int, [_vp, _int, ctypes.POINTER(_vp), _int, _vp, _u64, _int, _vp]),
}


class B200Error(RuntimeError):
    def __init__(self, code, what=""):
        self.code = code
        msg = lib().b200_error_string(code).decode() if _LIB is not None else str(code)
        super().__init__("%s (code %d)%s" % (msg, code, (": " + what) if what else ""))


def library_path():
    return os.path.join(_PKG, "libprimitiv_b200.so")


def lib():
    """Loads libprimitiv_b200.so.  Raises if it has not been built: there is no fallback."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not os.path.exists(path):
            raise ImportError(
                "libprimitiv_b200.so is not built (run `python -m primitiv_b200.build`); "
                "primitiv_b200 has no non-CUDA implementation")
        handle = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def _check(code, what=""):
    if code != 0:
        raise B200Error(code, what)


class Context:
    """One b200_ctx (one GPU).  Mirrors the lifetime of a primitiv::devices::B200 object."""

    def __init__(self, device_id=0):
        self._h = _vp()
        _check(lib().b200_ctx_create(device_id, ctypes.byref(self._h)), "b200_ctx_create")
        self.device_id = device_id

    def close(self):
        if self._h:
            lib().b200_ctx_destroy(self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def sm_count(self):
        d, n = _int(), _int()
        _check(lib().b200_ctx_device(self._h, ctypes.byref(d), ctypes.byref(n)))
        return n.value

    def status_poll(self, stream=None):
        c = _int()
        _check(lib().b200_status_poll(self._h, stream, ctypes.byref(c)))
        return c.value

    def gemm_3xtf32_noalloc(self, trans_a, trans_b, A, B, C, m, n, k, accumulate=False, stream=None):
        """One 3xTF32 product whose scratch is a fixed array inside the library: allocates nothing."""
        _check(lib().b200_gemm_3xtf32_noalloc(self._h, int(trans_a), int(trans_b), A, B, C, m, n, k,
                                              int(accumulate), stream), "gemm_3xtf32_noalloc")

    def set_path_policy(self, policy):
        _check(lib().b200_set_path_policy(self._h, policy), "set_path_policy")

    def set_async_launch(self, on):
        """Kernel launches issued by a worker thread (see include/primitiv_b200.h); drained by status_poll()."""
        _check(lib().b200_set_async_launch(self._h, int(on)), "set_async_launch")

    def set_dependent_launch(self, on):
        _check(lib().b200_set_dependent_launch(self._h, int(on)), "set_dependent_launch")

    def operand_cache_enable(self, max_bytes):
        """Keep the packed planes of fp32 operands between calls (0 = off); the caller then owes an
        operand_cache_invalidate for every array it writes."""
        _check(lib().b200_operand_cache_enable(self._h, max_bytes), "operand_cache_enable")

    def operand_cache_invalidate(self, ptr=None, nbytes=0):
        _check(lib().b200_operand_cache_invalidate(self._h, ptr, nbytes), "operand_cache_invalidate")

    def operand_cache_stats(self):
        arr = (_u64 * 4)()
        _check(lib().b200_operand_cache_stats(self._h, arr))
        return dict(hits=arr[0], misses=arr[1], bytes=arr[2], entries=arr[3])

    def set_correction_policy(self, policy):
        """fp32 mode: 0 = correction passes on the bf16 pipe (default), 1 = TF32 planes throughout."""
        _check(lib().b200_set_correction_policy(self._h, policy), "set_correction_policy")

    def set_pair_policy(self, policy):
        _check(lib().b200_set_pair_policy(self._h, policy), "set_pair_policy")

    def profile_enable(self, on=True):
        _check(lib().b200_profile_enable(self._h, int(on)))

    def profile_read(self):
        """-> {kind: (milliseconds, launches)} since the last read."""
        ms = (ctypes.c_double * 4)()
        n = (_u64 * 4)()
        _check(lib().b200_profile_read(self._h, ms, n))
        names = ("gemm_tc", "pack", "gemm_simt", "elementwise")
        return {k: (ms[i], n[i]) for i, k in enumerate(names)}

    def launch_count(self):
        n = _u64()
        _check(lib().b200_launch_count(self._h, ctypes.byref(n)))
        return n.value

    # -- pool --
    def pool_alloc(self, nbytes):
        p, got = _vp(), ctypes.c_size_t()
        _check(lib().b200_pool_alloc(self._h, nbytes, ctypes.byref(p), ctypes.byref(got)), "pool_alloc")
        return p.value, got.value

    def pool_free(self, ptr):
        _check(lib().b200_pool_free(self._h, ptr), "pool_free")

    def pool_release_cached(self):
        _check(lib().b200_pool_release_cached(self._h))

    def pool_set_limit(self, nbytes):
        _check(lib().b200_pool_set_limit(self._h, nbytes))

    def measure_l2_ingest(self, stream=None):
        """-> (bytes per SM clock, GB/s per SM) that bulk copies from L2 into shared memory reach on this GPU."""
        a, b = ctypes.c_double(0), ctypes.c_double(0)
        _check(lib().b200_measure_l2_ingest(self._h, stream, ctypes.byref(a), ctypes.byref(b)), "measure_l2_ingest")
        return a.value, b.value

    def pool_set_guard(self, nbytes):
        _check(lib().b200_pool_set_guard(self._h, nbytes))

    def pool_check_guards(self, stream=None):
        """-> (number of blocks with a damaged guard band, lowest such block or None, side bits)."""
        n, first, side = _u64(0), ctypes.c_void_p(None), ctypes.c_int(0)
        _check(lib().b200_pool_check_guards(self._h, stream, ctypes.byref(n), ctypes.byref(first), ctypes.byref(side)))
        return n.value, first.value, side.value

    def pool_stats(self):
        arr = (_u64 * 4)()
        _check(lib().b200_pool_stats(self._h, arr))
        return dict(in_use=arr[0], cached=arr[1], mallocs=arr[2], hits=arr[3])

    # -- hot path (device pointers as ints) --
    def matmul_fw(self, mode, a, b, y, di, dj, dk, ba, bb, stream=None):
        _check(lib().b200_matmul_fw(self._h, mode, a, b, y, di, dj, dk, ba, bb, stream), "matmul_fw")

    def matmul_bw(self, mode, a, b, gy, ga, gb, di, dj, dk, ba, bb, stream=None):
        _check(lib().b200_matmul_bw(self._h, mode, a, b, gy, ga, gb, di, dj, dk, ba, bb, stream),
               "matmul_bw")

    def matmul_bw_ex(self, mode, a, b, gy, ga, gb, di, dj, dk, ba, bb, accumulate_a=True, accumulate_b=True,
                     stream=None):
        """matmul_bw with `+=` (True) or `=` (False) per gradient; ga / gb may be None to skip one."""
        _check(lib().b200_matmul_bw_ex(self._h, mode, a, b, gy, ga, gb, di, dj, dk, ba, bb,
                                       int(accumulate_a), int(accumulate_b), stream), "matmul_bw_ex")

    def matmul_fw_host(self, mode, a, b, y, di, dj, dk, ba, bb):
        _check(lib().b200_matmul_fw_host(self._h, mode, a, b, y, di, dj, dk, ba, bb), "matmul_fw_host")

    def matmul_bw_host(self, mode, a, b, gy, ga, gb, di, dj, dk, ba, bb):
        _check(lib().b200_matmul_bw_host(self._h, mode, a, b, gy, ga, gb, di, dj, dk, ba, bb),
               "matmul_bw_host")

    def matmul_fw_bw_host(self, mode, a, b, gy, y, ga, gb, di, dj, dk, ba, bb, accumulate_a=True, accumulate_b=True):
        """Forward and both gradients from host buffers in one pipelined pass (addresses as ints, None to skip)."""
        _check(lib().b200_matmul_fw_bw_host(self._h, mode, a, b, gy, y, ga, gb, di, dj, dk, ba, bb,
                                            int(accumulate_a), int(accumulate_b)), "matmul_fw_bw_host")

    def selftest_wait_timeout(self, stream=None):
        _check(lib().b200_selftest_wait_timeout(self._h, stream), "selftest_wait_timeout")

    def op(self, name, *args):
        """Calls any other entry point by name (the elementwise / movement / reduction set)."""
        _check(getattr(lib(), name)(self._h, *args), name)

    def gemm(self, mode, trans_a, trans_b, A, B, C, m, n, k, groups=1, red=1,
             a_gs=0, a_rs=0, b_gs=0, b_rs=0, c_gs=0, accumulate=False, force_path=0, stream=None):
        _check(lib().b200_gemm(self._h, mode, int(trans_a), int(trans_b), A, B, C, m, n, k, groups, red,
                               a_gs, a_rs, b_gs, b_rs, c_gs, int(accumulate), force_path, stream),
               "gemm")

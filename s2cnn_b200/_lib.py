"""ctypes binding of the C ABI in include/s2cnn_b200.h.

The product loads exactly one library, the CUDA build ``lib/libs2cnn_b200.so``; if it is missing
the import of any op fails loudly (there is no CPU or eager fallback).  ``Lib(path)`` can also
wrap the host-emulation build that the CPU test-suite compiles from the same sources.
"""
import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_long, c_size_t, c_void_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
CUDA_LIB_PATH = os.path.join(_HERE, "lib", "libs2cnn_b200.so")

_P = c_void_p


class S2cError(RuntimeError):
    pass


_SIGNATURES = {
    "s2c_last_error": (c_char_p, []),
    "s2c_version": (c_int, []),
    "s2c_launch_count": (c_long, []),
    "s2c_clear_tables": (None, []),
    "s2c_set_table_cache_dir": (None, [c_char_p]),
    "s2c_table_cache_hits": (c_long, []),
    "s2c_table_cache_stores": (c_long, []),
    "s2c_tables_computed": (c_long, []),
    "s2c_is_cuda_build": (c_int, []),
    "s2c_timing_begin": (None, []),
    "s2c_timing_end": (c_int, [c_char_p, c_size_t]),
    "s2c_wigner_d": (c_int, [c_int, c_double, _P]),
    "s2c_quadrature_weights": (c_int, [c_int, _P]),
    "s2c_so3_wigner_table": (c_int, [c_int, c_int, c_int, _P]),
    "s2c_s2_wigner_table": (c_int, [c_int, c_int, c_int, _P]),
    "s2c_s2_ft_matrix": (c_int, [c_int, _P, c_int, _P]),
    "s2c_so3_ft_matrix": (c_int, [c_int, _P, c_int, _P]),
    "s2c_so3_fft_workspace": (c_size_t, [c_long, c_int, c_int]),
    "s2c_so3_fft_workspace_min": (c_size_t, [c_int, c_int]),
    "s2c_so3_rfft": (c_int, [_P, _P, c_long, c_int, c_int, c_int, _P, c_size_t, _P]),
    "s2c_so3_rfft_relu": (c_int, [_P, _P, c_long, c_int, c_int, _P, c_size_t, _P]),
    "s2c_so3_rfft_sums": (c_int, [_P, _P, _P, c_long, c_int, c_int, c_int, _P]),
    "s2c_debug_force_general_path": (None, [c_int]),
    "s2c_debug_plane_chunk": (None, [c_int]),
    "s2c_so3_fft": (c_int, [_P, _P, c_long, c_int, c_int, c_int, _P, c_size_t, _P]),
    "s2c_so3_rifft": (c_int, [_P, _P, c_long, c_int, c_int, c_int, _P, c_int, _P, c_size_t, _P]),
    "s2c_so3_rifft_relu_grad": (c_int, [_P, _P, _P, c_long, c_int, c_int, _P]),
    "s2c_so3_rifft_relu_integrate": (c_int, [_P, _P, c_long, c_int, c_int, _P, c_int, _P]),
    "s2c_s2_conv_relu_so3_rfft": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P]),
    "s2c_so3_rifft_relu_rfft": (c_int, [_P, _P, c_long, c_int, c_int, c_int, _P, c_int, _P]),
    "s2c_so3_rifft_static": (c_int, [_P, _P, c_long, c_int, c_int, c_int, _P, c_int, _P]),
    "s2c_so3_rifft_static_max_bytes": (c_size_t, []),
    "s2c_s2_conv_synthesis_workspace": (c_size_t, [c_int, c_int, c_int]),
    "s2c_s2_conv_synthesis": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, c_size_t, _P]),
    "s2c_so3_ifft": (c_int, [_P, _P, c_long, c_int, c_int, c_int, _P, c_size_t, _P]),
    "s2c_s2_fft_workspace": (c_size_t, [c_long, c_int, c_int]),
    "s2c_s2_fft": (c_int, [_P, c_int, _P, c_long, c_int, c_int, c_int, _P, c_size_t, _P]),
    "s2c_s2_ifft": (c_int, [_P, _P, c_int, c_long, c_int, c_int, c_int, _P, c_size_t, _P]),
    "s2c_so3_mm": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "s2c_so3_mm_tc_status": (c_int, []),
    "s2c_so3_mm_gradx": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "s2c_so3_mm_grady": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "s2c_s2_mm": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "s2c_s2_mm_gradx": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "s2c_s2_mm_grady": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "s2c_rft_forward": (c_int, [_P, _P, _P, c_int, c_int, c_int, _P]),
    "s2c_rft_forward_t": (c_int, [_P, _P, _P, c_int, c_int, c_int, _P]),
    "s2c_rft_backward": (c_int, [_P, _P, _P, c_int, c_int, c_int, _P]),
    "s2c_so3_integrate": (c_int, [_P, _P, c_long, c_int, c_int, _P]),
    "s2c_so3_integrate_backward": (c_int, [_P, _P, _P, c_long, c_int, c_int, _P]),
    "s2c_so3_rotation_matrices": (c_int, [c_int, c_double, c_double, c_double, _P]),
    "s2c_so3_rotate_spectrum": (c_int, [_P, _P, _P, c_int, c_long, c_int, _P]),
    "s2c_project_on_sphere": (c_int, [_P, c_int, _P, c_int, _P, c_int, _P, _P]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


class Lib:
    """A loaded build of the library with typed entry points; ``call`` raises on a non-zero
    status with the library's own message."""

    def __init__(self, path):
        if not os.path.exists(path):
            raise S2cError(
                "s2cnn_b200: compiled library not found at %s - build it with "
                "`python -m s2cnn_b200.build` (there is no fallback path)" % path)
        self.path = path
        self.cdll = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(self.cdll, name)  # AttributeError if a declared symbol is missing
            fn.restype = res
            fn.argtypes = args
        self.is_cuda = bool(self.cdll.s2c_is_cuda_build())
        self._nvtx = self.is_cuda and os.environ.get("S2CNN_B200_NVTX", "0") not in ("", "0")

    def last_error(self):
        return self.cdll.s2c_last_error().decode()

    def call(self, name, *args):
        """One library entry point; with S2CNN_B200_NVTX=1 on a CUDA build the call sits inside an
        NVTX range of the same name (the kernels it launches nest under it in a profiler trace)."""
        if self._nvtx:
            import torch
            torch.cuda.nvtx.range_push(name)
            try:
                rc = getattr(self.cdll, name)(*args)
            finally:
                torch.cuda.nvtx.range_pop()
        else:
            rc = getattr(self.cdll, name)(*args)
        if rc != 0:
            raise S2cError("%s failed (status %d): %s" % (name, rc, self.last_error()))

    def try_call(self, name, *args):
        """Like ``call`` for entry points that answer status 4 ("unsupported", nothing written) for
        sizes outside their fast path: returns False then, True on success, raises otherwise."""
        rc = getattr(self.cdll, name)(*args)
        if rc == 4:
            return False
        if rc != 0:
            raise S2cError("%s failed (status %d): %s" % (name, rc, self.last_error()))
        return True

    def __getattr__(self, name):
        return getattr(self.cdll, name)


_cuda_lib = None


def cuda_lib():
    """The CUDA build (loaded once).  Raises if it has not been built."""
    global _cuda_lib
    if _cuda_lib is None:
        lib = Lib(CUDA_LIB_PATH)
        if not lib.is_cuda:
            raise S2cError("s2cnn_b200: %s is not a CUDA build" % CUDA_LIB_PATH)
        _cuda_lib = lib
    return _cuda_lib

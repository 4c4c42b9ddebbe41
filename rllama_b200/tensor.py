"""Device tensors: the Python mirror of rllama's ``OpenCLTensor`` surface
(``src/tensor_opencl_support.rs:171-412``) over the C ABI, used by the op-level parity tests
the way ``src/tensor.rs``'s ``#[cfg(feature = "opencl")]`` tests use the OpenCL backend.
"""
import ctypes
import sys

import numpy as np

from . import _ffi
from ._ffi import F16, F32, check


def capacity_cols(cols, dtype):
    """Row stride rllama's Tensor uses: cols rounded up to 8 (f32) or 16 (f16)
    (``src/tensor.rs:192-222``)."""
    m = 16 if dtype == F16 else 8
    return (int(cols) + m - 1) // m * m


class Cuda:
    """Counterpart of ``OpenCL`` (``OpenCL::new(verbose, nth_device)``)."""

    def __init__(self, verbose=False, nth_device=0):
        self._h = ctypes.c_void_p()
        check(_ffi.lib().rlb_ctx_create(int(verbose), int(nth_device), ctypes.byref(self._h)))

    def flush(self):
        check(_ffi.lib().rlb_ctx_flush(self._h))

    def kernel_launches(self):
        n = ctypes.c_uint64()
        check(_ffi.lib().rlb_ctx_kernel_launches(self._h, ctypes.byref(n)))
        return n.value

    def close(self):
        if self._h:
            _ffi.lib().rlb_ctx_destroy(self._h)
            self._h = ctypes.c_void_p()

    # -- tensors ------------------------------------------------------------------------
    def upload(self, array):
        """``OpenCL::data_u16_to_gpu``: pads rows to the capacity rule and uploads."""
        a = np.asarray(array)
        if a.ndim == 1:
            a = a.reshape(1, -1)
        dt = F16 if a.dtype == np.float16 else F32
        a = a.astype(np.float16 if dt == F16 else np.float32, copy=False)
        cap = capacity_cols(a.shape[1], dt)
        padded = np.zeros((a.shape[0], cap), dtype=a.dtype)
        padded[:, : a.shape[1]] = a
        t = CudaTensor(self, a.shape[0], a.shape[1], cap, dt)
        t._keep = padded  # must outlive the asynchronous copy
        check(_ffi.lib().rlb_tensor_upload(self._h, padded.ctypes.data_as(ctypes.c_void_p), a.shape[0], a.shape[1], cap, dt,
                                           ctypes.byref(t._h)))
        return t

    def zeros(self, rows, cols, dtype):
        cap = capacity_cols(cols, dtype)
        t = CudaTensor(self, rows, cols, cap, dtype)
        check(_ffi.lib().rlb_tensor_zeros(self._h, rows, cols, cap, dtype, ctypes.byref(t._h)))
        return t


class CudaTensor:
    def __init__(self, cl, rows, cols, cap, dtype):
        self.cl, self.rows, self.cols, self.cap, self.dtype = cl, int(rows), int(cols), int(cap), dtype
        self._h = ctypes.c_void_p()
        self._keep = None

    def wait_until_ready(self):
        check(_ffi.lib().rlb_tensor_wait(self._h))
        self._keep = None

    def to_numpy(self):
        """``data_u16_from_gpu`` + ``OpenCLEvent::wait``; returns the unpadded values."""
        out = np.empty((self.rows, self.cap), dtype=np.float16 if self.dtype == F16 else np.float32)
        ev = ctypes.c_void_p()
        check(_ffi.lib().rlb_tensor_download(self._h, out.ctypes.data_as(ctypes.c_void_p), ctypes.byref(ev)))
        check(_ffi.lib().rlb_event_wait(ev))
        return out[:, : self.cols].copy()

    def copy_inplace(self, other):
        check(_ffi.lib().rlb_copy_inplace(self._h, other._h))

    def transpose_from(self, other):
        check(_ffi.lib().rlb_transpose_from(self._h, other._h))

    def hadamard_product_inplace(self, other):
        check(_ffi.lib().rlb_hadamard_product_inplace(self._h, other._h))

    def silu_inplace(self):
        check(_ffi.lib().rlb_silu_inplace(self._h))

    def matrix_mul_inplace_transposed(self, src, other):
        check(_ffi.lib().rlb_matrix_mul_inplace_transposed(self._h, src._h, other._h))

    def attention_decode(self, q, kcache, vcache, heads, max_seq_len, pos, n_split=1):
        """self <- single-query attention of q over positions 0..pos of the caches."""
        check(_ffi.lib().rlb_attention_decode(self._h, q._h, kcache._h, vcache._h, heads, max_seq_len, pos, n_split))

    def attention_prefill(self, q, kcache, vcache, heads, max_seq_len, start_pos=0, tensor_cores=True):
        """self <- causal attention of the rows of q (row i attends to positions 0..start_pos+i)."""
        check(_ffi.lib().rlb_attention_prefill(self._h, q._h, kcache._h, vcache._h, heads, max_seq_len, start_pos, int(bool(tensor_cores))))

    def attention_decode_static(self, q, kcache, vcache, heads, max_seq_len, pos, n_split=1):
        """Same as ``attention_decode`` but allocation-free: the kernel's scratch is a fixed
        array inside the library (for hosts that cannot allocate on the token path). Fails
        beyond 256 heads or 262144 scratch floats; calls on one device must not overlap."""
        check(_ffi.lib().rlb_attention_decode_static(self._h, q._h, kcache._h, vcache._h, heads, max_seq_len, pos, n_split))

    def free(self):
        if self._h:
            _ffi.lib().rlb_tensor_free(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        # at interpreter shutdown the CUDA runtime may already be gone: leave the memory to process exit
        try:
            if sys is not None and not sys.is_finalizing():
                self.free()
        except Exception:
            pass

"""ctypes binding of the CPU oracle (``oracle/rllama_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's CPU-baseline leg; the product package never imports it.

The oracle restates rllama's CPU forward (``src/transformer.rs:343-382`` and the
``src/tensor.rs`` ops below it); model-level parity with the real Rust binary is
unpinned (the reference holds no golden logits and cannot be compiled here).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

KINDS = {
    "tok_embeddings": 0, "wq": 1, "wk": 2, "wv": 3, "wo": 4, "w1": 5, "w2": 6, "w3": 7,
    "attention_norm": 8, "ffn_norm": 9, "norm": 10, "output": 11,
}


def build(force=False):
    """Compile the oracle with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "rllama_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        vp, ci, cd = ctypes.c_void_p, ctypes.c_int, ctypes.c_double
        L.orc_model_create.restype = vp
        L.orc_model_create.argtypes = [ci, ci, ci, ci, ci, cd, ci, ci, ci]
        L.orc_model_free.argtypes = [vp]
        L.orc_model_set_tensor.argtypes = [vp, ci, ci, vp, ci, ci, ci]
        L.orc_caches_create.restype = vp
        L.orc_caches_create.argtypes = [vp]
        L.orc_caches_free.argtypes = [vp]
        L.orc_caches_shift_left.argtypes = [vp, ci]
        L.orc_caches_get.restype = ctypes.c_float
        L.orc_caches_get.argtypes = [vp, ci, ci, ci, ci, ci]
        L.orc_forward.argtypes = [vp, vp, vp, ci, ci, vp]
        L.orc_matrix_mul_transposed.argtypes = [vp, ci, vp, ci, ci, ci, ci, vp]
        L.orc_matrix_mul_f32.argtypes = [vp, ci, ci, vp, ci, vp]
        L.orc_matrix_mul_naive.argtypes = [vp, ci, ci, vp, ci, ci, vp]
        L.orc_rmsnorm.argtypes = [vp, ci, ci, vp, cd, vp]
        L.orc_softmax.argtypes = [vp, ci, ci]
        L.orc_silu.argtypes = [vp, ctypes.c_int64]
        L.orc_f32_to_f16.argtypes = [vp, vp, ctypes.c_int64]
        L.orc_f16_to_f32.argtypes = [vp, vp, ctypes.c_int64]
        L.orc_freqs_cis.argtypes = [ci, ci, vp]
        L.orc_hw_threads.restype = ci
        _lib = L
    return _lib


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _dt(a):
    if a.dtype == np.float32:
        return 0
    if a.dtype == np.float16:
        return 1
    raise TypeError("oracle tensors are float32 or float16")


class OracleTransformer:
    """rllama's ``Transformer`` on the CPU (``src/transformer.rs:240-383``)."""

    def __init__(self, dim, n_layers, n_heads, ffn, vocab, norm_eps, max_seq_len, force_f16, nthreads=0):
        self.dim, self.n_layers, self.n_heads, self.ffn, self.vocab = dim, n_layers, n_heads, ffn, vocab
        self.max_seq_len = max_seq_len
        self._m = lib().orc_model_create(dim, n_layers, n_heads, ffn, vocab, float(norm_eps), max_seq_len,
                                         int(bool(force_f16)), int(nthreads))

    def set_tensor(self, kind, layer, array):
        a = np.ascontiguousarray(array)
        if a.ndim == 1:
            a = a.reshape(1, -1)
        rc = lib().orc_model_set_tensor(self._m, KINDS[kind], int(layer), _ptr(a), a.shape[0], a.shape[1], _dt(a))
        if rc != 0:
            raise ValueError("oracle rejected tensor %s/%d" % (kind, layer))

    def make_caches(self):
        return OracleCaches(self)

    def forward(self, tokens, start_pos, caches):
        toks = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        out = np.empty(self.vocab, dtype=np.float32)
        rc = lib().orc_forward(self._m, caches._c, _ptr(toks), len(toks), int(start_pos), _ptr(out))
        if rc != 0:
            raise RuntimeError("oracle forward: the reference panics on this call (n>1 with start_pos>0, or out of range)")
        return out

    def __del__(self):
        if getattr(self, "_m", None):
            lib().orc_model_free(self._m)
            self._m = None


class OracleCaches:
    def __init__(self, model):
        self._model = model
        self._c = lib().orc_caches_create(model._m)

    def shift_left(self, shifts):
        lib().orc_caches_shift_left(self._c, int(shifts))

    def get(self, which, layer, head, d, pos):
        return lib().orc_caches_get(self._c, {"k": 0, "v": 1}[which], layer, head, d, pos)

    def __del__(self):
        if getattr(self, "_c", None):
            lib().orc_caches_free(self._c)
            self._c = None


def matrix_mul_transposed(a, b, nthreads=1):
    """``Tensor::matrix_mul_transposed`` (src/tensor.rs:999-1025): a @ b.T in a's dtype."""
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    assert a.dtype == b.dtype and a.shape[1] == b.shape[1]
    out = np.empty((a.shape[0], b.shape[0]), dtype=a.dtype)
    lib().orc_matrix_mul_transposed(_ptr(a), a.shape[0], _ptr(b), b.shape[0], a.shape[1], _dt(a), nthreads, _ptr(out))
    return out


def matrix_mul(a, b):
    """``Tensor::matrix_mul`` on f32 (src/tensor.rs:979-997)."""
    a = np.ascontiguousarray(a, dtype=np.float32); b = np.ascontiguousarray(b, dtype=np.float32)
    out = np.empty((a.shape[0], b.shape[1]), dtype=np.float32)
    lib().orc_matrix_mul_f32(_ptr(a), a.shape[0], a.shape[1], _ptr(b), b.shape[1], _ptr(out))
    return out


def matrix_mul_naive(a, b):
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    out = np.empty((a.shape[0], b.shape[1]), dtype=a.dtype)
    lib().orc_matrix_mul_naive(_ptr(a), a.shape[0], a.shape[1], _ptr(b), b.shape[1], _dt(a), _ptr(out))
    return out


def rmsnorm(x, gain, eps):
    x = np.ascontiguousarray(x, dtype=np.float32); gain = np.ascontiguousarray(gain, dtype=np.float32)
    out = np.empty_like(x)
    lib().orc_rmsnorm(_ptr(x), x.shape[0], x.shape[1], _ptr(gain), float(eps), _ptr(out))
    return out


def softmax(x):
    x = np.array(x, dtype=np.float32, order="C")
    lib().orc_softmax(_ptr(x), x.shape[0], x.shape[1])
    return x


def silu(x):
    x = np.array(x, dtype=np.float32, order="C")
    lib().orc_silu(_ptr(x), x.size)
    return x


def to_f16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.float16)
    lib().orc_f32_to_f16(_ptr(x), _ptr(out), x.size)
    return out


def to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.float16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_f16_to_f32(_ptr(x), _ptr(out), x.size)
    return out


def freqs_cis(head_dim, max_seq_len):
    out = np.empty((max_seq_len, head_dim // 2, 2), dtype=np.float32)
    lib().orc_freqs_cis(head_dim, max_seq_len, _ptr(out))
    return out


def hw_threads():
    return lib().orc_hw_threads()

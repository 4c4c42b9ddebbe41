"""Checkpoint loading: the Python mirror of rllama's ``DataSource`` (``src/data_source.rs``),
``ModelParams`` (``src/model_params.rs``) and of ``Transformer::from_unpickled``
(``src/transformer.rs:242-326``) over the C ABI.
"""
import ctypes

import numpy as np

from . import _ffi
from ._ffi import ModelParams as _CParams
from ._ffi import check

ROWS, COLS, FIRST = 0, 1, 2  # FromPiecesDirection (src/tensor.rs:2340-2343) + "first shard only"


class ModelParams:
    """``ModelParams`` (``src/model_params.rs:4-14``): dim, n_heads, n_layers, norm_eps, vocab_size."""

    def __init__(self, dim, n_heads, n_layers, norm_eps, vocab_size):
        self.dim, self.n_heads, self.n_layers, self.norm_eps, self.vocab_size = dim, n_heads, n_layers, norm_eps, vocab_size

    @classmethod
    def from_json(cls, path):
        p = _CParams()
        check(_ffi.lib().rlb_model_params_from_json(str(path).encode(), ctypes.byref(p)))
        return cls(p.dim, p.n_heads, p.n_layers, p.norm_eps, p.vocab_size)


class DataSource:
    """``DataSource::LLaMASource``: ``<model>/consolidated.NN/{data.pkl, data/<key>}``."""

    def __init__(self, handle, path):
        self._h, self.path = handle, str(path)

    @classmethod
    def from_llama_source(cls, path):
        h = ctypes.c_void_p()
        check(_ffi.lib().rlb_data_source_open(str(path).encode(), ctypes.byref(h)))
        return cls(h, path)

    @classmethod
    def from_vicuna_source(cls, path):
        """``DataSource::from_vicuna_source``: a HuggingFace directory (``config.json``,
        ``pytorch_model.bin.index.json``, ``*.bin`` torch.save archives)."""
        h = ctypes.c_void_p()
        check(_ffi.lib().rlb_data_source_open_vicuna(str(path).encode(), ctypes.byref(h)))
        return cls(h, path)

    @classmethod
    def from_inferred_source(cls, path):
        """``DataSource::from_inferred_source`` (``src/data_source.rs:188-204``)."""
        h = ctypes.c_void_p()
        check(_ffi.lib().rlb_data_source_open_inferred(str(path).encode(), ctypes.byref(h)))
        return cls(h, path)

    def need_to_do_antitranspose(self):
        v = ctypes.c_int32()
        check(_ffi.lib().rlb_data_source_need_antitranspose(self._h, ctypes.byref(v)))
        return bool(v.value)

    def shards(self):
        n = ctypes.c_int32()
        check(_ffi.lib().rlb_data_source_shards(self._h, ctypes.byref(n)))
        return n.value

    def tensor_shape(self, name, direction=ROWS):
        r, c = ctypes.c_int64(), ctypes.c_int64()
        check(_ffi.lib().rlb_data_source_tensor_shape(self._h, name.encode(), direction, ctypes.byref(r), ctypes.byref(c)))
        return r.value, c.value

    def tensor(self, name, direction=ROWS):
        """The named tensor, shards concatenated along ``direction``, as float16."""
        rows, cols = self.tensor_shape(name, direction)
        out = np.empty((rows, cols), dtype=np.float16)
        check(_ffi.lib().rlb_data_source_read_f16(self._h, name.encode(), direction, out.ctypes.data_as(ctypes.c_void_p), rows, cols))
        return out

    def close(self):
        if self._h:
            _ffi.lib().rlb_data_source_free(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def huggingface_llama_model_antitranspose(w, n_heads):
    """``Tensor::huggingface_llama_model_antitranspose`` (``src/tensor.rs:841-909``) on a float16 matrix."""
    w = np.ascontiguousarray(w, dtype=np.float16)
    out = np.empty_like(w)
    check(_ffi.lib().rlb_huggingface_antitranspose_f16(w.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                                                       w.shape[0], w.shape[1], int(n_heads)))
    return out

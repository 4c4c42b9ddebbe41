"""Host-side mirror of rllama's model surface (``src/transformer.rs``) over the C ABI:
``DataSettings``, ``Transformer`` (construction, ``make_caches``, ``forward``) and
``TransformerCaches`` (``true_clone``, ``shift_left``). Names and argument order follow the
reference so that tests read like its own.
"""
import ctypes
import sys
import weakref

import numpy as np

from . import _ffi
from ._ffi import F16, F32, ModelParams, check
from .synthetic import TENSOR_KINDS
from .tensor import Cuda


class DataSettings:
    """``DataSettings`` (``src/transformer.rs:38-109``). ``percentage_to_gpu``: layer ``i`` is resident in
    HBM iff ``i <= round(p * (n_layers - 1))``; this backend has no CPU path, so the matrices of the other
    layers wait in pinned host memory and are copied into an HBM staging buffer inside every forward call."""

    def __init__(self, cl=None):
        self.cl = cl
        self._force_f16 = False
        self._percentage_to_gpu = 1.0

    def force_f16(self):
        self._force_f16 = True
        return self

    def percentage_to_gpu(self, percentage):
        p = float(percentage)
        if p != p:  # NaN -> 0 (src/transformer.rs:91-103)
            p = 0.0
        self._percentage_to_gpu = min(1.0, max(0.0, p))
        return self

    def layers_on_gpu(self, n_layers):
        """Number of layers resident in HBM (src/transformer.rs:262-274; f32 arithmetic, round half away from zero)."""
        x = float(np.float32(self._percentage_to_gpu) * np.float32(n_layers - 1))
        return min(n_layers, int(np.floor(x + 0.5)) + 1)


class Transformer:
    """``Transformer`` (``src/transformer.rs:22-36``, ``:240-383``).

    Construction takes the model dimensions and then tensors by checkpoint name through
    ``set_tensor`` (what ``from_unpickled`` pulls out of the unpickled data source), followed
    by ``finalize``.
    """

    def __init__(self, dim, n_layers, n_heads, ffn_dim, vocab_size, max_seq_len, eps, data_settings=None,
                 tp_rank=0, tp_size=1, verbose=False):
        ds = data_settings or DataSettings()
        self.cl = ds.cl or Cuda(verbose=verbose, nth_device=0)
        self.dim, self.n_layers, self.n_heads, self.ffn_dim = dim, n_layers, n_heads, ffn_dim
        self.vocab_size, self.max_seq_len, self.eps = vocab_size, max_seq_len, eps
        self.force_f16 = ds._force_f16
        self.tp_rank, self.tp_size = tp_rank, tp_size
        p = ModelParams(dim, n_layers, n_heads, ffn_dim, vocab_size, max_seq_len, float(eps), int(ds._force_f16),
                        int(tp_rank), int(tp_size), 1, float(ds._percentage_to_gpu))
        self._h = ctypes.c_void_p()
        check(_ffi.lib().rlb_model_create(self.cl._h, ctypes.byref(p), ctypes.byref(self._h)))

    # -- construction -------------------------------------------------------------------
    @classmethod
    def from_unpickled(cls, dim, n_layers, n_heads, max_seq_len, eps, data_settings, data_source, tp_rank=0, tp_size=1):
        """``Transformer::from_unpickled(emb, dim, n_layers, n_heads, max_seq_len, eps, data_settings,
        data_source)``: loads every tensor of a LLaMA checkpoint by its Meta or HuggingFace name (the embedding
        table included; FFN width and vocabulary size come from the tensors)."""
        self = cls.__new__(cls)
        ds = data_settings or DataSettings()
        self.cl = ds.cl or Cuda(verbose=False, nth_device=0)
        p = ModelParams(dim, n_layers, n_heads, 0, 0, max_seq_len, float(eps), int(ds._force_f16), int(tp_rank), int(tp_size),
                        1, float(ds._percentage_to_gpu))
        self._h = ctypes.c_void_p()
        check(_ffi.lib().rlb_model_from_llama_source(self.cl._h, data_source._h, ctypes.byref(p), ctypes.byref(self._h)))
        self.dim, self.n_layers, self.n_heads = dim, n_layers, n_heads
        self.ffn_dim = int(self.get_stat("ffn_dim"))        # from the w1 tensor
        self.vocab_size = int(self.get_stat("vocab_size"))  # from the embedding table
        self.max_seq_len, self.eps, self.force_f16 = max_seq_len, eps, ds._force_f16
        self.tp_rank, self.tp_size = tp_rank, tp_size
        return self

    def set_tensor(self, kind, layer, array):
        """One whole checkpoint tensor (numpy f16/f32, or a torch tensor on any device)."""
        k = TENSOR_KINDS[kind] if isinstance(kind, str) else int(kind)
        if hasattr(array, "data_ptr"):  # torch tensor: passed by pointer, host or device
            t = array.contiguous()
            if t.is_cuda:  # the library copies on its own stream: the producer must be done
                import torch
                torch.cuda.current_stream(t.device).synchronize()
            if t.dim() == 1:
                t = t.reshape(1, -1)
            dt = {2: F16, 4: F32}[t.element_size()]
            ptr, rows, cols = ctypes.c_void_p(t.data_ptr()), t.shape[0], t.shape[1]
            keep = t
        else:
            a = np.ascontiguousarray(array)
            if a.ndim == 1:
                a = a.reshape(1, -1)
            if a.dtype not in (np.float16, np.float32):
                a = a.astype(np.float32)
            dt = F16 if a.dtype == np.float16 else F32
            ptr, rows, cols = a.ctypes.data_as(ctypes.c_void_p), a.shape[0], a.shape[1]
            keep = a
        check(_ffi.lib().rlb_model_set_tensor(self._h, k, int(layer), ptr, rows, cols, cols, dt))
        del keep

    def finalize(self):
        check(_ffi.lib().rlb_model_finalize(self._h))
        return self

    # -- tensor parallel ----------------------------------------------------------------
    @staticmethod
    def nccl_unique_id():
        buf = ctypes.create_string_buffer(128)
        check(_ffi.lib().rlb_tp_nccl_unique_id(buf))
        return buf.raw

    def nccl_init(self, unique_id):
        check(_ffi.lib().rlb_tp_nccl_init(self._h, ctypes.c_char_p(unique_id)))

    def peer_export(self):
        buf = ctypes.create_string_buffer(128)
        check(_ffi.lib().rlb_tp_peer_export(self._h, buf))
        return buf.raw

    def peer_import(self, handles):
        blob = b"".join(handles)
        check(_ffi.lib().rlb_tp_peer_import(self._h, ctypes.c_char_p(blob), len(handles)))

    def peer_import_local(self, models):
        """Peer exchange buffers of ranks that live in this process: the models of all ranks, by rank."""
        arr = (ctypes.c_void_p * len(models))(*[m._h for m in models])
        check(_ffi.lib().rlb_tp_peer_import_local(self._h, arr, len(models)))

    def set_tp_mode(self, mode):
        check(_ffi.lib().rlb_tp_set_mode(self._h, {"nccl": 0, "push": 1}.get(mode, mode)))

    # -- the reference surface ----------------------------------------------------------
    def make_caches(self):
        return TransformerCaches(self)

    def forward(self, tokens, start_pos, caches):
        """``Transformer::forward``: logits (vocab_size f32) of the last token."""
        toks = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        out = np.empty(self.vocab_size, dtype=np.float32)
        check(_ffi.lib().rlb_forward(self._h, caches._h, toks.ctypes.data_as(ctypes.c_void_p), len(toks), int(start_pos),
                                     out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def forward_greedy(self, tokens, start_pos, caches):
        toks = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        nxt = ctypes.c_int32()
        check(_ffi.lib().rlb_forward_greedy(self._h, caches._h, toks.ctypes.data_as(ctypes.c_void_p), len(toks), int(start_pos),
                                            ctypes.byref(nxt)))
        return nxt.value

    def decode_greedy(self, first_token, start_pos, n_steps, caches):
        """Greedy loop with the token fed back on the device. Returns (tokens, device ms)."""
        out = np.empty(n_steps, dtype=np.int32)
        ms = ctypes.c_float()
        check(_ffi.lib().rlb_decode_greedy(self._h, caches._h, int(first_token), int(start_pos), int(n_steps),
                                           out.ctypes.data_as(ctypes.c_void_p), ctypes.byref(ms)))
        return out, ms.value

    def set_option(self, name, value):
        check(_ffi.lib().rlb_model_set_option(self._h, name.encode(), int(value)))

    def get_stat(self, name):
        v = ctypes.c_double()
        check(_ffi.lib().rlb_model_get_stat(self._h, name.encode(), ctypes.byref(v)))
        return v.value

    def free(self):
        if getattr(self, "_h", None):
            # caches refer to their model inside the library: they go first
            for c in list(getattr(self, "_caches", ())):
                c.free()
            _ffi.lib().rlb_model_free(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        # at interpreter shutdown the CUDA runtime may already be gone: leave the memory to process exit
        try:
            if sys is not None and not sys.is_finalizing():
                self.free()
        except Exception:
            pass


class TransformerCaches:
    """``TransformerCaches`` (``src/transformer.rs:111-113``, ``:200-214``)."""

    def __init__(self, transformer, _handle=None):
        self.transformer = transformer
        self._h = ctypes.c_void_p()
        if _handle is None:
            check(_ffi.lib().rlb_caches_create(transformer._h, ctypes.byref(self._h)))
        else:
            self._h = _handle
        if not hasattr(transformer, "_caches"):
            transformer._caches = weakref.WeakSet()
        transformer._caches.add(self)

    def true_clone(self):
        h = ctypes.c_void_p()
        check(_ffi.lib().rlb_caches_true_clone(self._h, ctypes.byref(h)))
        return TransformerCaches(self.transformer, h)

    def shift_left(self, shifts):
        check(_ffi.lib().rlb_caches_shift_left(self._h, int(shifts)))

    def read(self, which, layer, head, pos):
        hd = self.transformer.dim // self.transformer.n_heads
        out = np.empty(hd, dtype=np.float32)
        check(_ffi.lib().rlb_caches_read(self._h, {"k": 0, "v": 1}[which], layer, head, pos, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def free(self):
        if getattr(self, "_h", None):
            _ffi.lib().rlb_caches_free(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        # at interpreter shutdown the CUDA runtime may already be gone: leave the memory to process exit
        try:
            if sys is not None and not sys.is_finalizing():
                self.free()
        except Exception:
            pass

"""``Tokenizer`` (``src/tokenizer.rs``) over the library's C++ implementation."""
import ctypes
import os
import sys

import numpy as np

from ._ffi import check, lib


class Tokenizer:
    def __init__(self, handle):
        self._h = handle

    @classmethod
    def load(cls, path):
        """``Tokenizer::load`` (``src/tokenizer.rs:46-96``): a SentencePiece model file."""
        h = ctypes.c_void_p()
        check(lib().rlb_tokenizer_load(os.fspath(path).encode(), ctypes.byref(h)))
        return cls(h)

    def n_pieces(self):
        n = ctypes.c_int32()
        check(lib().rlb_tokenizer_n_pieces(self._h, ctypes.byref(n)))
        return n.value

    def id_to_str(self, token_id):
        out = ctypes.c_char_p()
        check(lib().rlb_tokenizer_id_to_str(self._h, int(token_id), ctypes.byref(out)))
        return out.value.decode("utf-8")

    def str_to_id(self, s):
        out = ctypes.c_int32()
        check(lib().rlb_tokenizer_str_to_id(self._h, s.encode("utf-8"), ctypes.byref(out)))
        return None if out.value < 0 else out.value

    def tokenize_to_ids(self, text):
        raw = text.encode("utf-8")
        n = ctypes.c_int32()
        check(lib().rlb_tokenizer_tokenize_to_ids(self._h, raw, None, 0, ctypes.byref(n)))
        ids = np.zeros(n.value, dtype=np.int32)
        check(lib().rlb_tokenizer_tokenize_to_ids(self._h, raw, ids.ctypes.data_as(ctypes.c_void_p), n.value, ctypes.byref(n)))
        return [int(t) for t in ids]

    def free(self):
        if self._h:
            lib().rlb_tokenizer_free(self._h)
            self._h = None

    def __del__(self):
        if not sys.is_finalizing():
            self.free()

"""``TokenSampler`` (``src/token_sampler.rs``): temperature, repetition penalty, top-k, top-p
over the ``vocab x 1`` logits that ``Transformer::forward`` returns.

The reference iterates ``0..logits.rows()`` AFTER transposing the logits to ``1 x vocab``
(``src/token_sampler.rs:105``, ``:113``, ``:121``), so its repetition penalty and its
max-subtraction touch token 0 only. That behaviour is reproduced (``reference_quirks=True``,
the default) so that sampled distributions match the reference's; pass ``False`` for the
behaviour its comments describe.
"""
import ctypes
import sys

import numpy as np

from ._ffi import check, lib


class TokenSampler:
    def __init__(self, reference_quirks=True, rng=None):
        # TokenSampler::new (src/token_sampler.rs:20-28)
        self._temperature = 0.2
        self._top_p = 1.0
        self._top_k = 1
        self._repetition_penalty = 0.8
        self._quirks = reference_quirks
        self._rng = rng or np.random.default_rng()

    def get_temperature(self): return self._temperature
    def get_top_p(self): return self._top_p
    def get_top_k(self): return self._top_k
    def get_repetition_penalty(self): return self._repetition_penalty

    def temperature(self, v): self._temperature = float(v); return self
    def top_p(self, v): self._top_p = float(v); return self
    def top_k(self, v): self._top_k = int(v); return self
    def repetition_penalty(self, v): self._repetition_penalty = float(v); return self

    def candidates(self, logits, existing_tokens=()):
        """The (token, probability) list ``sample`` draws from (after top-k and top-p)."""
        order, probs, _ = self._candidates(logits, existing_tokens)
        return [(int(t), float(p)) for t, p in zip(order, probs)]

    def sample(self, logits, existing_tokens=()):
        """Returns ``(token_id, probability)`` (``src/token_sampler.rs:83-174``)."""
        order, probs, total_p = self._candidates(logits, existing_tokens)
        draw = np.float32(self._rng.uniform(0.0, float(total_p))) if total_p > 0.0 else np.float32(0.0)
        acc = np.float32(0.0)
        for tok, v in zip(order, probs):
            acc += v
            if acc >= draw:
                return int(tok), float(v / total_p)
        return 0, 0.0

    def _candidates(self, logits, existing_tokens):
        x = np.asarray(logits, dtype=np.float32).reshape(-1).copy()
        n = x.shape[0]
        if self._temperature > 0.0:
            x *= np.float32(1.0 / self._temperature)
        touched = range(1) if self._quirks else range(n)
        if self._repetition_penalty != 1.0:
            counts = {}
            for t in existing_tokens:
                counts[int(t)] = counts.get(int(t), 0) + 1
            for idx in touched:
                if idx in counts:
                    x[idx] *= np.float32(self._repetition_penalty ** np.float32(counts[idx]))
        maxv = np.float32(-np.inf)
        for idx in touched if self._quirks else [int(np.argmax(x))]:
            if x[idx] > maxv:
                maxv = x[idx]
        if self._quirks:
            x[0] -= maxv
        else:
            x -= maxv
        with np.errstate(over="ignore", invalid="ignore"):
            e = np.exp(x)
            p = e / np.cumsum(e, dtype=np.float32)[-1]  # sequential f32 sum, as Tensor::softmax does
        # descending by probability, NaNs last (src/token_sampler.rs:127-142)
        key = np.where(np.isnan(p), -np.inf, p)
        order = np.argsort(-key, kind="stable")
        order = order[: self._top_k]
        probs = p[order]
        acc = np.float32(0.0)
        for i, v in enumerate(probs):
            acc += v
            if acc >= self._top_p:
                order, probs = order[: i + 1], probs[: i + 1]
                break
        total_p = np.float32(0.0)
        for v in probs:
            total_p += v
        return order, probs, total_p


class NativeTokenSampler:
    """The library's C++ ``TokenSampler`` (``rlb_sampler_*``): same builder interface; the draw comes
    from a seeded generator (``seed``) where the reference uses ``rand::thread_rng``."""

    def __init__(self, seed=None):
        self._h = ctypes.c_void_p()
        check(lib().rlb_sampler_create(ctypes.byref(self._h)))
        if seed is not None:
            check(lib().rlb_sampler_seed(self._h, int(seed)))

    def _get(self):
        t, p, r, k = ctypes.c_float(), ctypes.c_float(), ctypes.c_float(), ctypes.c_int32()
        check(lib().rlb_sampler_get(self._h, ctypes.byref(t), ctypes.byref(p), ctypes.byref(k), ctypes.byref(r)))
        return [t.value, p.value, k.value, r.value]

    def _set(self, i, v):
        cur = self._get()
        cur[i] = v
        check(lib().rlb_sampler_set(self._h, float(cur[0]), float(cur[1]), int(cur[2]), float(cur[3])))
        return self

    def get_temperature(self): return self._get()[0]
    def get_top_p(self): return self._get()[1]
    def get_top_k(self): return self._get()[2]
    def get_repetition_penalty(self): return self._get()[3]
    def temperature(self, v): return self._set(0, v)
    def top_p(self, v): return self._set(1, v)
    def top_k(self, v): return self._set(2, v)
    def repetition_penalty(self, v): return self._set(3, v)

    @staticmethod
    def _args(logits, existing_tokens):
        x = np.ascontiguousarray(np.asarray(logits, dtype=np.float32).reshape(-1))
        e = np.ascontiguousarray(np.asarray(list(existing_tokens), dtype=np.int32))
        return x, e

    def candidates(self, logits, existing_tokens=()):
        """The (token, probability) list ``sample`` draws from."""
        x, e = self._args(logits, existing_tokens)
        toks = np.zeros(x.shape[0], dtype=np.int32)
        probs = np.zeros(x.shape[0], dtype=np.float32)
        n = ctypes.c_int32()
        check(lib().rlb_sampler_candidates(self._h, x.ctypes.data_as(ctypes.c_void_p), x.shape[0], e.ctypes.data_as(ctypes.c_void_p),
                                           e.shape[0], toks.ctypes.data_as(ctypes.c_void_p), probs.ctypes.data_as(ctypes.c_void_p),
                                           x.shape[0], ctypes.byref(n)))
        return [(int(t), float(p)) for t, p in zip(toks[: n.value], probs[: n.value])]

    def sample(self, logits, existing_tokens=()):
        x, e = self._args(logits, existing_tokens)
        tok, prob = ctypes.c_int32(), ctypes.c_float()
        check(lib().rlb_sampler_sample(self._h, x.ctypes.data_as(ctypes.c_void_p), x.shape[0], e.ctypes.data_as(ctypes.c_void_p),
                                       e.shape[0], ctypes.byref(tok), ctypes.byref(prob)))
        return tok.value, prob.value

    def __del__(self):
        if not sys.is_finalizing() and self._h:
            lib().rlb_sampler_free(self._h)
            self._h = None

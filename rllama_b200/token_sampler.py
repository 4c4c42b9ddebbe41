"""``TokenSampler`` (``src/token_sampler.rs``): temperature, repetition penalty, top-k, top-p
over the ``vocab x 1`` logits that ``Transformer::forward`` returns.

The reference iterates ``0..logits.rows()`` AFTER transposing the logits to ``1 x vocab``
(``src/token_sampler.rs:105``, ``:113``, ``:121``), so its repetition penalty and its
max-subtraction touch token 0 only. That behaviour is reproduced (``reference_quirks=True``,
the default) so that sampled distributions match the reference's; pass ``False`` for the
behaviour its comments describe.
"""
import numpy as np


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

    def sample(self, logits, existing_tokens=()):
        """Returns ``(token_id, probability)`` (``src/token_sampler.rs:83-174``)."""
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
            p = e / np.float32(np.sum(e, dtype=np.float32))
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
        total_p = np.float32(probs.sum(dtype=np.float32))
        draw = np.float32(self._rng.uniform(0.0, float(total_p))) if total_p > 0.0 else np.float32(0.0)
        acc = np.float32(0.0)
        for tok, v in zip(order, probs):
            acc += v
            if acc >= draw:
                return int(tok), float(v / total_p)
        return 0, 0.0

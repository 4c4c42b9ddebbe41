"""Independent float64 LLaMA forward pass (numpy), written from the architecture.

TEST INFRASTRUCTURE ONLY. A second opinion on the C++ oracle: RMSNorm, interleaved-pair
RoPE (theta 10000), causal softmax attention scaled by 1/sqrt(head_dim), SwiGLU FFN,
untied output head. No f16 rounding anywhere, so it is compared with the f32 oracle.
"""
import numpy as np


class F64Transformer:
    def __init__(self, dim, n_layers, n_heads, norm_eps, max_seq_len):
        self.dim, self.n_layers, self.n_heads = dim, n_layers, n_heads
        self.hd = dim // n_heads
        self.eps = float(norm_eps)
        self.max_seq_len = max_seq_len
        self.w = {}
        inv = 1.0 / (10000.0 ** (np.arange(0, self.hd, 2, dtype=np.float64) / self.hd))
        ang = np.outer(np.arange(max_seq_len, dtype=np.float64), inv)
        self.cos, self.sin = np.cos(ang), np.sin(ang)

    def set_tensor(self, kind, layer, array):
        self.w[(kind, layer)] = np.asarray(array, dtype=np.float64)

    def make_caches(self):
        return {"k": [np.zeros((self.max_seq_len, self.n_heads, self.hd)) for _ in range(self.n_layers)],
                "v": [np.zeros((self.max_seq_len, self.n_heads, self.hd)) for _ in range(self.n_layers)]}

    def _norm(self, x, g):
        return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + self.eps) * g

    def _rope(self, x, pos0):
        n = x.shape[0]
        c = self.cos[pos0:pos0 + n][:, None, :]
        s = self.sin[pos0:pos0 + n][:, None, :]
        re, im = x[..., 0::2], x[..., 1::2]
        out = np.empty_like(x)
        out[..., 0::2] = re * c - im * s
        out[..., 1::2] = re * s + im * c
        return out

    def forward(self, tokens, start_pos, caches):
        tokens = np.asarray(tokens)
        n = len(tokens)
        T = start_pos + n
        x = self.w[("tok_embeddings", 0)][tokens]
        for l in range(self.n_layers):
            W = lambda k: self.w[(k, l)]
            a = self._norm(x, W("attention_norm").reshape(-1))
            q = (a @ W("wq").T).reshape(n, self.n_heads, self.hd)
            k = (a @ W("wk").T).reshape(n, self.n_heads, self.hd)
            v = (a @ W("wv").T).reshape(n, self.n_heads, self.hd)
            q, k = self._rope(q, start_pos), self._rope(k, start_pos)
            caches["k"][l][start_pos:T] = k
            caches["v"][l][start_pos:T] = v
            K, V = caches["k"][l][:T], caches["v"][l][:T]
            s = np.einsum("ihd,thd->hit", q, K) / np.sqrt(self.hd)
            mask = np.arange(T)[None, :] > (np.arange(n)[:, None] + start_pos)
            s = np.where(mask[None], -np.inf, s)
            s = s - s.max(axis=-1, keepdims=True)
            p = np.exp(s)
            p /= p.sum(axis=-1, keepdims=True)
            o = np.einsum("hit,thd->ihd", p, V).reshape(n, self.dim)
            h = x + o @ W("wo").T
            f = self._norm(h, W("ffn_norm").reshape(-1))
            g1 = f @ W("w1").T
            g = g1 / (1.0 + np.exp(-g1)) * (f @ W("w3").T)
            x = h + g @ W("w2").T
        x = self._norm(x, self.w[("norm", 0)].reshape(-1))
        return x[-1] @ self.w[("output", 0)].T

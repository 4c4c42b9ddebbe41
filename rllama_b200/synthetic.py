"""Seeded synthetic LLaMA-shape checkpoints and prompts.

Real LLaMA weights are not needed by any measured configuration: weights are i.i.d.
N(0, 0.02) rounded to f16 (rllama's loader accepts only ``torch.HalfStorage``,
``src/unpickler.rs:186-191``, so "f32 weights" are f16-representable values widened
to f32), RMSNorm gains are 1.0, and prompts are uniform random token ids.
Tensor names follow the Meta checkpoint names rllama looks up
(``src/transformer.rs:489-506``, ``:594-617``, ``:296-307``; ``src/embedding.rs:17``).
"""
import numpy as np

# name -> (kind id used by the C ABI, is per-layer)
TENSOR_KINDS = {
    "tok_embeddings": 0, "wq": 1, "wk": 2, "wv": 3, "wo": 4, "w1": 5, "w2": 6, "w3": 7,
    "attention_norm": 8, "ffn_norm": 9, "norm": 10, "output": 11,
}

CONFIGS = {
    # name: dim, n_layers, n_heads, ffn, vocab, norm_eps, f16, prompt, decode, max_seq_len
    "tiny": dict(dim=512, n_layers=8, n_heads=8, ffn=1376, vocab=32000, norm_eps=1e-6, f16=False, prompt=16, decode=64, max_seq_len=80),
    "7b": dict(dim=4096, n_layers=32, n_heads=32, ffn=11008, vocab=32000, norm_eps=1e-6, f16=True, prompt=128, decode=256, max_seq_len=384),
    "13b": dict(dim=5120, n_layers=40, n_heads=40, ffn=13824, vocab=32000, norm_eps=1e-6, f16=True, prompt=512, decode=128, max_seq_len=640),
    "30b": dict(dim=6656, n_layers=60, n_heads=52, ffn=17920, vocab=32000, norm_eps=1e-6, f16=True, prompt=64, decode=256, max_seq_len=320),
    "65b": dict(dim=8192, n_layers=80, n_heads=64, ffn=22016, vocab=32000, norm_eps=1e-6, f16=True, prompt=1792, decode=256, max_seq_len=2048),
}


def tensor_shape(kind, cfg):
    d, F, V = cfg["dim"], cfg["ffn"], cfg["vocab"]
    return {
        "tok_embeddings": (V, d), "output": (V, d),
        "wq": (d, d), "wk": (d, d), "wv": (d, d), "wo": (d, d),
        "w1": (F, d), "w3": (F, d), "w2": (d, F),
        "attention_norm": (1, d), "ffn_norm": (1, d), "norm": (1, d),
    }[kind]


def tensor_list(cfg):
    """(kind, layer) pairs in load order."""
    out = [("tok_embeddings", 0)]
    for l in range(cfg["n_layers"]):
        for k in ("attention_norm", "wq", "wk", "wv", "wo", "ffn_norm", "w1", "w2", "w3"):
            out.append((k, l))
    out += [("norm", 0), ("output", 0)]
    return out


def synth_tensor(kind, layer, cfg, seed=1234):
    """One tensor as float16 (gains as float32 ones), reproducible from (seed, kind, layer)."""
    rows, cols = tensor_shape(kind, cfg)
    if kind in ("attention_norm", "ffn_norm", "norm"):
        return np.ones((rows, cols), dtype=np.float32)
    rng = np.random.Generator(np.random.Philox(key=[int(seed), TENSOR_KINDS[kind] * 4096 + int(layer)]))
    out = np.empty((rows, cols), dtype=np.float16)
    step = max(1, (1 << 24) // cols)
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        out[r0:r1] = (rng.standard_normal((r1 - r0, cols), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    return out


def synth_tokens(n, vocab=32000, seed=4321):
    rng = np.random.Generator(np.random.Philox(key=[int(seed), 0]))
    return rng.integers(0, vocab, size=n, dtype=np.int64).astype(np.int32)


def load_into(model, cfg, seed=1234):
    """Feed every tensor of a synthetic checkpoint to ``model.set_tensor(kind, layer, array)``."""
    for kind, layer in tensor_list(cfg):
        model.set_tensor(kind, layer, synth_tensor(kind, layer, cfg, seed))

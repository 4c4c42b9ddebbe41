"""Model-level checks of the CPU oracle: against the committed golden vectors, against an
independent float64 forward pass, and the reference's defined/undefined call shapes."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from oracle.llama_f64 import F64Transformer
from rllama_b200 import synthetic as S

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make_oracle(cfg, f16, nthreads=4):
    m = O.OracleTransformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"], cfg["norm_eps"],
                            cfg["max_seq_len"], f16, nthreads=nthreads)
    S.load_into(m, cfg)
    return m


def small_cfg(n_layers=2, vocab=2000):
    cfg = dict(S.CONFIGS["tiny"])
    cfg.update(n_layers=n_layers, vocab=vocab)
    return cfg


@pytest.mark.parametrize("case,f16", [("tiny_f32", False), ("tiny_f16", True)])
def test_oracle_reproduces_golden(case, f16):
    g = np.load(os.path.join(GOLDEN, "golden_%s.npz" % case))
    cfg = S.CONFIGS["tiny"]
    m = make_oracle(cfg, f16)
    caches = m.make_caches()
    assert np.array_equal(g["prompt"], S.synth_tokens(cfg["prompt"], cfg["vocab"]))
    logits = m.forward(g["prompt"], 0, caches)
    # libm differences between hosts are allowed a few ulps; tokens must be identical
    assert np.allclose(logits, g["logits_step0"], rtol=0, atol=2e-5)
    for i, want in enumerate(g["tokens"][:8]):
        tok = int(np.argmax(logits))
        assert tok == int(want)
        logits = m.forward([tok], cfg["prompt"] + i, caches)
        if i == 0:
            assert np.allclose(logits, g["logits_step1"], rtol=0, atol=2e-5)


def test_oracle_agrees_with_float64_second_opinion():
    cfg = small_cfg()
    m = make_oracle(cfg, False)
    f = F64Transformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["norm_eps"], cfg["max_seq_len"])
    S.load_into(f, cfg)
    toks = S.synth_tokens(16, cfg["vocab"])
    c, fc = m.make_caches(), f.make_caches()
    lo, lf = m.forward(toks, 0, c), f.forward(toks, 0, fc)
    assert np.abs(lo - lf).max() / np.abs(lf).max() < 1e-5
    for i in range(4):
        tok = int(np.argmax(lf))
        lo, lf = m.forward([tok], 16 + i, c), f.forward([tok], 16 + i, fc)
        assert np.abs(lo - lf).max() / np.abs(lf).max() < 1e-5


def test_f16_run_is_close_to_f32_run():
    cfg = small_cfg()
    toks = S.synth_tokens(12, cfg["vocab"])
    a = make_oracle(cfg, False); b = make_oracle(cfg, True)
    la = a.forward(toks, 0, a.make_caches()); lb = b.forward(toks, 0, b.make_caches())
    assert np.abs(la - lb).max() < 2e-2


def test_prefill_equals_token_by_token_decode():
    """Causality: feeding the prompt one token at a time gives the same last-token logits."""
    cfg = small_cfg()
    m = make_oracle(cfg, False)
    toks = S.synth_tokens(9, cfg["vocab"])
    full = m.forward(toks, 0, m.make_caches())
    c = m.make_caches()
    for i, t in enumerate(toks):
        step = m.forward([int(t)], i, c)
    assert np.abs(full - step).max() / np.abs(full).max() < 1e-5


def test_reference_panics_are_errors():
    cfg = small_cfg()
    m = make_oracle(cfg, False)
    c = m.make_caches()
    m.forward(S.synth_tokens(4, cfg["vocab"]), 0, c)
    with pytest.raises(RuntimeError):  # n x n mask added to n x T scores (src/tensor.rs:576-584)
        m.forward([1, 2], 4, c)
    with pytest.raises(RuntimeError):
        m.forward([cfg["vocab"]], 4, c)  # embedding lookup out of range (src/embedding.rs:50-52)
    with pytest.raises(RuntimeError):
        m.forward([1], cfg["max_seq_len"], c)  # freqs_cis index out of range


def test_cache_layout_and_shift_left():
    cfg = small_cfg(n_layers=1)
    m = make_oracle(cfg, True)
    c = m.make_caches()
    m.forward(S.synth_tokens(6, cfg["vocab"]), 0, c)
    before = [c.get("k", 0, 1, 3, p) for p in range(8)]
    assert before[6] == 0.0 and before[5] != 0.0
    c.shift_left(2)
    after = [c.get("k", 0, 1, 3, p) for p in range(8)]
    assert after[:4] == before[2:6]
    # cached values are f16-representable under force_f16 (src/transformer.rs:138-142)
    v = np.float32(before[2])
    assert np.float32(np.float16(v)) == v

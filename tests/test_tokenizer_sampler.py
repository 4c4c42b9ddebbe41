"""Tokenizer and TokenSampler of the library (C++, ``rllama_b200/csrc/host.cu``) against the
plain-Python restatements of ``src/tokenizer.rs`` and ``src/token_sampler.rs``. CPU only."""
import io
import random
import struct

import numpy as np
import pytest

from oracle import tokenizer_ref
from rllama_b200 import NativeTokenSampler, RllamaError, TokenSampler, Tokenizer


def train_model(byte_fallback=True, vocab=400, seed=7):
    """A small SentencePiece BPE model trained on seeded pseudo-words (stands in for LLaMA's
    tokenizer.model, which is not in the tree): same file format, same piece types."""
    import sentencepiece as spm

    rnd = random.Random(seed)
    syll = ["ka", "lo", "mi", "ren", "tas", "vu", "shi", "dor", "el", "an", "qui", "po", "zé", "ñu", "ty", "ba"]
    words = ["".join(rnd.choice(syll) for _ in range(rnd.randint(1, 4))) for _ in range(400)]
    lines = [" ".join(rnd.choice(words) for _ in range(rnd.randint(3, 12))) + rnd.choice([".", "!", "?", ""]) for _ in range(3000)]
    out = io.BytesIO()
    spm.SentencePieceTrainer.train(sentence_iterator=iter(lines), model_writer=out, vocab_size=vocab, model_type="bpe",
                                   byte_fallback=byte_fallback, character_coverage=1.0, unk_id=0, bos_id=1, eos_id=2, pad_id=-1,
                                   minloglevel=2)
    return out.getvalue(), words


TEXTS = [
    "", " ", "kalo miren", "kalo  miren tas", "kalo\nmiren", "\n\nkalo", "kalo\n", "zéñu ty ba!", "Hello, World?",
    "ka日本 lo", "日本", "ka <0x0A> lo", "</s> ka <s>", "tab\there", "x" * 50, "ka lo mi ren tas vu shi dor el an qui po",
]


@pytest.mark.parametrize("byte_fallback", [True, False])
def test_tokenizer_matches_the_restated_reference(tmp_path, byte_fallback):
    model, words = train_model(byte_fallback=byte_fallback, vocab=400 if byte_fallback else 160)
    path = tmp_path / "tokenizer.model"
    path.write_bytes(model)
    tk = Tokenizer.load(path)
    pieces = tokenizer_ref.load_pieces(model)
    # the protobuf reader agrees with sentencepiece's own
    assert tk.n_pieces() == len(pieces)
    for text, idx in pieces.items():
        assert tk.id_to_str(idx) == text
        assert tk.str_to_id(text) == idx
    assert tk.str_to_id("no such piece ▁") is None
    with pytest.raises(RllamaError):
        tk.id_to_str(len(pieces))
    assert ("<0x0A>" in pieces) == byte_fallback
    rnd = random.Random(1)
    texts = TEXTS + [" ".join(rnd.choice(words) for _ in range(rnd.randint(1, 30))) for _ in range(40)]
    for text in texts:
        want = tokenizer_ref.tokenize_to_ids(pieces, text)
        got = tk.tokenize_to_ids(text)
        assert got == want, text
        assert got[0] == 1
    if not byte_fallback:  # a newline without a "<0x0A>" piece is dropped
        assert tk.tokenize_to_ids("ka\nlo") == tk.tokenize_to_ids("kalo")[:1] + tokenizer_ref.tokenize_to_ids(pieces, "ka\nlo")[1:]


def _varint(v):
    out = b""
    while True:
        b = v & 0x7F
        v >>= 7
        out += bytes([b | (0x80 if v else 0)])
        if not v:
            return out


def _piece(text=None, score=None, ptype=None):
    body = b""
    if text is not None:
        raw = text.encode("utf-8")
        body += b"\x0a" + _varint(len(raw)) + raw
    if score is not None:
        body += b"\x15" + struct.pack("<f", score)
    if ptype is not None:
        body += b"\x18" + _varint(ptype)
    return b"\x0a" + _varint(len(body)) + body


def test_tokenizer_file_edge_cases(tmp_path):
    # hand-assembled ModelProto: a piece without text keeps its index, a repeated text keeps the last
    # index, unknown top-level fields are skipped, an unknown piece type is an error
    blob = (_piece("<unk>", 0.0, 2) + _piece("<s>", 0.0, 3) + _piece(None, -1.0, 1) + _piece("ab", -1.0) + _piece("a", -2.0, 1)
            + _piece("ab", -3.0, 1) + b"\x12\x03abc" + _piece("▁", -4.0, 1) + _piece("b", -5.0, 1))
    path = tmp_path / "hand.model"
    path.write_bytes(blob)
    tk = Tokenizer.load(path)
    assert tk.n_pieces() == 8
    assert tk.str_to_id("ab") == 5 and tk.id_to_str(5) == "ab"
    with pytest.raises(RllamaError):
        tk.id_to_str(3)  # the earlier "ab" lost its entry
    with pytest.raises(RllamaError):
        tk.id_to_str(2)  # no text
    assert tk.tokenize_to_ids("ab a") == [1, 6, 5, 6, 4]
    assert tk.tokenize_to_ids("ac b") == [1, 6, 4, 6, 7]  # "c" matches nothing: one byte skipped
    bad = tmp_path / "bad.model"
    bad.write_bytes(_piece("x", 0.0, 9))
    with pytest.raises(RllamaError):
        Tokenizer.load(bad)
    trunc = tmp_path / "trunc.model"
    trunc.write_bytes(blob[:-3])
    with pytest.raises(RllamaError):
        Tokenizer.load(trunc)
    with pytest.raises(RllamaError):
        Tokenizer.load(tmp_path / "missing.model")


@pytest.mark.parametrize("temperature,top_p,top_k,penalty", [
    (1.0, 1.0, 20, 1.0),     # the CLI's defaults (src/rllama_main.rs:753-757)
    (0.2, 1.0, 1, 0.8),      # TokenSampler::new()
    (0.7, 0.9, 40, 1.3), (1.5, 0.5, 5, 0.5), (0.0, 1.0, 3, 1.0), (1.0, 0.0, 10, 1.0), (1.0, 1.0, 0, 1.0),
])
def test_sampler_candidates_match_the_restated_reference(temperature, top_p, top_k, penalty):
    rng = np.random.default_rng(11)
    for trial in range(6):
        logits = rng.normal(0.0, 3.0, size=997).astype(np.float32)
        existing = [int(t) for t in rng.integers(0, 5, size=trial * 3)]  # token 0 appears among them
        py = TokenSampler().temperature(temperature).top_p(top_p).top_k(top_k).repetition_penalty(penalty)
        cc = NativeTokenSampler(seed=trial).temperature(temperature).top_p(top_p).top_k(top_k).repetition_penalty(penalty)
        want, got = py.candidates(logits, existing), cc.candidates(logits, existing)
        assert [t for t, _ in got] == [t for t, _ in want]
        np.testing.assert_allclose([p for _, p in got], [p for _, p in want], rtol=2e-6, atol=1e-12)
        tok, prob = cc.sample(logits, existing)
        if got:
            assert tok in [t for t, _ in got] and 0.0 < prob <= 1.0 + 1e-6
        else:
            assert (tok, prob) == (0, 0.0)


def test_sampler_quirk_defaults_and_seed():
    s = NativeTokenSampler()
    assert (round(s.get_temperature(), 6), s.get_top_p(), s.get_top_k(), round(s.get_repetition_penalty(), 6)) == (0.2, 1.0, 1, 0.8)
    logits = np.array([2.0, 5.0, 1.0, 4.9], dtype=np.float32)
    # top_k 1 is the arg-max whatever the other settings are
    assert s.sample(logits, [1, 1, 1])[0] == 1
    # the penalty touches token 0 only (src/token_sampler.rs:105): token 1 keeps winning although it repeats
    s2 = NativeTokenSampler().temperature(1.0).top_k(4).repetition_penalty(0.01)
    c_rep = dict(s2.candidates(logits, [1] * 10))
    c_none = dict(s2.candidates(logits, []))
    assert c_rep == c_none
    # ... and even that is cancelled: the "max" loop also sees token 0 only, so its logit always ends as 0
    c_zero = dict(s2.candidates(logits, [0]))
    assert c_zero == c_none
    e = np.exp(np.array([0.0, 5.0, 1.0, 4.9], dtype=np.float32))
    assert abs(c_none[0] - float(e[0] / e.sum())) < 1e-7
    # the same seed repeats the same draws; the draws follow the candidate probabilities
    a = NativeTokenSampler(seed=5).temperature(1.0).top_k(4).repetition_penalty(1.0)
    b = NativeTokenSampler(seed=5).temperature(1.0).top_k(4).repetition_penalty(1.0)
    da = [a.sample(logits)[0] for _ in range(2000)]
    assert da == [b.sample(logits)[0] for _ in range(2000)]
    probs = dict(a.candidates(logits))
    for tok, p in probs.items():
        assert abs(da.count(tok) / 2000.0 - p) < 0.04

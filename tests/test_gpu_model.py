"""Model-level parity of the CUDA path (through the C ABI) against the CPU oracle and the
committed golden vectors. Bounds: per-token logits within 1e-4 relative (max |delta| / max |logit|)
for f32, within 2e-2 max-abs for f16, identical greedy tokens."""
import os

import numpy as np
import pytest

from rllama_b200 import RllamaError
from rllama_b200 import synthetic as S
from helpers import build_pair, cfg_variant, rel_err, top2_margin

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
F32_REL = 1e-4
F16_ABS = 2e-2


def greedy_protocol(model, prompt, steps, caches=None):
    """Prefill at position 0, then `steps` single-token decodes (src/rllama_main.rs:821-901)."""
    caches = caches or model.make_caches()
    logits = [model.forward(prompt, 0, caches)]
    tokens = []
    for i in range(steps):
        tokens.append(int(np.argmax(logits[-1])))
        logits.append(model.forward([tokens[-1]], len(prompt) + i, caches))
    return tokens, logits


def test_tiny_f32_full_protocol_matches_oracle_and_golden(cuda_ctx):
    cfg = S.CONFIGS["tiny"]
    gpu, orc = build_pair(cfg, False, cuda_ctx, oracle_threads=4)
    prompt = S.synth_tokens(cfg["prompt"], cfg["vocab"])
    gt, gl = greedy_protocol(gpu, prompt, cfg["decode"])
    ot, ol = greedy_protocol(orc, prompt, cfg["decode"])
    worst = max(rel_err(a, b) for a, b in zip(gl, ol))
    assert worst <= F32_REL, worst
    assert gt == ot
    g = np.load(os.path.join(GOLDEN, "golden_tiny_f32.npz"))
    assert gt == g["tokens"].tolist()
    for step in (0, 1, 64):
        assert rel_err(gl[step], g["logits_step%d" % step]) <= F32_REL


def test_tiny_f16_full_protocol(cuda_ctx):
    cfg = S.CONFIGS["tiny"]
    gpu, orc = build_pair(cfg, True, cuda_ctx, oracle_threads=4)
    prompt = S.synth_tokens(cfg["prompt"], cfg["vocab"])
    # teacher-forced on the oracle's tokens so that one near-tie cannot hide later steps
    ot, ol = greedy_protocol(orc, prompt, cfg["decode"])
    caches = gpu.make_caches()
    gl = [gpu.forward(prompt, 0, caches)]
    for i, tok in enumerate(ot):
        gl.append(gpu.forward([tok], len(prompt) + i, caches))
    worst = max(float(np.abs(a - b).max()) for a, b in zip(gl, ol))
    assert worst <= F16_ABS, worst
    for a, b in zip(gl, ol):
        if int(np.argmax(a)) != int(np.argmax(b)):
            # a different arg-max is only acceptable at a near-tie of the oracle's own logits
            assert top2_margin(b) <= 2 * float(np.abs(a - b).max())
    g = np.load(os.path.join(GOLDEN, "golden_tiny_f16.npz"))
    assert float(np.abs(gl[0] - g["logits_step0"]).max()) <= F16_ABS
    # free-running greedy sequence
    gt, _ = greedy_protocol(gpu, prompt, cfg["decode"])
    first_diff = next((i for i, (a, b) in enumerate(zip(gt, ot)) if a != b), None)
    if first_diff is not None:
        assert top2_margin(ol[first_diff]) <= 2 * worst, "greedy sequences diverge at step %d away from a near-tie" % first_diff


@pytest.mark.parametrize("f16", [False, True])
def test_7b_shape_two_layers(cuda_ctx, f16):
    """Full 7B layer shapes (dim 4096, 32 heads, FFN 11008, vocab 32000) at reduced depth."""
    cfg = cfg_variant("7b", n_layers=2, max_seq_len=48)
    gpu, orc = build_pair(cfg, f16, cuda_ctx)
    prompt = S.synth_tokens(24, cfg["vocab"])
    ot, ol = greedy_protocol(orc, prompt, 6)
    caches = gpu.make_caches()
    gl = [gpu.forward(prompt, 0, caches)]
    for i, tok in enumerate(ot):
        gl.append(gpu.forward([tok], len(prompt) + i, caches))
    if f16:
        assert max(float(np.abs(a - b).max()) for a, b in zip(gl, ol)) <= F16_ABS
    else:
        assert max(rel_err(a, b) for a, b in zip(gl, ol)) <= F32_REL


@pytest.mark.parametrize("dim,heads", [(5120, 40), (8192, 64)])
def test_wide_rows_one_layer(cuda_ctx, dim, heads):
    """Rows of more than 4096 elements (the 13B and 65B widths): the norm prologue holds the row in
    eight register groups; the attended context grows past two attention splits."""
    cfg = cfg_variant("tiny", dim=dim, n_heads=heads, ffn=1536, n_layers=1, vocab=1024, max_seq_len=160)
    gpu, orc = build_pair(cfg, True, cuda_ctx)
    prompt = S.synth_tokens(126, cfg["vocab"])
    ot, ol = greedy_protocol(orc, prompt, 6)
    caches = gpu.make_caches()
    gl = [gpu.forward(prompt, 0, caches)]
    for i, tok in enumerate(ot):
        gl.append(gpu.forward([tok], len(prompt) + i, caches))
    assert max(float(np.abs(a - b).max()) for a, b in zip(gl, ol)) <= F16_ABS


def teacher_forced_parity(gpu, orc, prompt, steps, f16):
    """Prefill + `steps` decodes on the oracle's own greedy tokens; returns the worst error in the
    measure of the dtype's bound."""
    ot, ol = greedy_protocol(orc, prompt, steps)
    caches = gpu.make_caches()
    gl = [gpu.forward(prompt, 0, caches)]
    for i, tok in enumerate(ot):
        gl.append(gpu.forward([tok], len(prompt) + i, caches))
    if f16:
        return max(float(np.abs(a - b).max()) for a, b in zip(gl, ol))
    return max(rel_err(a, b) for a, b in zip(gl, ol))


def test_30b_width_one_layer(cuda_ctx):
    """The 30B layer shape: rows of 6656 elements (6.5 register groups of the norm prologue: the last
    group is half empty), 52 heads, FFN 17920, full vocabulary; a 64-token prompt goes through the
    tensor-core GEMM, the decode steps through the staged GEMV chain."""
    cfg = cfg_variant("30b", n_layers=1, max_seq_len=80)
    gpu, orc = build_pair(cfg, True, cuda_ctx)
    prompt = S.synth_tokens(64, cfg["vocab"])
    assert teacher_forced_parity(gpu, orc, prompt, 4, True) <= F16_ABS


@pytest.mark.parametrize("base,f16", [("13b", True), ("13b", False), ("65b", True)])
def test_real_ffn_widths_one_layer(cuda_ctx, base, f16):
    """Full 13B / 65B layer shapes at depth 1: the w2 contraction runs over K = 13824 / 22016 (split-K
    at prefill, many ring wraps at decode); in f32 the prefill takes the two-pass TF32 form at
    K = 5120 and 13824."""
    cfg = cfg_variant(base, n_layers=1, vocab=2048, max_seq_len=96)
    gpu, orc = build_pair(cfg, f16, cuda_ctx)
    prompt = S.synth_tokens(72, cfg["vocab"])
    assert teacher_forced_parity(gpu, orc, prompt, 4, f16) <= (F16_ABS if f16 else F32_REL)


@pytest.mark.parametrize("f16", [True, False])
def test_long_context_decode(cuda_ctx, f16):
    """More than a thousand attended positions: every attention CTA of the head's cluster walks
    several batches of cache rows, and the prompt goes through the batched prefill path."""
    cfg = cfg_variant("tiny", dim=256, n_heads=2, ffn=352, n_layers=1, vocab=512, max_seq_len=1100)
    gpu, orc = build_pair(cfg, f16, cuda_ctx)
    prompt = S.synth_tokens(1040, cfg["vocab"])
    ot, ol = greedy_protocol(orc, prompt, 4)
    caches = gpu.make_caches()
    gl = [gpu.forward(prompt, 0, caches)]
    for i, tok in enumerate(ot):
        gl.append(gpu.forward([tok], len(prompt) + i, caches))
    if f16:
        assert max(float(np.abs(a - b).max()) for a, b in zip(gl, ol)) <= F16_ABS
    else:
        assert max(rel_err(a, b) for a, b in zip(gl, ol)) <= F32_REL


def test_odd_head_dim_and_ffn_shapes(cuda_ctx):
    """head_dim 64 and 128, FFN widths that are not multiples of the tile sizes."""
    for over in (dict(dim=256, n_heads=2, ffn=696, n_layers=2, vocab=1000), dict(dim=384, n_heads=6, ffn=1032, n_layers=1, vocab=512)):
        cfg = cfg_variant("tiny", **over)
        for f16 in (False, True):
            gpu, orc = build_pair(cfg, f16, cuda_ctx)
            prompt = S.synth_tokens(5, cfg["vocab"])
            ot, ol = greedy_protocol(orc, prompt, 3)
            caches = gpu.make_caches()
            gl = [gpu.forward(prompt, 0, caches)]
            for i, tok in enumerate(ot):
                gl.append(gpu.forward([tok], len(prompt) + i, caches))
            if f16:
                assert max(float(np.abs(a - b).max()) for a, b in zip(gl, ol)) <= F16_ABS
            else:
                assert max(rel_err(a, b) for a, b in zip(gl, ol)) <= F32_REL


def test_single_token_prompt_and_last_position(cuda_ctx):
    cfg = cfg_variant("tiny", n_layers=2, vocab=2000, max_seq_len=8)
    gpu, orc = build_pair(cfg, False, cuda_ctx)
    gc, oc = gpu.make_caches(), orc.make_caches()
    tok = 7
    for pos in range(8):  # decode from an empty cache up to the maximum sequence length
        a, b = gpu.forward([tok], pos, gc), orc.forward([tok], pos, oc)
        assert rel_err(a, b) <= F32_REL
        tok = int(np.argmax(b))
    with pytest.raises(RllamaError):
        gpu.forward([tok], 8, gc)


def test_prefill_equals_token_by_token_and_chunked(cuda_ctx):
    cfg = cfg_variant("tiny", n_layers=2, vocab=2000, max_seq_len=160)
    gpu, _ = build_pair(cfg, False, cuda_ctx, with_oracle=False)
    toks = S.synth_tokens(11, cfg["vocab"])
    full = gpu.forward(toks, 0, gpu.make_caches())
    c = gpu.make_caches()
    for i, t in enumerate(toks):
        step = gpu.forward([int(t)], i, c)
    assert rel_err(step, full) <= F32_REL
    # a multi-token call at start_pos > 0 (the reference panics there) is a causal chunk
    c2 = gpu.make_caches()
    gpu.forward(toks[:4], 0, c2)
    chunked = gpu.forward(toks[4:], 4, c2)
    assert rel_err(chunked, full) <= F32_REL
    # chunks long enough for the tiled attention kernel, the second one at start_pos > 0 and across its
    # 64-row blocks
    long_toks = S.synth_tokens(150, cfg["vocab"])
    c3 = gpu.make_caches()
    full3 = gpu.forward(long_toks, 0, c3)
    c4 = gpu.make_caches()
    gpu.forward(long_toks[:37], 0, c4)
    chunked3 = gpu.forward(long_toks[37:], 37, c4)
    assert rel_err(chunked3, full3) <= F32_REL
    # the cache rows agree to f32 rounding (the GEMM's K split depends on the number of token tiles, so the
    # summation order of a 150-row call and a 113-row call differs)
    k_full, k_chunk = c3.read("k", 1, 3, 149), c4.read("k", 1, 3, 149)
    assert np.abs(k_full - k_chunk).max() <= 1e-5 * np.abs(k_full).max()


def test_chunked_prefill_f16_on_tensor_cores(cuda_ctx):
    """f16: a prompt given in two chunks (the second one at start_pos > 0 goes through the tensor-core attention
    with its mask offset and through the tensor-core GEMM) agrees with the same prompt given at once and with the
    oracle's logits for it."""
    cfg = cfg_variant("tiny", dim=512, n_heads=4, n_layers=2, vocab=2000, max_seq_len=256)   # head_dim 128
    gpu, orc = build_pair(cfg, True, cuda_ctx)
    toks = S.synth_tokens(200, cfg["vocab"])
    want = orc.forward(toks, 0, orc.make_caches())
    full = gpu.forward(toks, 0, gpu.make_caches())
    c = gpu.make_caches()
    gpu.forward(toks[:70], 0, c)
    chunked = gpu.forward(toks[70:], 70, c)
    assert float(np.abs(full - want).max()) <= F16_ABS
    assert float(np.abs(chunked - want).max()) <= F16_ABS
    assert float(np.abs(chunked - full).max()) <= F16_ABS / 4


def test_device_greedy_loop_equals_host_loop(cuda_ctx):
    cfg = cfg_variant("tiny", n_layers=3, vocab=4000)
    for f16 in (False, True):
        gpu, _ = build_pair(cfg, f16, cuda_ctx, with_oracle=False)
        prompt = S.synth_tokens(9, cfg["vocab"])
        host_tokens, _ = greedy_protocol(gpu, prompt, 20)
        c = gpu.make_caches()
        first = gpu.forward_greedy(prompt, 0, c)
        assert first == host_tokens[0]
        dev_tokens, ms = gpu.decode_greedy(first, len(prompt), 19, c)
        assert dev_tokens.tolist() == host_tokens[1:20]
        assert ms > 0.0
        assert gpu.get_stat("kernels_per_step") == 5 * cfg["n_layers"] + 2


def test_cache_contents_clone_and_shift(cuda_ctx):
    cfg = cfg_variant("tiny", n_layers=2, vocab=2000, max_seq_len=16)
    gpu, orc = build_pair(cfg, True, cuda_ctx)
    toks = S.synth_tokens(6, cfg["vocab"])
    gc, oc = gpu.make_caches(), orc.make_caches()
    gpu.forward(toks, 0, gc); orc.forward(toks, 0, oc)
    hd = cfg["dim"] // cfg["n_heads"]
    for which in ("k", "v"):
        for pos in (0, 5):
            got = gc.read(which, 1, 3, pos)
            want = np.array([oc.get(which, 1, 3, d, pos) for d in range(hd)], dtype=np.float32)
            assert np.abs(got - want).max() <= 2e-3  # f16-rounded values, one ulp apart at most
    assert np.all(gc.read("k", 1, 3, 6) == 0.0)  # Tensor::zeros beyond the written prefix
    clone = gc.true_clone()
    nxt = 11
    a = gpu.forward([nxt], 6, gc)
    assert np.all(clone.read("k", 0, 0, 6) == 0.0)  # the clone is independent
    b = gpu.forward([nxt], 6, clone)
    assert np.array_equal(a, b)
    before = [gc.read("v", 0, 2, p).copy() for p in range(16)]
    gc.shift_left(2)
    for p in range(14):
        assert np.array_equal(gc.read("v", 0, 2, p), before[p + 2])
    assert np.array_equal(gc.read("v", 0, 2, 15), before[15]) and np.array_equal(gc.read("v", 0, 2, 14), before[15])


@pytest.mark.parametrize("f16", [False, True])
def test_percentage_to_gpu_gives_identical_logits(cuda_ctx, f16):
    """--percentage-to-gpu (src/transformer.rs:91-103, :262-274): layers beyond round(p * (L - 1)) are not
    resident in HBM; their matrices are copied in from pinned host memory inside every call and the same
    kernels run, so the logits are bit-identical to the all-resident model."""
    from rllama_b200 import DataSettings, Transformer
    cfg = cfg_variant("tiny", n_layers=8, vocab=2000, max_seq_len=64)
    prompt = S.synth_tokens(40, cfg["vocab"])
    runs = {}
    for p in (1.0, 0.5, 0.0, float("nan")):
        ds = DataSettings(cl=cuda_ctx).percentage_to_gpu(p)
        if f16:
            ds = ds.force_f16()
        m = Transformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"], cfg["max_seq_len"], cfg["norm_eps"], ds)
        S.load_into(m, cfg)
        m.finalize()
        assert int(m.get_stat("layers_on_gpu")) == ds.layers_on_gpu(cfg["n_layers"])
        c = m.make_caches()
        out = [m.forward(prompt, 0, c)]
        for i in range(3):
            out.append(m.forward([int(np.argmax(out[-1]))], len(prompt) + i, c))
        c2 = m.make_caches()
        first = m.forward_greedy(prompt, 0, c2)
        toks, _ = m.decode_greedy(first, len(prompt), 6, c2)   # graph replays with the copies inside
        runs[repr(p)] = (np.stack(out), toks)
        m.free()
    assert DataSettings().percentage_to_gpu(0.5).layers_on_gpu(8) == 5   # round(3.5) = 4 -> layers 0..4
    assert DataSettings().percentage_to_gpu(0.0).layers_on_gpu(8) == 1 and DataSettings().percentage_to_gpu(float("nan")).layers_on_gpu(8) == 1
    assert DataSettings().percentage_to_gpu(7.0).layers_on_gpu(8) == 8
    ref_logits, ref_toks = runs[repr(1.0)]
    for key, (logits, toks) in runs.items():
        assert np.array_equal(logits, ref_logits), key
        assert np.array_equal(toks, ref_toks), key


def test_exchange_wait_runs_out_and_reports(cuda_ctx):
    """A tensor-parallel rank whose peer never sends: the bounded wait of the push exchange runs out, the
    kernels return, forward reports a communication error (status 6) and the context stays usable. Both
    "ranks" are models in this process on one GPU; only rank 0 ever runs, so no kernel waits on another."""
    from rllama_b200 import DataSettings, F32, Transformer
    cfg = cfg_variant("tiny", dim=256, n_heads=4, ffn=512, n_layers=1, vocab=1024, max_seq_len=16)
    ranks = []
    for r in range(2):
        m = Transformer(cfg["dim"], 1, cfg["n_heads"], cfg["ffn"], cfg["vocab"], cfg["max_seq_len"], cfg["norm_eps"],
                        DataSettings(cl=cuda_ctx).force_f16(), tp_rank=r, tp_size=2)
        S.load_into(m, cfg)
        m.finalize()
        ranks.append(m)
    ranks[0].peer_import_local(ranks)
    ranks[0].set_tp_mode("push")
    c = ranks[0].make_caches()
    with pytest.raises(RllamaError) as e:
        ranks[0].forward([5], 0, c)   # one token: the decode chain, whose exchanges wait for rank 1
    assert e.value.status == 6 and "another rank" in str(e.value)
    # the context is intact: an unrelated op still runs and gives the right answer
    t = cuda_ctx.upload(np.arange(12, dtype=np.float32).reshape(3, 4))
    u = cuda_ctx.zeros(4, 3, F32)
    u.transpose_from(t)
    assert np.array_equal(u.to_numpy(), np.arange(12, dtype=np.float32).reshape(3, 4).T)
    for m in ranks:
        m.free()


def test_construction_errors(cuda_ctx):
    from rllama_b200 import DataSettings, Transformer
    cfg = cfg_variant("tiny", n_layers=1, vocab=1000)
    m = Transformer(cfg["dim"], 1, cfg["n_heads"], cfg["ffn"], cfg["vocab"], 16, 1e-6, DataSettings(cl=cuda_ctx))
    with pytest.raises(RllamaError):  # MissingField
        m.finalize()
    with pytest.raises(RllamaError):
        m.set_tensor("wq", 0, np.zeros((cfg["dim"], cfg["dim"] + 16), np.float16))
    with pytest.raises(RllamaError):
        m.set_tensor("wq", 5, np.zeros((cfg["dim"], cfg["dim"]), np.float16))
    with pytest.raises(RllamaError):
        Transformer(100, 1, 3, 64, 100, 16, 1e-6, DataSettings(cl=cuda_ctx))
    S.load_into(m, cfg)
    m.finalize()
    c = m.make_caches()
    with pytest.raises(RllamaError):
        m.forward([1000], 0, c)
    with pytest.raises(RllamaError):
        m.forward(list(range(17)), 0, c)

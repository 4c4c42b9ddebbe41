"""The allocation-free attention entry point (``rlb_attention_decode_static``).

It exists for hosts that cannot let the library allocate while tokens are generated (all of
HBM already handed to weights and caches, or a thread that must not stall the device in
cudaMalloc): its scratch is a fixed array inside the library. The test calls it through the C
ABI several times in a row -- the array keeps the previous call's contents, so every later
call checks that what must start at zero is cleared and that stale records are not read --
and compares each result with the allocating entry point ``rlb_attention_decode`` on the same
inputs and with a float64 statement of the attention itself. The shapes are chosen so that the
fixed array is really used: more than sixteen splits (the splits of a head then meet through
records and an arrival counter in the array, not through a cluster's shared memory) and a
head dimension that takes the general kernel. This file sorts last so that a run stopping at
the first failure has already run every other test.
"""
import numpy as np
import pytest

from rllama_b200 import F16, F32, RllamaError

pytestmark = pytest.mark.gpu


def attention_f64(q, k, v, heads, hd, max_seq, pos):
    """softmax(q K^T / sqrt(hd)) V per head over positions 0..pos in float64 (rllama src/transformer.rs:768-779)."""
    out = np.zeros(heads * hd)
    for h in range(heads):
        K = k[h * max_seq: h * max_seq + pos + 1].astype(np.float64)
        V = v[h * max_seq: h * max_seq + pos + 1].astype(np.float64)
        s = K @ q[0, h * hd:(h + 1) * hd].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        out[h * hd:(h + 1) * hd] = (p / p.sum()) @ V
    return out


def run_both(ctx, rng, heads, hd, max_seq, pos, n_split, dtype):
    q = rng.normal(0, 1, (1, heads * hd)).astype(np.float32)
    k = rng.normal(0, 1, (heads * max_seq, hd)).astype(dtype)
    v = rng.normal(0, 1, (heads * max_seq, hd)).astype(dtype)
    tq, tk, tv = ctx.upload(q), ctx.upload(k), ctx.upload(v)
    dt = F16 if dtype == np.float16 else F32
    ref, got = ctx.zeros(1, heads * hd, dt), ctx.zeros(1, heads * hd, dt)
    ref.attention_decode(tq, tk, tv, heads, max_seq, pos, n_split)
    got.attention_decode_static(tq, tk, tv, heads, max_seq, pos, n_split)
    a, b = ref.to_numpy().astype(np.float64)[0], got.to_numpy().astype(np.float64)[0]
    for t in (tq, tk, tv, ref, got):
        t.free()
    return a, b, attention_f64(q, k, v, heads, hd, max_seq, pos)


# (heads, head_dim, max_seq, pos, n_split). The first three take the path through the fixed array's
# records and counters (24 or 20 splits of 64 positions or more; up to 16 splits would form a cluster);
# the fourth the general kernel (head_dim 192), also through the records; the last four the cluster
# path (16 splits included), which only needs the array to be left alone.
CASES = [(8, 128, 2048, 2047, 24), (8, 128, 2048, 2047, 24), (6, 64, 2048, 2000, 20), (3, 192, 300, 299, 5),
         (8, 128, 2048, 2047, 16), (8, 128, 512, 500, 8), (4, 64, 96, 70, 3), (8, 128, 512, 37, 8)]


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_static_scratch_matches_allocating_entry_point_calls_in_a_row(cuda_ctx, dtype):
    rng = np.random.default_rng(11)
    tol = 2e-3 if dtype == np.float16 else 2e-6  # the bounds of the attention op's own parity test
    for case in CASES:  # each call reuses what the previous one left in the array
        a, b, want = run_both(cuda_ctx, rng, *case, dtype)
        assert np.abs(a).max() > 0
        assert np.abs(a - b).max() <= tol, case
        assert np.abs(b - want).max() <= tol, case


def test_static_scratch_rejects_sizes_beyond_its_maximum(cuda_ctx):
    heads, hd, max_seq = 64, 128, 64
    q = cuda_ctx.zeros(1, heads * hd, F32)
    k = cuda_ctx.zeros(heads * max_seq, hd, F16)
    out = cuda_ctx.zeros(1, heads * hd, F16)
    with pytest.raises(RllamaError) as e:  # 64 * 64 * 130 floats > 262144
        out.attention_decode_static(q, k, k, heads, max_seq, 10, 64)
    assert e.value.status == 7 and "exceed" in str(e.value)
    out.attention_decode_static(q, k, k, heads, max_seq, 10, 16)  # within the limit
    cuda_ctx.flush()

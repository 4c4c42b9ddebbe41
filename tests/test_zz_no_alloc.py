"""The allocation-free attention entry point (``rlb_attention_decode_static``).

It exists for hosts that cannot let the library allocate while tokens are generated (all of
HBM already handed to weights and caches, or a thread that must not stall the device in
cudaMalloc): its scratch is a fixed array inside the library. The test calls it through the C
ABI twice in a row -- the array keeps the previous call's contents, so the second call checks
that everything that must start at zero is cleared -- and compares each result with the
allocating entry point ``rlb_attention_decode`` on the same inputs. This file sorts last so
that a run stopping at the first failure has already run every other test.
"""
import numpy as np
import pytest

from rllama_b200 import F16, F32, RllamaError

pytestmark = pytest.mark.gpu


def run_both(ctx, rng, heads, hd, max_seq, pos, n_split, dtype):
    q = rng.normal(0, 1, (1, heads * hd)).astype(np.float32)
    k = rng.normal(0, 1, (heads * max_seq, hd)).astype(dtype)
    v = rng.normal(0, 1, (heads * max_seq, hd)).astype(dtype)
    tq, tk, tv = ctx.upload(q), ctx.upload(k), ctx.upload(v)
    dt = F16 if dtype == np.float16 else F32
    ref, got = ctx.zeros(1, heads * hd, dt), ctx.zeros(1, heads * hd, dt)
    ref.attention_decode(tq, tk, tv, heads, max_seq, pos, n_split)
    got.attention_decode_static(tq, tk, tv, heads, max_seq, pos, n_split)
    a, b = ref.to_numpy().astype(np.float64), got.to_numpy().astype(np.float64)
    for t in (tq, tk, tv, ref, got):
        t.free()
    return a, b


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_static_scratch_matches_allocating_entry_point_twice_in_a_row(cuda_ctx, dtype):
    rng = np.random.default_rng(11)
    tol = 2e-3 if dtype == np.float16 else 2e-6  # the bounds of the attention op's own parity test
    # two calls in a row with different shapes: the second one reuses what the first left behind
    for heads, hd, max_seq, pos, n_split in [(8, 128, 512, 500, 8), (4, 64, 96, 70, 3), (8, 128, 512, 37, 8)]:
        a, b = run_both(cuda_ctx, rng, heads, hd, max_seq, pos, n_split, dtype)
        assert np.abs(a).max() > 0
        assert np.abs(a - b).max() <= tol, (heads, hd, max_seq, pos, n_split)


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

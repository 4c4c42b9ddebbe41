"""Op-level pins of the CPU oracle: the reference's own unit-test properties
(rllama ``src/tensor.rs:2548-3209``), re-expressed with seeded inputs and the same shape
ranges and tolerances."""
import numpy as np
import pytest

from oracle import oracle as O


def rel_close(a, b, eps):
    """approx::assert_relative_eq!(a, b, epsilon = eps): |a-b| <= eps or relative <= default."""
    a = np.asarray(a, dtype=np.float64); b = np.asarray(b, dtype=np.float64)
    diff = np.abs(a - b)
    ok = (diff <= eps) | (diff <= np.maximum(np.abs(a), np.abs(b)) * np.finfo(np.float32).eps)
    return bool(ok.all())


def rand(rng, r, c, dtype=np.float32):
    return rng.uniform(-1.0, 1.0, size=(r, c)).astype(dtype)


def test_mat_mul_transposed_agrees_with_regular_mat_mul():
    # src/tensor.rs:2554-2578
    rng = np.random.default_rng(1)
    for _ in range(200):
        a, b, c = rng.integers(1, 128, size=3)
        x, y = rand(rng, a, b), rand(rng, b, c)
        assert rel_close(O.matrix_mul(x, y), O.matrix_mul_transposed(x, np.ascontiguousarray(y.T)), 1e-3)


def test_mat_mul_transposed_f32_agrees_f16():
    # src/tensor.rs:2581-2608
    rng = np.random.default_rng(2)
    for _ in range(200):
        a, b, c = rng.integers(1, 128, size=3)
        x, y = rand(rng, a, b), rand(rng, c, b)
        r32 = O.matrix_mul_transposed(x, y)
        r16 = O.matrix_mul_transposed(x.astype(np.float16), y.astype(np.float16))
        assert rel_close(r32, r16.astype(np.float32), 1e-1)


def test_mat_vector_mul_transposed_f32_agrees_f16():
    # src/tensor.rs:2611-2637
    rng = np.random.default_rng(3)
    for _ in range(200):
        a, b = rng.integers(1, 128, size=2)
        x, y = rand(rng, a, b), rand(rng, 1, b)
        r32 = O.matrix_mul_transposed(x, y)
        r16 = O.matrix_mul_transposed(x.astype(np.float16), y.astype(np.float16))
        assert rel_close(r32, r16.astype(np.float32), 1e-1)


def test_gemv_variants_match_naive():
    # src/tensor.rs:2701-2746, :2803-2824: 1..100, 1e-5
    rng = np.random.default_rng(4)
    for _ in range(200):
        r, c = rng.integers(1, 100, size=2)
        m, v = rand(rng, r, c), rand(rng, c, 1)
        assert rel_close(O.matrix_mul_transposed(m, np.ascontiguousarray(v.T)), O.matrix_mul_naive(m, v), 1e-5)
        v2, m2 = rand(rng, 1, r), rand(rng, r, c)
        assert rel_close(O.matrix_mul(v2, m2), O.matrix_mul_naive(v2, m2), 1e-5)


def test_naive_and_fast_are_same_f32():
    # src/tensor.rs:2749-2800
    rng = np.random.default_rng(5)
    for _ in range(100):
        a, b, c = rng.integers(1, 50, size=3)
        x, y = rand(rng, a, b), rand(rng, b, c)
        assert rel_close(O.matrix_mul(x, y), O.matrix_mul_naive(x, y), 1e-5)
    x = rand(rng, 16, 16)
    assert rel_close(O.matrix_mul(x, x), O.matrix_mul_naive(x, x), 1e-5)


def test_naive_and_fast_are_same_f16():
    # src/tensor.rs:2827-2857: 16x32 * 32x16 within 1e-1 (through the transposed f16 kernel)
    rng = np.random.default_rng(6)
    x, y = rand(rng, 16, 32, np.float16), rand(rng, 32, 16, np.float16)
    fast = O.matrix_mul_transposed(x, np.ascontiguousarray(y.T))
    naive = O.matrix_mul_naive(x, y)
    assert rel_close(fast.astype(np.float32), naive.astype(np.float32), 1e-1)


def test_conversions_are_round_to_nearest_even():
    # src/tensor.rs:2881-2920: F16C agrees with the `half` crate (IEEE RNE) exactly
    rng = np.random.default_rng(7)
    x = np.concatenate([rng.uniform(-1, 1, 5000), rng.normal(0, 100, 5000), [0.0, -0.0, 65504.0, 1e-8, 6.1e-5]]).astype(np.float32)
    h = O.to_f16(x)
    assert np.array_equal(h.view(np.uint16), x.astype(np.float16).view(np.uint16))
    assert np.array_equal(O.to_f32(h), h.astype(np.float32))


def test_dot_order_is_lane_then_fold():
    """One output is 8 lane partials (k mod 8) folded as ((l0+l4)+(l1+l5))+((l2+l6)+(l3+l7))
    (src/simd_support.rs:96-116); checked bit for bit against a scalar emulation."""
    rng = np.random.default_rng(8)
    for K in (8, 24, 64, 100):
        a, b = rand(rng, 1, K), rand(rng, 1, K)
        got = O.matrix_mul_transposed(a, b)[0, 0]
        kp = (K + 7) // 8 * 8
        ap = np.zeros(kp, np.float32); bp = np.zeros(kp, np.float32)
        ap[:K], bp[:K] = a[0], b[0]
        lanes = np.zeros(8, np.float32)
        for k0 in range(0, kp, 8):
            for l in range(8):
                # fused multiply-add: exact product, one rounding
                lanes[l] = np.float32(np.float64(ap[k0 + l]) * np.float64(bp[k0 + l]) + np.float64(lanes[l]))
        s = [np.float32(lanes[i] + lanes[i + 4]) for i in range(4)]
        want = np.float32(np.float32(s[0] + s[1]) + np.float32(s[2] + s[3]))
        assert got == want


def test_softmax_has_no_max_subtraction_and_sums_to_one():
    rng = np.random.default_rng(9)
    x = rng.normal(0, 2, size=(5, 37)).astype(np.float32)
    p = O.softmax(x)
    e = np.exp(x.astype(np.float64))
    assert np.allclose(p, e / e.sum(axis=1, keepdims=True), rtol=1e-5)
    big = np.full((1, 4), 100.0, dtype=np.float32)  # exp overflows to inf -> inf/inf = NaN, as in the reference
    assert np.isnan(O.softmax(big)).all()


def test_rmsnorm_and_silu():
    rng = np.random.default_rng(10)
    x = rng.normal(0, 1, size=(3, 512)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, size=(1, 512)).astype(np.float32)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6) * g
    assert np.allclose(O.rmsnorm(x, g, 1e-6), want, rtol=2e-6, atol=1e-7)
    v = rng.normal(0, 3, size=1000).astype(np.float32)
    assert np.allclose(O.silu(v), v / (1 + np.exp(-v.astype(np.float64))), rtol=1e-6, atol=1e-7)


def test_freqs_cis_table():
    t = O.freqs_cis(64, 80)
    inv = 1.0 / (10000.0 ** (np.arange(0, 64, 2, dtype=np.float64) / 64))
    ang = np.outer(np.arange(80, dtype=np.float64), inv)
    assert np.array_equal(t[..., 0], np.cos(ang).astype(np.float32))
    assert np.array_equal(t[..., 1], np.sin(ang).astype(np.float32))


def test_thread_count_does_not_change_results():
    rng = np.random.default_rng(11)
    x, y = rand(rng, 37, 200), rand(rng, 53, 200)
    assert np.array_equal(O.matrix_mul_transposed(x, y, nthreads=1), O.matrix_mul_transposed(x, y, nthreads=5))

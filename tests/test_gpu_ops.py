"""Op-level parity of the CUDA backend against the CPU oracle: the reference's
``#[cfg(feature = "opencl")]`` tests (rllama ``src/tensor.rs:2922-3208``) with seeded inputs,
same shapes and tolerances, plus the f32 variants the CUDA backend adds."""
import numpy as np
import pytest

from oracle import oracle as O
from rllama_b200 import F16, F32, RllamaError

pytestmark = pytest.mark.gpu


def rel_close(a, b, eps, f16_ulps=0):
    """|a - b| <= eps, or (for f16 results) within `f16_ulps` units in the last place of b:
    a different summation order may move an f16-rounded result by one ulp, which exceeds a
    fixed epsilon once |b| >= 16."""
    a = np.asarray(a, dtype=np.float64); b = np.asarray(b, dtype=np.float64)
    tol = np.full(b.shape, eps)
    if f16_ulps:
        tol = np.maximum(tol, f16_ulps * np.spacing(np.abs(b).astype(np.float16)).astype(np.float64))
    return bool((np.abs(a - b) <= tol).all())


def gpu_mmt(ctx, x, y):
    a, b = ctx.upload(x), ctx.upload(y)
    c = ctx.zeros(x.shape[0], y.shape[0], F16 if x.dtype == np.float16 else F32)
    c.matrix_mul_inplace_transposed(a, b)
    out = c.to_numpy()
    for t in (a, b, c):
        t.free()
    return out


def test_matrix_mul_transposed_512x1024_768x1024(cuda_ctx):
    # src/tensor.rs:2922-2951 (1e-1 against the f32 CPU result)
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, (512, 1024)).astype(np.float32); y = rng.uniform(-1, 1, (768, 1024)).astype(np.float32)
    want = O.matrix_mul_transposed(x, y, nthreads=4)
    got = gpu_mmt(cuda_ctx, x.astype(np.float16), y.astype(np.float16)).astype(np.float32)
    assert rel_close(got, want, 1e-1)
    got32 = gpu_mmt(cuda_ctx, x, y)
    assert np.abs(got32 - want).max() <= 1e-4 * np.abs(want).max()


def test_matrix_mul_transposed_1024_square(cuda_ctx):
    # src/tensor.rs:2954-2983
    rng = np.random.default_rng(1)
    x = rng.uniform(-1, 1, (1024, 1024)).astype(np.float16); y = rng.uniform(-1, 1, (1024, 1024)).astype(np.float16)
    want = O.matrix_mul_transposed(x, y, nthreads=4).astype(np.float32)
    got = gpu_mmt(cuda_ctx, x, y).astype(np.float32)
    assert rel_close(got, want, 1e-1)


@pytest.mark.parametrize("n,M,K", [(300, 40000, 1024), (640, 38000, 520), (129, 40000, 256)])
def test_matrix_mul_transposed_many_tiles(cuda_ctx, n, M, K):
    """Enough output tiles for every schedule of the tensor-core GEMM: whole 256-token x 256-row tiles handed
    out round-robin plus a K-split remainder, a partial last token tile, a partial last row tile, a K that is not
    a multiple of the 64-column k-block."""
    rng = np.random.default_rng(9)
    x = rng.uniform(-1, 1, (n, K)).astype(np.float16); w = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    want = O.matrix_mul_transposed(x, w, nthreads=8).astype(np.float32)
    got = gpu_mmt(cuda_ctx, x, w).astype(np.float32)
    assert got.shape == want.shape
    assert rel_close(got, want, 1e-2, f16_ulps=1)
    assert (got == want).mean() > 0.97  # same f32 sums up to order, one f16 rounding


def test_gemm_epilogue_rounding_matches_plain_conversions(tmp_path):
    """The prefill GEMM rounds its f32 accumulators to f16 values with a packed conversion and a mixed-precision
    add (csrc/round_f16.h). tests/cuda/round_pair_check.cu compares that on the device, bit for bit, with
    __float2half_rn / __half2float: every f16 bit pattern for the widening (subnormals, infinities, NaN), 2^26 f32
    bit patterns and their negatives for the rounding."""
    import os, shutil, subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc on this machine to build the check program")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "round_pair_check")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-I", os.path.join(root, "rllama_b200", "csrc"),
                    "-o", exe, os.path.join(root, "tests", "cuda", "round_pair_check.cu")], check=True, capture_output=True, text=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "widening mismatches: 0; rounding mismatches: 0" in r.stdout


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_matrix_mul_transposed_random_sizes(cuda_ctx, dtype):
    # src/tensor.rs:2986-3090: sizes up to 300, including one row on either side; 1e-2
    rng = np.random.default_rng(2)
    shapes = [(int(a), int(b), int(c)) for a, b, c in rng.integers(1, 300, size=(40, 3))]
    shapes += [(1, int(b), int(c)) for b, c in rng.integers(1, 300, size=(20, 2))]
    shapes += [(int(a), int(b), 1) for a, b in rng.integers(1, 300, size=(20, 2))]
    shapes += [(1, 7, 1), (1, 300, 300), (300, 1, 300), (4, 16, 4)]
    for a, b, c in shapes:
        x = rng.uniform(-1, 1, (a, b)).astype(dtype); y = rng.uniform(-1, 1, (c, b)).astype(dtype)
        want = O.matrix_mul_transposed(x, y).astype(np.float32)
        got = gpu_mmt(cuda_ctx, x, y).astype(np.float32)
        assert got.shape == want.shape
        assert rel_close(got, want, 1e-2 if dtype == np.float16 else 1e-4, f16_ulps=1 if dtype == np.float16 else 0), (a, b, c)


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_silu_hadamard_transpose_copy(cuda_ctx, dtype):
    # src/tensor.rs:3093-3208, 1e-2 (f16)
    rng = np.random.default_rng(3)
    tol = 1e-2 if dtype == np.float16 else 1e-6
    for _ in range(20):
        r, c = (int(v) for v in rng.integers(1, 300, size=2))
        x = rng.uniform(-1, 1, (r, c)).astype(dtype); y = rng.uniform(-1, 1, (r, c)).astype(dtype)
        t = cuda_ctx.upload(x); t.silu_inplace()
        assert rel_close(t.to_numpy().astype(np.float32), O.silu(x.astype(np.float32)).reshape(r, c), tol)
        t2 = cuda_ctx.upload(x); u = cuda_ctx.upload(y); t2.hadamard_product_inplace(u)
        assert rel_close(t2.to_numpy().astype(np.float32), x.astype(np.float32) * y.astype(np.float32), tol)
        tt = cuda_ctx.zeros(c, r, F16 if dtype == np.float16 else F32); tt.transpose_from(u)
        assert np.array_equal(tt.to_numpy(), y.T)
        cp = cuda_ctx.zeros(r, c, F16 if dtype == np.float16 else F32); cp.copy_inplace(u)
        assert np.array_equal(cp.to_numpy(), y)
        for h in (t, t2, u, tt, cp):
            h.free()


def test_f16_result_is_a_rounded_f32_accumulation(cuda_ctx):
    """f16 operands: exact products, f32 accumulation, one RNE rounding of the result
    (src/tensor.rs:1476-1666) -- so the GPU may differ from the oracle by summation order
    only, i.e. by at most one f16 ulp of the result."""
    rng = np.random.default_rng(4)
    x = (rng.normal(0, 1, (1, 4096))).astype(np.float16); w = (rng.normal(0, 0.02, (512, 4096))).astype(np.float16)
    want = O.matrix_mul_transposed(x, w)
    got = gpu_mmt(cuda_ctx, x, w)
    ulp = np.spacing(np.abs(want).astype(np.float16)).astype(np.float32)
    assert (np.abs(got.astype(np.float32) - want.astype(np.float32)) <= ulp).all()
    assert (got.view(np.uint16) == want.view(np.uint16)).mean() > 0.97


def test_shape_and_dtype_errors(cuda_ctx):
    a = cuda_ctx.upload(np.zeros((4, 8), np.float32)); b = cuda_ctx.upload(np.zeros((4, 9), np.float32))
    c = cuda_ctx.zeros(4, 4, F32)
    with pytest.raises(RllamaError):  # "Invalid matrix multiplication" (src/tensor.rs:1261-1266)
        c.matrix_mul_inplace_transposed(a, b)
    h = cuda_ctx.upload(np.zeros((4, 8), np.float16))
    with pytest.raises(RllamaError):  # different dtypes (:1267-1272)
        c.matrix_mul_inplace_transposed(a, h)
    with pytest.raises(RllamaError):
        a.hadamard_product_inplace(b)
    assert cuda_ctx.kernel_launches() > 0


def attention_reference(q, k, v, heads, hd, max_seq, pos):
    """float64 softmax(q K^T / sqrt(hd)) V per head over positions 0..pos
    (rllama src/transformer.rs:768-779)."""
    out = np.zeros(heads * hd)
    for h in range(heads):
        K = k[h * max_seq: h * max_seq + pos + 1].astype(np.float64)
        V = v[h * max_seq: h * max_seq + pos + 1].astype(np.float64)
        s = K @ q[0, h * hd:(h + 1) * hd].astype(np.float64) / np.sqrt(hd)
        p = np.exp(s - s.max())
        out[h * hd:(h + 1) * hd] = (p / p.sum()) @ V
    return out


def attention_case(rng, heads, hd, max_seq, dtype):
    q = rng.normal(0, 1, (1, heads * hd)).astype(np.float32)
    k = rng.normal(0, 1, (heads * max_seq, hd)).astype(dtype)
    v = rng.normal(0, 1, (heads * max_seq, hd)).astype(dtype)
    return q, k, v


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_attention_decode_op(cuda_ctx, dtype):
    rng = np.random.default_rng(5)
    for heads, hd, max_seq, pos, n_split in [(4, 64, 96, 70, 1), (4, 64, 96, 70, 4), (3, 128, 300, 299, 5), (2, 128, 64, 0, 2),
                                             (8, 128, 2048, 2047, 16), (8, 128, 2048, 2047, 24), (5, 64, 1536, 1400, 12)]:
        q, k, v = attention_case(rng, heads, hd, max_seq, dtype)
        tq, tk, tv = cuda_ctx.upload(q), cuda_ctx.upload(k), cuda_ctx.upload(v)
        out = cuda_ctx.zeros(1, heads * hd, F16 if dtype == np.float16 else F32)
        out.attention_decode(tq, tk, tv, heads, max_seq, pos, n_split)
        got = out.to_numpy().astype(np.float64)[0]
        want = attention_reference(q, k, v, heads, hd, max_seq, pos)
        assert np.abs(got - want).max() <= (2e-3 if dtype == np.float16 else 2e-6), (heads, hd, max_seq, pos, n_split)
        for t in (tq, tk, tv, out):
            t.free()
    with pytest.raises(RllamaError):
        bad = cuda_ctx.zeros(1, 8, F32)
        bad.attention_decode(bad, bad, bad, 1, 4, 9, 1)


def prefill_reference(q, k, v, heads, hd, max_seq, start_pos):
    """float64 causal attention: row i over positions 0..start_pos+i (rllama src/transformer.rs:727-781,
    mask src/tensor.rs:496-508)."""
    n = q.shape[0]
    out = np.zeros((n, heads * hd))
    for h in range(heads):
        K = k[h * max_seq:(h + 1) * max_seq].astype(np.float64)
        V = v[h * max_seq:(h + 1) * max_seq].astype(np.float64)
        s = q[:, h * hd:(h + 1) * hd].astype(np.float64) @ K.T / np.sqrt(hd)
        for i in range(n):
            t = start_pos + i + 1
            p = np.exp(s[i, :t] - s[i, :t].max())
            out[i, h * hd:(h + 1) * hd] = (p / p.sum()) @ V[:t]
    return out


@pytest.mark.parametrize("heads,hd,max_seq,start_pos,n", [(3, 128, 512, 0, 300), (2, 64, 700, 0, 650), (2, 128, 400, 37, 200),
                                                          (5, 64, 160, 100, 33), (1, 128, 2048, 0, 1792)])
def test_attention_prefill_on_tensor_cores(cuda_ctx, heads, hd, max_seq, start_pos, n):
    """The tensor-core kernel (f16 cache, q and the softmax weights as two f16 halves each) against float64 and
    against the CUDA-core kernel: partial last query block, several cache tiles, the diagonal tiles' mask, a
    chunk at start_pos > 0, cache rows beyond the attended prefix holding other data."""
    rng = np.random.default_rng(7)
    q = rng.normal(0, 1.3, (n, heads * hd)).astype(np.float32)
    k = rng.normal(0, 1.0, (heads * max_seq, hd)).astype(np.float16)
    v = rng.normal(0, 1.0, (heads * max_seq, hd)).astype(np.float16)
    tq, tk, tv = cuda_ctx.upload(q), cuda_ctx.upload(k), cuda_ctx.upload(v)
    tc, cc = cuda_ctx.zeros(n, heads * hd, F16), cuda_ctx.zeros(n, heads * hd, F16)
    tc.attention_prefill(tq, tk, tv, heads, max_seq, start_pos, tensor_cores=True)
    cc.attention_prefill(tq, tk, tv, heads, max_seq, start_pos, tensor_cores=False)
    got, other = tc.to_numpy().astype(np.float64), cc.to_numpy().astype(np.float64)
    want = prefill_reference(q, k, v, heads, hd, max_seq, start_pos)
    # both kernels round an f32 result to f16 once: half an f16 ulp of values up to ~4, plus summation-order noise
    assert np.abs(got - want).max() <= 2e-3
    assert np.abs(other - want).max() <= 2e-3
    # the two kernels agree except where f32 noise flips the f16 rounding
    assert (got != other).mean() < 0.02
    for t in (tq, tk, tv, tc, cc):
        t.free()


def test_attention_prefill_split_precision(cuda_ctx):
    """An f32 output would show the precision of the two-half split; through the f16 output it shows as
    agreement of the rounded results: values chosen so that the softmax is sharp (large scores) and flat
    (tiny scores) in different heads."""
    rng = np.random.default_rng(8)
    heads, hd, max_seq, n = 2, 128, 256, 256
    q = rng.normal(0, 1.0, (n, heads * hd)).astype(np.float32)
    q[:, :hd] *= 6.0      # head 0: sharp softmax
    q[:, hd:] *= 0.01     # head 1: nearly uniform weights
    k = rng.normal(0, 1.0, (heads * max_seq, hd)).astype(np.float16)
    v = rng.normal(0, 1.0, (heads * max_seq, hd)).astype(np.float16)
    tq, tk, tv = cuda_ctx.upload(q), cuda_ctx.upload(k), cuda_ctx.upload(v)
    tc = cuda_ctx.zeros(n, heads * hd, F16)
    tc.attention_prefill(tq, tk, tv, heads, max_seq, 0)
    got = tc.to_numpy().astype(np.float64)
    want = prefill_reference(q, k, v, heads, hd, max_seq, 0)
    ulp = np.spacing(np.abs(want).astype(np.float16)).astype(np.float64)
    assert (np.abs(got - want) <= 0.51 * ulp + 1e-6).mean() > 0.99  # correctly rounded almost everywhere (a lost low half would flip ~10 %)
    assert np.abs(got - want).max() <= 2e-3
    for t in (tq, tk, tv, tc):
        t.free()

// CPU oracle for the rllama decode / prefill hot path.
//
// TEST INFRASTRUCTURE ONLY. This file restates, from the published algorithm, the CPU
// forward pass of Noeda/rllama (non-OpenCL build) so that the CUDA library can be
// checked against it. Nothing in the product path may call it; only the test-suite,
// the smoke check and the benchmark's CPU-baseline leg do.
//
// PARITY UNPINNED above the op level: the reference holds no golden logits or token
// transcripts, and its Rust sources cannot be compiled where this oracle was written.
// What is pinned are the reference's own op-level unit-test properties
// (src/tensor.rs:2548-3209), re-expressed in the test-suite, and an independent
// float64 forward pass used as a second opinion.
//
// Arithmetic that is reproduced literally (citations are paths inside rllama):
//  * every "transposed" contraction (src/tensor.rs:1250-1668 GEMM, :1837-1918 GEMV,
//    :1923-1983 vector*matrix) accumulates eight f32 lane partials (lane = k mod 8)
//    with fused multiply-add and folds them as ((l0+l4)+(l1+l5))+((l2+l6)+(l3+l7))
//    (src/simd_support.rs:96-116);
//  * the f16 GEMM widens operands to f32, accumulates in f32 and rounds the result
//    to f16 with round-to-nearest-even (src/tensor.rs:1476-1666);
//  * the plain matrix_mul used for prefill scores is a sequential-k FMA per output
//    (src/tensor.rs:1050-1115);
//  * softmax has no max subtraction and a left-to-right f32 sum (src/tensor.rs:479-494);
//  * RMSNorm is pow(2) -> sequential mean -> +eps -> 1/sqrt -> scale -> gain
//    (src/transformer.rs:476-480);
//  * RoPE rotates interleaved pairs with a table built in f64 (src/transformer.rs:823-885);
//  * the KV cache is head_dim x max_seq_len per head, f16 when force_f16
//    (src/transformer.rs:129-160, :751-766);
//  * f16 rounding points of a --f16 run (src/transformer.rs:538-570, :666-819).
//
// Build: see oracle/Makefile (g++ -O2 -mavx2 -mfma -mf16c -shared -fPIC -pthread).

#include <immintrin.h>
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace {

// ---------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------

typedef uint16_t f16bits;

inline float h2f(f16bits h) { return _cvtsh_ss(h); }
inline f16bits f2h(float f) { return _cvtss_sh(f, 0); }  // imm 0: round to nearest even
inline float round_f16(float f) { return h2f(f2h(f)); }

// src/simd_support.rs:96-116
inline float hsum8(__m256 v) {
    __m256 v2 = _mm256_permute2f128_ps(v, v, 1);
    v = _mm256_add_ps(v, v2);
    v = _mm256_hadd_ps(v, v);
    v = _mm256_hadd_ps(v, v);
    return _mm256_cvtss_f32(v);
}

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// A persistent worker pool (the reference keeps a rayon pool alive for the whole run,
// src/rllama_main.rs:148-157); a fork-join per contraction would otherwise dominate decode.
class Pool {
  public:
    explicit Pool(int n) : n_(n) {
        for (int t = 1; t < n_; t++) workers_.emplace_back([this, t]() { run(t); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> g(mu_);
            stop_ = true;
            gen_++;
        }
        cv_.notify_all();
        for (auto& w : workers_) w.join();
    }
    int size() const { return n_; }
    void parallel(int64_t n, const std::function<void(int64_t, int64_t)>& fn) {
        if (n_ <= 1 || n <= 1) { fn(0, n); return; }
        {
            std::lock_guard<std::mutex> g(mu_);
            fn_ = &fn; total_ = n; pending_ = n_ - 1; gen_++;
        }
        cv_.notify_all();
        fn(0, n / n_);
        std::unique_lock<std::mutex> g(mu_);
        done_.wait(g, [this]() { return pending_ == 0; });
    }
  private:
    void run(int t) {
        uint64_t seen = 0;
        for (;;) {
            const std::function<void(int64_t, int64_t)>* fn;
            int64_t total;
            {
                std::unique_lock<std::mutex> g(mu_);
                cv_.wait(g, [&]() { return gen_ != seen; });
                seen = gen_;
                if (stop_) return;
                fn = fn_; total = total_;
            }
            (*fn)(total * t / n_, total * (t + 1) / n_);
            {
                std::lock_guard<std::mutex> g(mu_);
                if (--pending_ == 0) done_.notify_one();
            }
        }
    }
    int n_;
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable cv_, done_;
    const std::function<void(int64_t, int64_t)>* fn_ = nullptr;
    int64_t total_ = 0;
    int pending_ = 0;
    uint64_t gen_ = 0;
    bool stop_ = false;
};

// nthreads <= 1 (or no pool) runs inline.
void parallel_for(Pool* pool, int64_t n, const std::function<void(int64_t, int64_t)>& fn) {
    if (!pool) { fn(0, n); return; }
    pool->parallel(n, fn);
}

// A 2-D row-major matrix with the reference's padding rule: row stride is cols rounded
// up to 8 (f32) or 16 (f16), padding zeroed (src/tensor.rs:192-222, :433-450).
struct Mat {
    int64_t rows = 0, cols = 0, cap = 0;
    bool is_f16 = false;
    void* data = nullptr;

    Mat() {}
    Mat(int64_t r, int64_t c, bool f16) { alloc(r, c, f16); }
    Mat(const Mat&) = delete;
    Mat& operator=(const Mat&) = delete;
    Mat(Mat&& o) noexcept { *this = std::move(o); }
    Mat& operator=(Mat&& o) noexcept {
        if (this != &o) {
            release();
            rows = o.rows; cols = o.cols; cap = o.cap; is_f16 = o.is_f16; data = o.data;
            o.data = nullptr; o.rows = o.cols = o.cap = 0;
        }
        return *this;
    }
    ~Mat() { release(); }
    void release() { if (data) free(data); data = nullptr; }
    // zero = false: the caller overwrites every element (only allowed when rows carry no padding)
    void alloc(int64_t r, int64_t c, bool f16, bool zero = true) {
        release();
        rows = r; cols = c; is_f16 = f16;
        cap = round_up(c, f16 ? 16 : 8);
        size_t bytes = (size_t)std::max<int64_t>(r, 1) * cap * (f16 ? 2 : 4);
        bytes = (size_t)round_up((int64_t)bytes, 32);
        data = aligned_alloc(32, bytes);
        if (zero || cap != c || r < 1) memset(data, 0, bytes);
    }
    float* f32() { return (float*)data; }
    const float* f32() const { return (const float*)data; }
    f16bits* h() { return (f16bits*)data; }
    const f16bits* h() const { return (const f16bits*)data; }
    float get(int64_t r, int64_t c) const {
        return is_f16 ? h2f(h()[r * cap + c]) : f32()[r * cap + c];
    }
    void set(int64_t r, int64_t c, float v) {
        if (is_f16) h()[r * cap + c] = f2h(v); else f32()[r * cap + c] = v;
    }
};

// Tensor::to_f16 / to_f32 (src/tensor.rs:2226-2314): RNE narrowing, exact widening.
Mat cast(const Mat& m, bool to_f16) {
    Mat out(m.rows, m.cols, to_f16);
    for (int64_t r = 0; r < m.rows; r++) {
        int64_t c = 0;
        if (m.is_f16 && !to_f16) {
            for (; c + 8 <= m.cols; c += 8)
                _mm256_storeu_ps(out.f32() + r * out.cap + c,
                                 _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(m.h() + r * m.cap + c))));
        } else if (!m.is_f16 && to_f16) {
            for (; c + 8 <= m.cols; c += 8)
                _mm_storeu_si128((__m128i*)(out.h() + r * out.cap + c),
                                 _mm256_cvtps_ph(_mm256_loadu_ps(m.f32() + r * m.cap + c), 0));
        } else {
            memcpy((char*)out.data + (size_t)r * out.cap * (to_f16 ? 2 : 4),
                   (const char*)m.data + (size_t)r * m.cap * (to_f16 ? 2 : 4), (size_t)m.cols * (to_f16 ? 2 : 4));
            c = m.cols;
        }
        for (; c < m.cols; c++) out.set(r, c, m.get(r, c));
    }
    return out;
}

// ---------------------------------------------------------------------------------
// contractions
// ---------------------------------------------------------------------------------

// One output of any "transposed" contraction over f32 operands: 8 lane partials, FMA,
// horizontal fold. kcap is the padded length (multiple of 8, padding is zero).
inline float dot8_f32(const float* a, const float* b, int64_t kcap) {
    __m256 acc = _mm256_setzero_ps();
    for (int64_t k = 0; k < kcap; k += 8)
        acc = _mm256_fmadd_ps(_mm256_loadu_ps(a + k), _mm256_loadu_ps(b + k), acc);
    return hsum8(acc);
}

inline float dot8_f16(const f16bits* a, const f16bits* b, int64_t kcap) {
    __m256 acc = _mm256_setzero_ps();
    for (int64_t k = 0; k < kcap; k += 8) {
        __m256 av = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(a + k)));
        __m256 bv = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(b + k)));
        acc = _mm256_fmadd_ps(av, bv, acc);
    }
    return hsum8(acc);
}

// Tensor::matrix_mul_transposed (src/tensor.rs:999-1025): C[i][j] = sum_k A[i][k]*B[j][k].
// f32: general path :1282-1475 or the GEMV shortcut :1837-1918 (same arithmetic per
// output). f16: :1476-1666, result rounded to f16. Work is dealt over threads by output
// rows; each output is produced by exactly one thread, as in the reference (:1337-1340),
// so the thread count never changes a value.
Mat matmul_t(const Mat& A, const Mat& B, Pool* pool) {
    Mat C(A.rows, B.rows, A.is_f16);
    const int64_t kcap = round_up(A.cols, 8);
    // 4 x 4 register blocking over (i, j); each accumulator is an independent dot8.
    const int64_t ib = (A.rows + 3) / 4, jb = (B.rows + 3) / 4;
    parallel_for(pool, ib * jb, [&](int64_t lo, int64_t hi) {
        for (int64_t blk = lo; blk < hi; blk++) {
            const int64_t i0 = (blk / jb) * 4, j0 = (blk % jb) * 4;
            const int ni = (int)std::min<int64_t>(4, A.rows - i0);
            const int nj = (int)std::min<int64_t>(4, B.rows - j0);
            __m256 acc[4][4];
            for (int a = 0; a < 4; a++)
                for (int b = 0; b < 4; b++) acc[a][b] = _mm256_setzero_ps();
            if (!A.is_f16) {
                for (int64_t k = 0; k < kcap; k += 8) {
                    __m256 av[4], bv[4];
                    for (int a = 0; a < ni; a++) av[a] = _mm256_loadu_ps(A.f32() + (i0 + a) * A.cap + k);
                    for (int b = 0; b < nj; b++) bv[b] = _mm256_loadu_ps(B.f32() + (j0 + b) * B.cap + k);
                    for (int a = 0; a < ni; a++)
                        for (int b = 0; b < nj; b++) acc[a][b] = _mm256_fmadd_ps(av[a], bv[b], acc[a][b]);
                }
                for (int a = 0; a < ni; a++)
                    for (int b = 0; b < nj; b++) C.f32()[(i0 + a) * C.cap + j0 + b] = hsum8(acc[a][b]);
            } else {
                for (int64_t k = 0; k < kcap; k += 8) {
                    __m256 av[4], bv[4];
                    for (int a = 0; a < ni; a++)
                        av[a] = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(A.h() + (i0 + a) * A.cap + k)));
                    for (int b = 0; b < nj; b++)
                        bv[b] = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(B.h() + (j0 + b) * B.cap + k)));
                    for (int a = 0; a < ni; a++)
                        for (int b = 0; b < nj; b++) acc[a][b] = _mm256_fmadd_ps(av[a], bv[b], acc[a][b]);
                }
                for (int a = 0; a < ni; a++)
                    for (int b = 0; b < nj; b++) C.h()[(i0 + a) * C.cap + j0 + b] = f2h(hsum8(acc[a][b]));
            }
        }
    });
    return C;
}

// Naive triple loop (Tensor::matrix_mul_naive): plain f32 multiply-add in k order. Used
// by the op-level tests exactly as the reference's tests use it (src/tensor.rs:2701-2857).
Mat matmul_naive(const Mat& A, const Mat& B) {
    Mat C(A.rows, B.cols, A.is_f16);
    for (int64_t i = 0; i < A.rows; i++)
        for (int64_t j = 0; j < B.cols; j++) {
            float s = 0.0f;
            for (int64_t k = 0; k < A.cols; k++) s += A.get(i, k) * B.get(k, j);
            C.set(i, j, s);
        }
    return C;
}

// Tensor::matrix_mul (src/tensor.rs:979-997) on f32 operands:
//  rows == 1  -> vector_matrix_mul (:1923-1983): per column, 8 lanes over k, fold;
//  otherwise  -> matrix_mul_inplace (:1050-1115): sequential-k FMA per output.
// (The matrix_vector_mul branch for other.cols == 1 is not reachable from the forward
// pass at head_dim > 1 and is folded into the general branch: same sequential order is
// NOT claimed for it.)
Mat matmul_plain_f32(const Mat& A, const Mat& B) {
    Mat C(A.rows, B.cols, false);
    if (A.rows == 1) {
        const int64_t kcap = round_up(B.rows, 8);
        std::vector<float> colbuf((size_t)kcap, 0.0f), left((size_t)kcap, 0.0f);
        for (int64_t k = 0; k < A.cols; k++) left[k] = A.f32()[k];
        for (int64_t col = 0; col < B.cols; col++) {
            for (int64_t k = 0; k < B.rows; k++) colbuf[k] = B.f32()[k * B.cap + col];
            C.f32()[col] = dot8_f32(left.data(), colbuf.data(), kcap);
        }
        return C;
    }
    for (int64_t i = 0; i < A.rows; i++)
        for (int64_t j = 0; j < B.cols; j++) {
            float acc = 0.0f;
            for (int64_t k = 0; k < A.cols; k++)
                acc = std::fmaf(A.f32()[i * A.cap + k], B.f32()[k * B.cap + j], acc);
            C.f32()[i * C.cap + j] = acc;
        }
    return C;
}

// ---------------------------------------------------------------------------------
// element-wise pieces
// ---------------------------------------------------------------------------------

// RMSNorm::forward (src/transformer.rs:476-480) over f32 rows.
Mat rmsnorm(const Mat& x, const Mat& gain, double eps) {
    Mat out(x.rows, x.cols, false);
    const float epsf = (float)eps;
    for (int64_t r = 0; r < x.rows; r++) {
        float sum = 0.0f;
        for (int64_t c = 0; c < x.cols; c++) sum += powf(x.f32()[r * x.cap + c], 2.0f);
        float inner = sum / (float)x.cols + epsf;
        float scale = 1.0f / sqrtf(inner);
        for (int64_t c = 0; c < x.cols; c++)
            out.f32()[r * out.cap + c] = (x.f32()[r * x.cap + c] * scale) * gain.f32()[c];
    }
    return out;
}

// Tensor::softmax (src/tensor.rs:479-494), in place over f32 rows.
void softmax_rows(Mat& m) {
    for (int64_t r = 0; r < m.rows; r++) {
        float* p = m.f32() + r * m.cap;
        float sum = 0.0f;
        for (int64_t c = 0; c < m.cols; c++) sum += expf(p[c]);
        for (int64_t c = 0; c < m.cols; c++) p[c] = expf(p[c]) / sum;
    }
}

inline float silu(float v) { return v / (1.0f + expf(-v)); }  // src/tensor.rs:822-832

// ---------------------------------------------------------------------------------
// model
// ---------------------------------------------------------------------------------

enum TensorKind { K_TOK_EMB = 0, K_WQ, K_WK, K_WV, K_WO, K_W1, K_W2, K_W3, K_ATTN_NORM, K_FFN_NORM, K_NORM, K_OUTPUT };

struct Layer {
    Mat wq, wk, wv, wo, w1, w2, w3, attn_norm, ffn_norm;
};

struct Model {
    int dim, n_layers, n_heads, head_dim, ffn, vocab, max_seq_len;
    double eps;
    bool force_f16;
    int nthreads;
    std::unique_ptr<Pool> pool;
    Mat tok_emb, norm, output;
    std::vector<Layer> layers;
    std::vector<float> freqs;  // [max_seq_len][head_dim/2][2] (re, im), f64 -> f32 at use
};

// AttentionCache (src/transformer.rs:122-160): per layer, per head, K and V are
// head_dim x max_seq_len, position contiguous.
struct Caches {
    int n_layers, n_heads;
    std::vector<Mat> k, v;  // [layer * n_heads + head]
};

// compute_freqs_cis (src/transformer.rs:858-885): f64 table, cast to f32 when applied.
void build_freqs(Model& m) {
    const int hd = m.head_dim;
    m.freqs.resize((size_t)m.max_seq_len * (hd / 2) * 2);
    for (int pos = 0; pos < m.max_seq_len; pos++)
        for (int i = 0; i < hd / 2; i++) {
            double freq = 1.0 / pow(10000.0, (double)i * 2.0 / (double)hd);
            double ang = freq * (double)pos;
            m.freqs[((size_t)pos * (hd / 2) + i) * 2 + 0] = (float)cos(ang);
            m.freqs[((size_t)pos * (hd / 2) + i) * 2 + 1] = (float)sin(ang);
        }
}

// Attention::forward (src/transformer.rs:657-820), non-OpenCL branches. x is n x dim f32.
Mat attention_forward(const Model& m, const Layer& L, const Mat& x, int start_pos, Caches& caches, int layer, bool& ok) {
    const int n = (int)x.rows, H = m.n_heads, hd = m.head_dim, T = start_pos + n;
    const bool f16 = L.wq.is_f16;
    Mat xin = cast(x, f16);                                   // :666-668
    Mat q = cast(matmul_t(xin, L.wq, m.pool.get()), false);      // :694-702
    Mat k = cast(matmul_t(xin, L.wk, m.pool.get()), false);
    Mat v = cast(matmul_t(xin, L.wv, m.pool.get()), false);

    // apply_rotary_emb (:823-856) on q and k, f32, interleaved pairs.
    for (int i = 0; i < n; i++)
        for (int h = 0; h < H; h++)
            for (int c = 0; c < hd / 2; c++) {
                const float fr = m.freqs[((size_t)(start_pos + i) * (hd / 2) + c) * 2 + 0];
                const float fi = m.freqs[((size_t)(start_pos + i) * (hd / 2) + c) * 2 + 1];
                float* qp = q.f32() + i * q.cap + h * hd + 2 * c;
                float* kp = k.f32() + i * k.cap + h * hd + 2 * c;
                const float qr = qp[0], qi = qp[1], kr = kp[0], ki = kp[1];
                qp[0] = qr * fr - qi * fi;
                qp[1] = qr * fi + qi * fr;
                kp[0] = kr * fr - ki * fi;
                kp[1] = kr * fi + ki * fr;
            }

    if (n > 1 && start_pos != 0) {
        // The reference adds an n x n mask to n x T scores and panics on the shape
        // mismatch (src/tensor.rs:576-584): multi-token calls are defined for start_pos 0 only.
        ok = false;
        return Mat();
    }

    Mat heads_out(n, (int64_t)H * hd, false);
    const float scale = 1.0f / sqrtf((float)hd);               // :770
    parallel_for(m.pool.get(), H, [&](int64_t lo, int64_t hi) {  // :727
        for (int64_t h = lo; h < hi; h++) {
            Mat& ck = caches.k[(size_t)layer * H + h];
            Mat& cv = caches.v[(size_t)layer * H + h];
            for (int pos = start_pos; pos < T; pos++)          // :754-761 (set_f32 rounds when f16)
                for (int d = 0; d < hd; d++) {
                    ck.set(d, pos, k.f32()[(pos - start_pos) * k.cap + h * hd + d]);
                    cv.set(d, pos, v.f32()[(pos - start_pos) * v.cap + h * hd + d]);
                }
            Mat keys(hd, T, false), values(hd, T, false);      // clip_cols + into_same_type (:762-766)
            for (int d = 0; d < hd; d++)
                for (int t = 0; t < T; t++) {
                    keys.f32()[d * keys.cap + t] = ck.get(d, t);
                    values.f32()[d * values.cap + t] = cv.get(d, t);
                }
            Mat qh(n, hd, false);
            for (int i = 0; i < n; i++)
                memcpy(qh.f32() + i * qh.cap, q.f32() + i * q.cap + h * hd, sizeof(float) * hd);
            Mat s = matmul_plain_f32(qh, keys);                // :768-769
            for (int i = 0; i < n; i++)
                for (int t = 0; t < T; t++) {
                    float val = s.f32()[i * s.cap + t] * scale;
                    // full_triu(n, n, start_pos + 1, -inf) added (:350-357, src/tensor.rs:496-508)
                    if (n > 1 && t >= i + start_pos + 1) val += -INFINITY;
                    s.f32()[i * s.cap + t] = val;
                }
            softmax_rows(s);
            Mat o = matmul_t(s, values, nullptr);                    // :777-778, general f32 path
            for (int i = 0; i < n; i++)
                memcpy(heads_out.f32() + i * heads_out.cap + h * hd, o.f32() + i * o.cap, sizeof(float) * hd);
        }
    });

    // :783-819: each row -> weight dtype -> wo -> back to f32.
    Mat ho = cast(heads_out, f16);
    return cast(matmul_t(ho, L.wo, m.pool.get()), false);
}

// FeedForward::forward (src/transformer.rs:536-582) + the caller's transpose (:444).
Mat ffn_forward(const Model& m, const Layer& L, const Mat& x) {
    const bool f16 = L.w1.is_f16;
    const int64_t n = x.rows, F = L.w1.rows;
    Mat xin = cast(x, f16);
    Mat a = cast(matmul_t(L.w1, xin, m.pool.get()), false);  // F x n
    Mat b = cast(matmul_t(L.w3, xin, m.pool.get()), false);
    Mat g(n, F, false);                                    // silu, hadamard, transpose
    for (int64_t j = 0; j < F; j++)
        for (int64_t i = 0; i < n; i++)
            g.f32()[i * g.cap + j] = silu(a.f32()[j * a.cap + i]) * b.f32()[j * b.cap + i];
    Mat gin = cast(g, L.w2.is_f16);
    Mat out_t = cast(matmul_t(L.w2, gin, m.pool.get()), false);  // dim x n
    Mat out(n, L.w2.rows, false);
    for (int64_t i = 0; i < n; i++)
        for (int64_t j = 0; j < L.w2.rows; j++) out.f32()[i * out.cap + j] = out_t.f32()[j * out_t.cap + i];
    return out;
}

Mat add(const Mat& a, const Mat& b) {
    Mat out(a.rows, a.cols, false);
    for (int64_t r = 0; r < a.rows; r++)
        for (int64_t c = 0; c < a.cols; c++) out.f32()[r * out.cap + c] = a.f32()[r * a.cap + c] + b.f32()[r * b.cap + c];
    return out;
}

}  // namespace

// ---------------------------------------------------------------------------------
// C interface (ctypes-friendly). dtype: 0 = f32, 1 = f16 (uint16 bit patterns).
// ---------------------------------------------------------------------------------
extern "C" {

void* orc_model_create(int dim, int n_layers, int n_heads, int ffn, int vocab, double eps,
                       int max_seq_len, int force_f16, int nthreads) {
    Model* m = new Model();
    m->dim = dim; m->n_layers = n_layers; m->n_heads = n_heads; m->head_dim = dim / n_heads;
    m->ffn = ffn; m->vocab = vocab; m->max_seq_len = max_seq_len; m->eps = eps;
    m->force_f16 = force_f16 != 0;
    m->nthreads = nthreads > 0 ? nthreads : (int)std::max(1u, std::thread::hardware_concurrency());
    if (m->nthreads > 1) m->pool.reset(new Pool(m->nthreads));
    m->layers.resize(n_layers);
    build_freqs(*m);
    return m;
}

void orc_model_free(void* mp) { delete (Model*)mp; }

// The loader always widens to f32 (src/tensor.rs:2467, :2538); the seven per-layer
// matrices then become f16 under force_f16 (src/transformer.rs:508-512, :624-629);
// embeddings, gains and the output head stay f32 (:302-308, :468).
int orc_model_set_tensor(void* mp, int kind, int layer, const void* data, int rows, int cols, int dtype) {
    Model* m = (Model*)mp;
    Mat src;
    src.alloc(rows, cols, dtype == 1, false);
    const size_t esz = dtype == 1 ? 2 : 4;
    for (int r = 0; r < rows; r++)
        memcpy((char*)src.data + (size_t)r * src.cap * esz, (const char*)data + (size_t)r * cols * esz, (size_t)cols * esz);
    // The reference widens every loaded tensor to f32 and, under --f16, narrows the seven per-layer matrices
    // again (src/tensor.rs:2388-2545, src/transformer.rs:514-525). f16 -> f32 -> f16 is the identity, so a
    // tensor that arrives in the type it is stored in is kept as it is.
    bool per_layer_matrix = kind >= K_WQ && kind <= K_W3;
    const bool want_f16 = per_layer_matrix && m->force_f16;
    Mat stored = (src.is_f16 == want_f16) ? std::move(src) : cast(src, want_f16);
    if (kind != K_TOK_EMB && kind != K_NORM && kind != K_OUTPUT && (layer < 0 || layer >= m->n_layers)) return -1;
    switch (kind) {
        case K_TOK_EMB: m->tok_emb = std::move(stored); break;
        case K_NORM: m->norm = std::move(stored); break;
        case K_OUTPUT: m->output = std::move(stored); break;
        case K_WQ: m->layers[layer].wq = std::move(stored); break;
        case K_WK: m->layers[layer].wk = std::move(stored); break;
        case K_WV: m->layers[layer].wv = std::move(stored); break;
        case K_WO: m->layers[layer].wo = std::move(stored); break;
        case K_W1: m->layers[layer].w1 = std::move(stored); break;
        case K_W2: m->layers[layer].w2 = std::move(stored); break;
        case K_W3: m->layers[layer].w3 = std::move(stored); break;
        case K_ATTN_NORM: m->layers[layer].attn_norm = std::move(stored); break;
        case K_FFN_NORM: m->layers[layer].ffn_norm = std::move(stored); break;
        default: return -1;
    }
    return 0;
}

void* orc_caches_create(void* mp) {  // Transformer::make_caches (src/transformer.rs:328-341)
    Model* m = (Model*)mp;
    Caches* c = new Caches();
    c->n_layers = m->n_layers; c->n_heads = m->n_heads;
    c->k.resize((size_t)m->n_layers * m->n_heads);
    c->v.resize((size_t)m->n_layers * m->n_heads);
    for (auto& t : c->k) t.alloc(m->head_dim, m->max_seq_len, m->force_f16);
    for (auto& t : c->v) t.alloc(m->head_dim, m->max_seq_len, m->force_f16);
    return c;
}

void orc_caches_free(void* cp) { delete (Caches*)cp; }

// TransformerCaches::shift_left (src/transformer.rs:180-205).
void orc_caches_shift_left(void* cp, int shifts) {
    Caches* c = (Caches*)cp;
    for (int s = 0; s < shifts; s++)
        for (size_t i = 0; i < c->k.size(); i++)
            for (int64_t d = 0; d < c->k[i].rows; d++)
                for (int64_t t = 0; t + 1 < c->k[i].cols; t++) {
                    c->k[i].set(d, t, c->k[i].get(d, t + 1));
                    c->v[i].set(d, t, c->v[i].get(d, t + 1));
                }
}

// Reads one cached value (for cache-content tests): which = 0 K, 1 V.
float orc_caches_get(void* cp, int which, int layer, int head, int d, int pos) {
    Caches* c = (Caches*)cp;
    const Mat& t = (which == 0 ? c->k : c->v)[(size_t)layer * c->n_heads + head];
    return t.get(d, pos);
}

// Transformer::forward (src/transformer.rs:343-382). Returns 0, or -1 where the
// reference would panic (multi-token call at start_pos > 0, out-of-range token/position).
int orc_forward(void* mp, void* cp, const int32_t* tokens, int n, int start_pos, float* logits_out) {
    Model* m = (Model*)mp;
    Caches* c = (Caches*)cp;
    if (n < 1 || start_pos < 0 || start_pos + n > m->max_seq_len) return -1;
    Mat x(n, m->dim, false);
    for (int i = 0; i < n; i++) {
        if (tokens[i] < 0 || tokens[i] >= m->tok_emb.rows) return -1;
        memcpy(x.f32() + i * x.cap, m->tok_emb.f32() + (int64_t)tokens[i] * m->tok_emb.cap, sizeof(float) * m->dim);
    }
    for (int l = 0; l < m->n_layers; l++) {  // TransformerBlock::forward (:424-446)
        const Layer& L = m->layers[l];
        Mat an = rmsnorm(x, L.attn_norm, m->eps);
        bool ok = true;
        Mat att = attention_forward(*m, L, an, start_pos, *c, l, ok);
        if (!ok) return -1;
        Mat h = add(x, att);
        Mat fn = rmsnorm(h, L.ffn_norm, m->eps);
        Mat ff = ffn_forward(*m, L, fn);
        x = add(h, ff);
    }
    Mat out = rmsnorm(x, m->norm, m->eps);  // :378
    Mat last(1, m->dim, false);             // :379
    memcpy(last.f32(), out.f32() + (int64_t)(n - 1) * out.cap, sizeof(float) * m->dim);
    Mat logits = matmul_t(m->output, last, m->pool.get());  // :381, f32 head
    for (int v = 0; v < m->vocab; v++) logits_out[v] = logits.f32()[(int64_t)v * logits.cap];
    return 0;
}

// --- op-level entry points (dense inputs without padding) -------------------------

static Mat from_dense(const void* p, int rows, int cols, int dtype) {
    Mat m(rows, cols, dtype == 1);
    const size_t esz = dtype == 1 ? 2 : 4;
    for (int r = 0; r < rows; r++)
        memcpy((char*)m.data + (size_t)r * m.cap * esz, (const char*)p + (size_t)r * cols * esz, (size_t)cols * esz);
    return m;
}
static void to_dense(const Mat& m, void* p) {
    const size_t esz = m.is_f16 ? 2 : 4;
    for (int64_t r = 0; r < m.rows; r++)
        memcpy((char*)p + (size_t)r * m.cols * esz, (const char*)m.data + (size_t)r * m.cap * esz, (size_t)m.cols * esz);
}

// out[a_rows x b_rows] = A * B^T, dtype of A and B.
void orc_matrix_mul_transposed(const void* a, int a_rows, const void* b, int b_rows, int k, int dtype, int nthreads, void* out) {
    Mat A = from_dense(a, a_rows, k, dtype), B = from_dense(b, b_rows, k, dtype);
    std::unique_ptr<Pool> pool(nthreads > 1 ? new Pool(nthreads) : nullptr);
    to_dense(matmul_t(A, B, pool.get()), out);
}
// out[a_rows x b_cols] = A * B (f32 only), the reference's matrix_mul dispatch.
void orc_matrix_mul_f32(const float* a, int a_rows, int a_cols, const float* b, int b_cols, float* out) {
    Mat A = from_dense(a, a_rows, a_cols, 0), B = from_dense(b, a_cols, b_cols, 0);
    to_dense(matmul_plain_f32(A, B), out);
}
void orc_matrix_mul_naive(const void* a, int a_rows, int a_cols, const void* b, int b_cols, int dtype, void* out) {
    Mat A = from_dense(a, a_rows, a_cols, dtype), B = from_dense(b, a_cols, b_cols, dtype);
    to_dense(matmul_naive(A, B), out);
}
void orc_rmsnorm(const float* x, int rows, int cols, const float* gain, double eps, float* out) {
    Mat X = from_dense(x, rows, cols, 0), G = from_dense(gain, 1, cols, 0);
    to_dense(rmsnorm(X, G, eps), out);
}
void orc_softmax(float* x, int rows, int cols) {
    Mat X = from_dense(x, rows, cols, 0);
    softmax_rows(X);
    to_dense(X, x);
}
void orc_silu(float* x, int64_t n) { for (int64_t i = 0; i < n; i++) x[i] = silu(x[i]); }
void orc_f32_to_f16(const float* in, uint16_t* out, int64_t n) { for (int64_t i = 0; i < n; i++) out[i] = f2h(in[i]); }
void orc_f16_to_f32(const uint16_t* in, float* out, int64_t n) { for (int64_t i = 0; i < n; i++) out[i] = h2f(in[i]); }
void orc_freqs_cis(int head_dim, int max_seq_len, float* out) {
    Model m; m.head_dim = head_dim; m.max_seq_len = max_seq_len;
    build_freqs(m);
    memcpy(out, m.freqs.data(), m.freqs.size() * sizeof(float));
}
int orc_hw_threads() { return (int)std::max(1u, std::thread::hardware_concurrency()); }

}  // extern "C"

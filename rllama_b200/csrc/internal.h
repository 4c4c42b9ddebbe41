// Internal declarations shared by the translation units of librllama_b200.so.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/rllama_b200.h"

// ---------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------
int rlb_fail(int code, const char* fmt, ...);  // records the thread's message, returns code

#define RLB_CUDA(expr)                                                                         \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return rlb_fail(_e == cudaErrorMemoryAllocation ? RLB_ERR_OOM : RLB_ERR_CUDA,      \
                            "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__,  \
                            __LINE__);                                                         \
    } while (0)

#define RLB_TRY(expr)            \
    do {                         \
        int _s = (expr);         \
        if (_s != RLB_OK) return _s; \
    } while (0)

// ---------------------------------------------------------------------------------------
// handles
// ---------------------------------------------------------------------------------------
struct rlb_ctx {
    int device = 0;
    int sm_count = 0;
    bool verbose = false;
    cudaStream_t stream = nullptr;
    std::recursive_mutex mu;
    uint64_t launches = 0;  // kernels launched by this library on this context
    void* op_scratch = nullptr;  // scratch of the standalone attention op, grown on demand
    size_t op_scratch_bytes = 0;
    void* gemm_scratch = nullptr;  // split-K partial tiles of the tensor-core GEMM, grown on demand
    size_t gemm_scratch_bytes = 0;
    // error word of the op-level kernels: mapped pinned host memory, so the host reads it after a
    // synchronisation without a copy (raised when a bounded device-side wait ran out)
    int* h_err = nullptr;
    int* d_err = nullptr;
    // set while the model's prefill enqueues its kernels: they are then launched as programmatic dependents
    // (each may start while its predecessor drains; every one of them waits for the predecessor before it
    // touches anything but weights)
    bool pdl_chain = false;
};
int ctx_check_error_word(rlb_ctx* ctx);  // after a synchronisation: RLB_ERR_CUDA if a kernel raised the word

struct rlb_tensor {
    rlb_ctx* ctx = nullptr;
    void* d = nullptr;
    int64_t rows = 0, cols = 0, cap = 0;
    rlb_dtype dtype = RLB_F32;
    cudaEvent_t ready = nullptr;  // last operation queued on this tensor
    size_t bytes() const { return (size_t)rows * cap * (dtype == RLB_F16 ? 2 : 4); }
};

struct rlb_event {
    rlb_ctx* ctx = nullptr;
    cudaEvent_t ev = nullptr;
};

static inline size_t dtype_size(rlb_dtype t) { return t == RLB_F16 ? 2 : 4; }

// ---------------------------------------------------------------------------------------
// decode GEMV family (gemv.cu)
// ---------------------------------------------------------------------------------------
enum GemvPrologue {
    PRO_COPY = 0,  // activation already in the weight dtype: act[k] = vec_in[k]
    PRO_NORM = 1,  // act = cast(rmsnorm(x_in + round(sum of partials)) * gain); block 0 stores the new residual
};
enum GemvEpilogue {
    EPI_STORE = 0,    // out[row * out_stride] = (weight dtype) acc          (tier-1 op, logits use EPI_F32)
    EPI_F32 = 1,      // out[row] = acc as f32, unrounded (partials, logits)
    EPI_QKV = 2,      // round, RoPE on q and k, write q buffer and KV cache
    EPI_SWIGLU = 3,   // two matrices: gate[row] = round(silu(round(a1)) * round(a3))
};

#define RLB_MAX_TP 8

struct GemvArgs {
    // weights
    const void* W = nullptr;   // [rows x K], row stride ldw elements
    const void* W2 = nullptr;  // second matrix (w3) for EPI_SWIGLU
    int rows = 0, K = 0;
    int64_t ldw = 0;
    // prologue
    const void* vec_in = nullptr;    // PRO_COPY source (weight dtype)
    const float* x_in = nullptr;     // PRO_NORM: residual stream (or embedding table when tok_ptr set)
    const int32_t* tok_ptr = nullptr;  // PRO_NORM: if set, x row = x_in + tok * K
    const float* parts = nullptr;    // PRO_NORM: n_parts partial sums of K floats, stride part_stride
    int n_parts = 0;
    int64_t part_stride = 0;
    int round_parts = 0;             // round the summed partials to f16 before the residual add
    float* x_out = nullptr;          // PRO_NORM: block 0 writes the updated residual here
    const float* gain = nullptr;
    float eps = 0.f;
    // epilogue
    void* out = nullptr;
    int64_t out_stride = 1;
    // Tensor-parallel push exchange. Values travel as 8-byte {f32 value, u32 sequence number}
    // entries written with one store, so a reader that sees the expected sequence number also
    // sees the value: no fence and no separate flag. The sequence number of an exchange is
    // (*epoch_ptr - 1) * seq_stride + seq_idx, unique per (decode step, layer, projection).
    uint2* ll_outs[RLB_MAX_TP] = {nullptr};  // EPI_F32 producer: every rank's inbox (peer memory); entry = out_offset + row
    int n_outs = 0;                  // 0: write `out` only
    int64_t out_offset = 0;
    const uint2* ll_inbox = nullptr; // PRO_NORM consumer: this rank's inbox, n_parts x K entries
    unsigned int* xready = nullptr;  // PRO_NORM consumer: counts the CTAs that have published their slice of x_out
    int gather_all = 0;              // PRO_NORM consumer: every CTA collects the whole row from the inbox itself (short rows, few ranks)
    uint32_t seq_idx = 0, seq_stride = 0, out_seq_idx = 0;
    const int32_t* epoch_ptr = nullptr;
    // EPI_QKV
    float* qbuf = nullptr;
    void* kcache = nullptr;          // this layer's K cache [heads][max_seq][hd]
    void* vcache = nullptr;
    const float* rope = nullptr;     // [max_seq][hd/2][2]
    const int32_t* pos_ptr = nullptr;
    int nq = 0, hd = 0, max_seq = 0;
};

// dtype: weight (= activation) dtype. Chooses rows-per-warp and grid from the shape.
int launch_gemv(rlb_ctx* ctx, rlb_dtype dtype, int prologue, int epilogue, const GemvArgs& args);
// Bulk-copy staged variant (gemv_stream.cu). Returns RLB_ERR_STATE, without an error message,
// for shapes it does not handle. err_flag: device int raised when a bounded wait ran out.
int launch_gemv_stream(rlb_ctx* ctx, rlb_dtype dtype, int prologue, int epilogue, const GemvArgs& args, int* err_flag, int allow_pdl);
// Grid size launch_gemv_stream would use for these arguments (0 if it does not take the shape).
int gemv_stream_grid(rlb_ctx* ctx, rlb_dtype dtype, int prologue, int epilogue, const GemvArgs& args);
// Tuning knobs (read once from the environment by gemv.cu): rows per warp, CTAs per SM.
void gemv_set_tuning(int rows_per_warp, int ctas_per_sm, int threads);

// ---------------------------------------------------------------------------------------
// attention (attention.cu)
// ---------------------------------------------------------------------------------------
struct AttnDecodeArgs {
    const float* q = nullptr;      // [heads][hd] f32, rotated
    const void* kcache = nullptr;  // [heads][max_seq][hd]
    const void* vcache = nullptr;
    void* out = nullptr;           // [heads*hd] in the weight dtype (rounded when f16)
    const int32_t* pos_ptr = nullptr;  // attends to positions 0..*pos_ptr ...
    int pos_value = 0;                 // ... or, when pos_ptr is null, to 0..pos_value
    int heads = 0, hd = 0, max_seq = 0;
    int n_split = 1;
    float* scratch = nullptr;      // [heads][n_split][hd + 2] partial (o, m, l)
    unsigned int* counters = nullptr;  // [heads], zero between launches
};
int launch_attn_decode(rlb_ctx* ctx, rlb_dtype cache_dtype, const AttnDecodeArgs& a, int allow_pdl);
// Argument checks shared by the standalone attention entry points (context.cu).
int attention_check(const rlb_tensor* out, const rlb_tensor* q, const rlb_tensor* kcache, const rlb_tensor* vcache, int32_t heads,
                    int32_t max_seq_len, int32_t pos, int32_t n_split, int* hd_out);
size_t attn_decode_scratch_floats(int heads, int hd, int n_split);

struct AttnPrefillArgs {
    const float* q = nullptr;      // n rows of heads*hd f32 (rotated), row stride q_ld
    int64_t q_ld = 0;
    const void* kcache = nullptr;
    const void* vcache = nullptr;
    void* out = nullptr;           // [n][heads*hd] weight dtype
    int n = 0, start_pos = 0, heads = 0, hd = 0, max_seq = 0;
    int* err = nullptr;            // device-visible error word for bounded waits (nullptr: the context's word)
    bool allow_tc = true;          // the tensor-core kernel may take the call
};
int launch_attn_prefill(rlb_ctx* ctx, rlb_dtype cache_dtype, const AttnPrefillArgs& a);
// Tensor-core form (attention_tc.cu): f16 caches, head_dim 64 / 128, at least 32 query rows.
bool attn_prefill_tc_supported(rlb_dtype cache_dtype, const AttnPrefillArgs& a);
int launch_attn_prefill_tc(rlb_ctx* ctx, const AttnPrefillArgs& a, int* err);

// ---------------------------------------------------------------------------------------
// row-wise / element-wise kernels used by prefill and the tier-1 ops (elementwise.cu)
// ---------------------------------------------------------------------------------------
int launch_embed(rlb_ctx* ctx, const float* table, const int32_t* tokens_dev, int n, int dim, float* x);
// a[n][dim] (weight dtype) = cast(rmsnorm(x) * gain)
int launch_rmsnorm_rows(rlb_ctx* ctx, const float* x, int n, int dim, const float* gain, float eps, rlb_dtype out_dtype,
                        void* out);
// x[n][dim] += round_f16?(y) (y may be null: no add), then a = cast(rmsnorm(x) * gain)
int launch_add_norm_rows(rlb_ctx* ctx, float* x, const float* y, int round_y, int n, int dim, const float* gain, float eps,
                         rlb_dtype out_dtype, void* out);
// q,k,v: n rows of nq f32 GEMM outputs (already rounded when f16), row stride ld. Rotates q in place, writes K (rotated)
// and V to the cache.
int launch_rope_append(rlb_ctx* ctx, float* q, const float* k, const float* v, int64_t ld, int n, int start_pos, int heads,
                       int hd, int max_seq, const float* rope, rlb_dtype cache_dtype, void* kcache, void* vcache);
// g[rows][cols] (weight dtype, dense) = cast(silu(a1) * a3); a1, a3 have row stride ld
int launch_swiglu_rows(rlb_ctx* ctx, const float* a1, const float* a3, int64_t ld, int64_t rows, int64_t cols, rlb_dtype out_dtype,
                       void* out);
// x[i] += round_f16?(y[i])
int launch_add_rows(rlb_ctx* ctx, float* x, const float* y, int64_t count, int round_f16);
// Optional wait of the arg-max kernels for pushed logits (tensor-parallel push mode), and the
// per-step epoch counter they advance.
struct StepSync {
    const uint2* ll_logits = nullptr;  // push mode: {value, sequence} entries written by every rank's head kernel
    float* dense_out = nullptr;        // ... unpacked here while they are polled
    uint32_t seq_idx = 0, seq_stride = 0;
    int32_t* epoch = nullptr;          // incremented once per decode step (if set)
    int32_t* err = nullptr;            // raised when a poll runs out
};
int launch_argmax(rlb_ctx* ctx, const float* logits, int n, int32_t* out_tok, const StepSync& sync = StepSync());
// greedy feedback: tok <- argmax, pos <- pos + 1, tokens_out[step] <- tok, step <- step + 1
int launch_argmax_advance(rlb_ctx* ctx, const float* logits, int n, int32_t* tok, int32_t* pos, int32_t* step,
                          int32_t* tokens_out, int32_t tokens_cap, const StepSync& sync = StepSync());
int launch_convert(rlb_ctx* ctx, const void* src, rlb_dtype src_dtype, int64_t src_ld, void* dst, rlb_dtype dst_dtype,
                   int64_t dst_ld, int64_t rows, int64_t cols);
int launch_silu(rlb_ctx* ctx, void* t, rlb_dtype dtype, int64_t rows, int64_t cols, int64_t cap);
int launch_hadamard(rlb_ctx* ctx, void* dst, const void* other, rlb_dtype dtype, int64_t rows, int64_t cols,
                    int64_t dst_cap, int64_t other_cap);
int launch_transpose(rlb_ctx* ctx, void* dst, const void* src, rlb_dtype dtype, int64_t dst_rows, int64_t dst_cols,
                     int64_t dst_cap, int64_t src_cap);
int launch_cache_shift_left(rlb_ctx* ctx, void* cache, rlb_dtype dtype, int64_t heads, int max_seq, int hd, int shifts);

// ---------------------------------------------------------------------------------------
// prefill GEMM (gemm.cu): C[n][M] f32 = A[n][K] * W[M][K]^T, optional f16 rounding of the result
// ---------------------------------------------------------------------------------------
// err: device-visible error word for the tensor-core path (nullptr: the context's word).
int launch_gemm_nt(rlb_ctx* ctx, rlb_dtype dtype, const void* A, int64_t lda, const void* W, int64_t ldw, float* C,
                   int64_t ldc, int n, int M, int K, int round_out, int* err = nullptr, int w_f16_exact = 0);
// (w_f16_exact: the f32 weights hold f16-representable values, so the two-pass TF32 tensor-core form is exact enough)
// Same contraction, output stored in the operand dtype (tier-1 op).
int launch_gemm_nt_typed(rlb_ctx* ctx, rlb_dtype dtype, const void* A, int64_t lda, const void* W, int64_t ldw, void* C,
                         int64_t ldc, int n, int M, int K);

// tcgen05 tile kernel for f16 operands (gemm_tc.cu)
bool gemm_tc_supported(const void* X, int64_t ldx, const void* W, int64_t ldw, int n, int M, int K);
// f32 operands whose weights hold f16-representable values (two TF32 passes over activations split into hi + lo)
bool gemm_tc_f32_supported(const void* X, int64_t ldx, const void* W, int64_t ldw, int n, int M, int K);
int launch_gemm_tc_f32w(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, float* C, int64_t ldc, int n, int M, int K,
                        int* err);
int launch_gemm_tc_f32out(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, float* C, int64_t ldc, int n, int M,
                          int K, int round_out, int* err);
int launch_gemm_tc_f16out(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, void* C, int64_t ldc, int n, int M,
                          int K, int* err);

// ---------------------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------------------
#ifdef __CUDACC__
// Programmatic dependent launch: rlb_pdl_trigger lets the next kernel of the stream start launching now;
// rlb_pdl_wait blocks until the previous kernel has completed and its writes are visible. Both are no-ops in a
// kernel launched the ordinary way. A kernel launched through rlb_launch must execute the wait in every CTA
// before it reads or writes anything an earlier kernel touches.
__device__ __forceinline__ void rlb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void rlb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Kernel launch on the context's stream; as a programmatic dependent while ctx->pdl_chain is set.
template <typename... KA, typename... A>
inline cudaError_t rlb_launch(void (*kern)(KA...), dim3 grid, dim3 block, size_t smem, rlb_ctx* ctx, A&&... args) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid; lc.blockDim = block; lc.dynamicSmemBytes = smem; lc.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = ctx->pdl_chain ? 1 : 0;
    return cudaLaunchKernelEx(&lc, kern, std::forward<A>(args)...);
}
#endif
static inline void count_launch(rlb_ctx* ctx, uint64_t n = 1) { ctx->launches += n; }
// Function attributes (shared-memory opt-in) are per device: a call site keeps one bit per device index in
// `mask`, tests it with attr_done and sets it with attr_mark once cudaFuncSetAttribute has succeeded there.
// Two threads may both set the attribute the first time; that is harmless.
static inline bool attr_done(const std::atomic<uint64_t>& mask, int device) { return (mask.load(std::memory_order_acquire) >> (device & 63)) & 1u; }
static inline void attr_mark(std::atomic<uint64_t>& mask, int device) { mask.fetch_or(1ull << (device & 63), std::memory_order_release); }
#define RLB_LAUNCH_CHECK()                                                                         \
    do {                                                                                           \
        cudaError_t _e = cudaGetLastError();                                                       \
        if (_e != cudaSuccess)                                                                     \
            return rlb_fail(RLB_ERR_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), \
                            __FILE__, __LINE__);                                                   \
    } while (0)

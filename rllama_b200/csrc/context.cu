// Context, device tensors and the op-level (tier-1) entry points: the CUDA counterpart of
// rllama's `OpenCL` / `OpenCLTensor` / `OpenCLEvent` (src/tensor_opencl_support.rs:30-57,
// :86-412) as used by Tensor's residency dispatch (src/tensor.rs:679-698, :768-781, :911-924,
// :999-1025, :2127-2206).
#include "internal.h"

#include <cstdarg>
#include <cstring>

namespace {
thread_local char g_err[1024] = "";
}

int rlb_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int ctx_check_error_word(rlb_ctx* ctx) {
    if (ctx && ctx->h_err && *reinterpret_cast<volatile int*>(ctx->h_err) != 0)
        return rlb_fail(RLB_ERR_CUDA, "a kernel gave up on a bounded wait (code %d); results on this context are invalid", *ctx->h_err);
    return RLB_OK;
}

extern "C" {

const char* rlb_last_error(void) { return g_err; }

int rlb_device_count(int* count) {
    if (!count) return rlb_fail(RLB_ERR_INVALID, "rlb_device_count: null pointer");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        return rlb_fail(RLB_ERR_NO_DEVICE, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
    }
    *count = n;
    return RLB_OK;
}

int rlb_ctx_create(int verbose, int nth_device, rlb_ctx** out) {
    if (!out) return rlb_fail(RLB_ERR_INVALID, "rlb_ctx_create: null out pointer");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return rlb_fail(RLB_ERR_NO_DEVICE, "no CUDA device: %s (this backend has no CPU fallback)", cudaGetErrorString(e));
    if (verbose) {
        printf("Enumerating CUDA devices:\n");
        for (int i = 0; i < n; i++) {
            cudaDeviceProp p;
            if (cudaGetDeviceProperties(&p, i) == cudaSuccess) printf("CUDA %d device: %s\n", i, p.name);
        }
    }
    if (nth_device < 0 || nth_device >= n) return rlb_fail(RLB_ERR_NO_DEVICE, "cannot select device %d of %d", nth_device, n);
    cudaDeviceProp prop;
    RLB_CUDA(cudaGetDeviceProperties(&prop, nth_device));
    if (prop.major != 10)
        return rlb_fail(RLB_ERR_NO_DEVICE, "device %d (%s) is compute capability %d.%d; this library is built for sm_100a only",
                        nth_device, prop.name, prop.major, prop.minor);
    if (verbose) printf("---\nSelected CUDA device: %s\n", prop.name);
    RLB_CUDA(cudaSetDevice(nth_device));
    rlb_ctx* ctx = new rlb_ctx();
    ctx->device = nth_device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->verbose = verbose != 0;
    cudaError_t se = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (se == cudaSuccess) se = cudaHostAlloc((void**)&ctx->h_err, 64, cudaHostAllocMapped);
    if (se == cudaSuccess) {
        *ctx->h_err = 0;
        se = cudaHostGetDevicePointer((void**)&ctx->d_err, ctx->h_err, 0);
    }
    if (se != cudaSuccess) {
        if (ctx->stream) cudaStreamDestroy(ctx->stream);
        if (ctx->h_err) cudaFreeHost(ctx->h_err);
        delete ctx;
        return rlb_fail(RLB_ERR_CUDA, "context set-up: %s", cudaGetErrorString(se));
    }
    *out = ctx;
    return RLB_OK;
}

int rlb_ctx_destroy(rlb_ctx* ctx) {
    if (!ctx) return RLB_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->op_scratch) cudaFree(ctx->op_scratch);
    if (ctx->gemm_scratch) cudaFree(ctx->gemm_scratch);
    if (ctx->h_err) cudaFreeHost(ctx->h_err);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return RLB_OK;
}

int rlb_ctx_flush(rlb_ctx* ctx) {
    if (!ctx) return rlb_fail(RLB_ERR_INVALID, "rlb_ctx_flush: null context");
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    RLB_CUDA(cudaStreamSynchronize(ctx->stream));
    return ctx_check_error_word(ctx);
}

int rlb_ctx_kernel_launches(rlb_ctx* ctx, uint64_t* count) {
    if (!ctx || !count) return rlb_fail(RLB_ERR_INVALID, "rlb_ctx_kernel_launches: null pointer");
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    *count = ctx->launches;
    return RLB_OK;
}

static int tensor_new(rlb_ctx* ctx, int64_t rows, int64_t cols, int64_t cap, rlb_dtype dtype, rlb_tensor** out) {
    if (!ctx || !out) return rlb_fail(RLB_ERR_INVALID, "tensor: null pointer");
    if (rows < 0 || cols < 0 || cap < cols || (dtype != RLB_F16 && dtype != RLB_F32))
        return rlb_fail(RLB_ERR_INVALID, "tensor: bad shape %lldx%lld (capacity %lld) or dtype %d", (long long)rows, (long long)cols,
                        (long long)cap, (int)dtype);
    // 128-bit vector access needs 16-byte aligned rows
    if ((cap * (int64_t)dtype_size(dtype)) % 16 != 0)
        return rlb_fail(RLB_ERR_INVALID, "tensor: capacity_cols %lld does not give 16-byte aligned rows", (long long)cap);
    rlb_tensor* t = new rlb_tensor();
    t->ctx = ctx; t->rows = rows; t->cols = cols; t->cap = cap; t->dtype = dtype;
    cudaSetDevice(ctx->device);
    size_t bytes = t->bytes();
    cudaError_t e = cudaMalloc(&t->d, bytes ? bytes : 16);
    if (e != cudaSuccess) {
        delete t;
        return rlb_fail(RLB_ERR_OOM, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    }
    e = cudaEventCreateWithFlags(&t->ready, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        cudaFree(t->d);
        delete t;
        return rlb_fail(RLB_ERR_CUDA, "cudaEventCreate: %s", cudaGetErrorString(e));
    }
    *out = t;
    return RLB_OK;
}

int rlb_tensor_upload(rlb_ctx* ctx, const void* host, int64_t rows, int64_t cols, int64_t capacity_cols, rlb_dtype dtype,
                      rlb_tensor** out) {
    if (!host) return rlb_fail(RLB_ERR_INVALID, "rlb_tensor_upload: null host pointer");
    RLB_TRY(tensor_new(ctx, rows, cols, capacity_cols, dtype, out));
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    rlb_tensor* t = *out;
    cudaError_t e = cudaMemcpyAsync(t->d, host, t->bytes(), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaEventRecord(t->ready, ctx->stream);
    if (e != cudaSuccess) {
        rlb_tensor_free(t);
        *out = nullptr;
        return rlb_fail(RLB_ERR_CUDA, "upload: %s", cudaGetErrorString(e));
    }
    return RLB_OK;
}

int rlb_tensor_zeros(rlb_ctx* ctx, int64_t rows, int64_t cols, int64_t capacity_cols, rlb_dtype dtype, rlb_tensor** out) {
    RLB_TRY(tensor_new(ctx, rows, cols, capacity_cols, dtype, out));
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    rlb_tensor* t = *out;
    cudaError_t e = cudaMemsetAsync(t->d, 0, t->bytes(), ctx->stream);
    if (e == cudaSuccess) e = cudaEventRecord(t->ready, ctx->stream);
    if (e != cudaSuccess) {
        rlb_tensor_free(t);
        *out = nullptr;
        return rlb_fail(RLB_ERR_CUDA, "zeros: %s", cudaGetErrorString(e));
    }
    return RLB_OK;
}

int rlb_tensor_wait(rlb_tensor* t) {
    if (!t) return rlb_fail(RLB_ERR_INVALID, "rlb_tensor_wait: null tensor");
    RLB_CUDA(cudaEventSynchronize(t->ready));
    return ctx_check_error_word(t->ctx);
}

int rlb_tensor_download(rlb_tensor* t, void* host, rlb_event** out_event) {
    if (!t || !host || !out_event) return rlb_fail(RLB_ERR_INVALID, "rlb_tensor_download: null pointer");
    rlb_ctx* ctx = t->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    rlb_event* ev = new rlb_event();
    ev->ctx = ctx;
    cudaError_t e = cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaMemcpyAsync(host, t->d, t->bytes(), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaEventRecord(ev->ev, ctx->stream);
    if (e != cudaSuccess) {
        if (ev->ev) cudaEventDestroy(ev->ev);
        delete ev;
        return rlb_fail(RLB_ERR_CUDA, "download: %s", cudaGetErrorString(e));
    }
    *out_event = ev;
    return RLB_OK;
}

int rlb_event_wait(rlb_event* ev) {
    if (!ev) return rlb_fail(RLB_ERR_INVALID, "rlb_event_wait: null event");
    cudaError_t e = cudaEventSynchronize(ev->ev);
    rlb_ctx* ctx = ev->ctx;
    cudaEventDestroy(ev->ev);
    delete ev;
    if (e != cudaSuccess) return rlb_fail(RLB_ERR_CUDA, "event wait: %s", cudaGetErrorString(e));
    return ctx_check_error_word(ctx);
}

int rlb_tensor_free(rlb_tensor* t) {
    if (!t) return RLB_OK;
    cudaSetDevice(t->ctx->device);
    if (t->ready) {
        cudaEventSynchronize(t->ready);  // the reference also waits for the initial write before dropping
        cudaEventDestroy(t->ready);
    }
    if (t->d) cudaFree(t->d);
    delete t;
    return RLB_OK;
}

static int same_ctx(const rlb_tensor* a, const rlb_tensor* b) {
    if (!a || !b) return rlb_fail(RLB_ERR_INVALID, "null tensor");
    if (a->ctx != b->ctx) return rlb_fail(RLB_ERR_INVALID, "tensors live on different contexts");
    return RLB_OK;
}

#define OP_PROLOGUE(ctxvar, t)                              \
    rlb_ctx* ctxvar = (t)->ctx;                             \
    std::lock_guard<std::recursive_mutex> _g(ctxvar->mu);   \
    RLB_CUDA(cudaSetDevice(ctxvar->device));

int rlb_copy_inplace(rlb_tensor* dst, const rlb_tensor* src) {
    RLB_TRY(same_ctx(dst, src));
    if (dst->rows != src->rows || dst->cols != src->cols || dst->dtype != src->dtype)
        return rlb_fail(RLB_ERR_INVALID, "copy_inplace: shape or dtype mismatch");
    OP_PROLOGUE(ctx, dst);
    RLB_CUDA(cudaMemcpy2DAsync(dst->d, dst->cap * dtype_size(dst->dtype), src->d, src->cap * dtype_size(src->dtype),
                               (size_t)src->cols * dtype_size(src->dtype), (size_t)src->rows, cudaMemcpyDeviceToDevice, ctx->stream));
    RLB_CUDA(cudaEventRecord(dst->ready, ctx->stream));
    return RLB_OK;
}

int rlb_transpose_from(rlb_tensor* dst, const rlb_tensor* src) {
    RLB_TRY(same_ctx(dst, src));
    if (dst->rows != src->cols || dst->cols != src->rows || dst->dtype != src->dtype)
        return rlb_fail(RLB_ERR_INVALID, "transpose_from: %lldx%lld cannot hold the transpose of %lldx%lld", (long long)dst->rows,
                        (long long)dst->cols, (long long)src->rows, (long long)src->cols);
    OP_PROLOGUE(ctx, dst);
    RLB_TRY(launch_transpose(ctx, dst->d, src->d, dst->dtype, dst->rows, dst->cols, dst->cap, src->cap));
    RLB_CUDA(cudaEventRecord(dst->ready, ctx->stream));
    return RLB_OK;
}

int rlb_hadamard_product_inplace(rlb_tensor* dst, const rlb_tensor* other) {
    RLB_TRY(same_ctx(dst, other));
    if (dst->rows != other->rows || dst->cols != other->cols || dst->dtype != other->dtype)
        return rlb_fail(RLB_ERR_INVALID, "hadamard_product_inplace: shape or dtype mismatch");
    OP_PROLOGUE(ctx, dst);
    RLB_TRY(launch_hadamard(ctx, dst->d, other->d, dst->dtype, dst->rows, dst->cols, dst->cap, other->cap));
    RLB_CUDA(cudaEventRecord(dst->ready, ctx->stream));
    return RLB_OK;
}

int rlb_silu_inplace(rlb_tensor* t) {
    if (!t) return rlb_fail(RLB_ERR_INVALID, "silu_inplace: null tensor");
    OP_PROLOGUE(ctx, t);
    RLB_TRY(launch_silu(ctx, t->d, t->dtype, t->rows, t->cols, t->cap));
    RLB_CUDA(cudaEventRecord(t->ready, ctx->stream));
    return RLB_OK;
}

int rlb_matrix_mul_inplace_transposed(rlb_tensor* dst, const rlb_tensor* src, const rlb_tensor* other) {
    RLB_TRY(same_ctx(dst, src));
    RLB_TRY(same_ctx(dst, other));
    // the reference's panics (src/tensor.rs:1261-1278)
    if (src->cols != other->cols)
        return rlb_fail(RLB_ERR_INVALID, "Invalid matrix multiplication %lldx%lld vs %lldx%lld", (long long)src->rows, (long long)src->cols,
                        (long long)other->rows, (long long)other->cols);
    if (src->dtype != other->dtype || dst->dtype != src->dtype) return rlb_fail(RLB_ERR_INVALID, "Invalid matrix multiplication, different dtypes");
    if (dst->rows != src->rows) return rlb_fail(RLB_ERR_INVALID, "Invalid matrix multiplication, different number of rows");
    if (dst->cols != other->rows) return rlb_fail(RLB_ERR_INVALID, "Invalid matrix multiplication, different number of cols");
    OP_PROLOGUE(ctx, dst);
    const int vec = dst->dtype == RLB_F16 ? 8 : 4;
    // Rows are zero padded up to capacity_cols (src/tensor.rs:433-450), so the contraction may
    // run over the padded length.
    const int64_t kp = (src->cols + vec - 1) / vec * vec;
    const bool padded_ok = kp <= src->cap && kp <= other->cap;
    if (src->rows == 1 && padded_ok && other->rows > 0) {
        GemvArgs a;
        a.W = other->d; a.rows = (int)other->rows; a.K = (int)kp; a.ldw = other->cap;
        a.vec_in = src->d; a.out = dst->d; a.out_stride = 1;
        RLB_TRY(launch_gemv(ctx, dst->dtype, PRO_COPY, EPI_STORE, a));
    } else if (other->rows == 1 && padded_ok && src->rows > 0) {
        GemvArgs a;
        a.W = src->d; a.rows = (int)src->rows; a.K = (int)kp; a.ldw = src->cap;
        a.vec_in = other->d; a.out = dst->d; a.out_stride = dst->cap;
        RLB_TRY(launch_gemv(ctx, dst->dtype, PRO_COPY, EPI_STORE, a));
    } else if (src->rows > 0 && other->rows > 0) {
        RLB_TRY(launch_gemm_nt_typed(ctx, dst->dtype, src->d, src->cap, other->d, other->cap, dst->d, dst->cap, (int)src->rows,
                                     (int)other->rows, (int)src->cols));
    }
    RLB_CUDA(cudaEventRecord(dst->ready, ctx->stream));
    return RLB_OK;
}

}  // extern "C"

// Shape checks shared by the attention entry points. Returns the head dimension in *hd_out.
int attention_check(const rlb_tensor* out, const rlb_tensor* q, const rlb_tensor* kcache, const rlb_tensor* vcache, int32_t heads,
                    int32_t max_seq_len, int32_t pos, int32_t n_split, int* hd_out) {
    RLB_TRY(same_ctx(out, q));
    RLB_TRY(same_ctx(out, kcache));
    RLB_TRY(same_ctx(out, vcache));
    if (heads < 1 || max_seq_len < 1 || pos < 0 || pos >= max_seq_len || n_split < 1 || n_split > 64)
        return rlb_fail(RLB_ERR_INVALID, "attention: bad heads %d, max_seq_len %d, pos %d or n_split %d", heads, max_seq_len, pos, n_split);
    const int64_t hd = kcache->cols;
    if (kcache->cap != hd || vcache->cap != hd || vcache->cols != hd || kcache->rows != (int64_t)heads * max_seq_len ||
        vcache->rows != kcache->rows || kcache->dtype != vcache->dtype)
        return rlb_fail(RLB_ERR_INVALID, "attention: caches must be (heads*max_seq_len) x head_dim without row padding");
    if (q->dtype != RLB_F32 || q->rows != 1 || q->cols != (int64_t)heads * hd) return rlb_fail(RLB_ERR_INVALID, "attention: q must be 1 x heads*head_dim f32");
    if (out->dtype != kcache->dtype || out->rows != 1 || out->cols != (int64_t)heads * hd)
        return rlb_fail(RLB_ERR_INVALID, "attention: out must be 1 x heads*head_dim in the cache dtype");
    *hd_out = (int)hd;
    return RLB_OK;
}

extern "C" int rlb_attention_decode(rlb_tensor* out, const rlb_tensor* q, const rlb_tensor* kcache, const rlb_tensor* vcache, int32_t heads,
                                    int32_t max_seq_len, int32_t pos, int32_t n_split) {
    int hd = 0;
    RLB_TRY(attention_check(out, q, kcache, vcache, heads, max_seq_len, pos, n_split, &hd));
    OP_PROLOGUE(ctx, out);
    // scratch: [pos : 256 B][counters : heads, padded to 256 B][records]
    const size_t cnt_bytes = ((size_t)heads * sizeof(unsigned int) + 255) & ~(size_t)255;
    const size_t need = 256 + cnt_bytes + attn_decode_scratch_floats(heads, hd, n_split) * sizeof(float);
    if (need > ctx->op_scratch_bytes) {
        RLB_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->op_scratch) cudaFree(ctx->op_scratch);
        ctx->op_scratch = nullptr;
        ctx->op_scratch_bytes = 0;
        cudaError_t e = cudaMalloc(&ctx->op_scratch, need);
        if (e != cudaSuccess) return rlb_fail(RLB_ERR_OOM, "attention scratch (%zu bytes): %s", need, cudaGetErrorString(e));
        ctx->op_scratch_bytes = need;
    }
    char* base = (char*)ctx->op_scratch;
    RLB_CUDA(cudaMemsetAsync(base, 0, 256 + cnt_bytes, ctx->stream));
    AttnDecodeArgs a;
    a.q = (const float*)q->d; a.kcache = kcache->d; a.vcache = vcache->d; a.out = out->d;
    a.pos_ptr = nullptr; a.pos_value = pos;  // by value: no copy from a stack variable on the stream
    a.heads = heads; a.hd = hd; a.max_seq = max_seq_len; a.n_split = n_split;
    a.counters = (unsigned int*)(base + 256);
    a.scratch = (float*)(base + 256 + cnt_bytes);
    RLB_TRY(launch_attn_decode(ctx, kcache->dtype, a, 0));
    RLB_CUDA(cudaEventRecord(out->ready, ctx->stream));
    return RLB_OK;
}

// The per-head part of Attention::forward for a multi-token call as a standalone op: row i of q attends to
// positions 0 .. start_pos + i of the caches (the mask of Tensor::full_triu, src/tensor.rs:496-508).
extern "C" int rlb_attention_prefill(rlb_tensor* out, const rlb_tensor* q, const rlb_tensor* kcache, const rlb_tensor* vcache, int32_t heads,
                                     int32_t max_seq_len, int32_t start_pos, int32_t tensor_cores) {
    RLB_TRY(same_ctx(out, q));
    RLB_TRY(same_ctx(out, kcache));
    RLB_TRY(same_ctx(out, vcache));
    const int64_t n = q->rows, hd = kcache->cols;
    if (heads < 1 || max_seq_len < 1 || n < 1 || start_pos < 0 || start_pos + n > max_seq_len)
        return rlb_fail(RLB_ERR_INVALID, "attention_prefill: bad heads %d, max_seq_len %d, start_pos %d or %lld rows", heads, max_seq_len, start_pos,
                        (long long)n);
    if (kcache->cap != hd || vcache->cap != hd || vcache->cols != hd || kcache->rows != (int64_t)heads * max_seq_len ||
        vcache->rows != kcache->rows || kcache->dtype != vcache->dtype)
        return rlb_fail(RLB_ERR_INVALID, "attention_prefill: caches must be (heads*max_seq_len) x head_dim without row padding");
    if (q->dtype != RLB_F32 || q->cols != (int64_t)heads * hd) return rlb_fail(RLB_ERR_INVALID, "attention_prefill: q must be n x heads*head_dim f32");
    if (out->dtype != kcache->dtype || out->rows != n || out->cols != q->cols || out->cap != out->cols)
        return rlb_fail(RLB_ERR_INVALID, "attention_prefill: out must be n x heads*head_dim in the cache dtype, without row padding");
    OP_PROLOGUE(ctx, out);
    AttnPrefillArgs a;
    a.q = (const float*)q->d; a.q_ld = q->cap; a.kcache = kcache->d; a.vcache = vcache->d; a.out = out->d;
    a.n = (int)n; a.start_pos = start_pos; a.heads = heads; a.hd = (int)hd; a.max_seq = max_seq_len;
    a.allow_tc = tensor_cores != 0;
    RLB_TRY(launch_attn_prefill(ctx, kcache->dtype, a));
    RLB_CUDA(cudaEventRecord(out->ready, ctx->stream));
    return RLB_OK;
}

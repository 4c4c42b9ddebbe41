// Decode-time weight streaming: y = W * a for one activation row, the contraction that
// rllama runs as Tensor::matrix_mul_transposed with a one-row operand
// (src/tensor.rs:999-1025; CPU kernels :1250-1668 and :1837-1918; OpenCL kernel
// matrix_mul_transposed_one_row_f16, src/tensor_opencl_support.rs:559-616).
//
// The kernel is bound by HBM bandwidth: every weight is read exactly once per token.
//  * a persistent grid (a small multiple of the SM count); each warp owns R consecutive
//    weight rows at a time and walks K with 128-bit no-allocate loads, 16 independent
//    loads in flight per thread;
//  * the activation row is staged once per CTA in shared memory; the prologue that
//    produces it is fused: residual add of the previous projection's partial sums,
//    RMSNorm (src/transformer.rs:476-480) and the cast to the weight dtype;
//  * f16 weights are widened to f32, multiplied and accumulated in f32 (products of two
//    f16 values are exact in f32), and the f16 rounding of the result happens in the
//    fused epilogue, at the points where the reference rounds
//    (src/transformer.rs:538-570, :666-702, :793-819);
//  * epilogues: RoPE + KV-cache append for q/k/v (src/transformer.rs:719-761, :823-856),
//    SiLU gate for w1/w3 (src/transformer.rs:551-565, src/tensor.rs:822-832), raw f32
//    partial sums for wo / w2 / the vocabulary head.
#include "internal.h"

#include <cstdlib>

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <typename T> struct Vec;
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}

__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }

template <typename T> __device__ __forceinline__ T cast_to(float v);
template <> __device__ __forceinline__ __half cast_to<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast_to<float>(float v) { return v; }

template <typename T> __device__ __forceinline__ float maybe_round(float v);
template <> __device__ __forceinline__ float maybe_round<__half>(float v) { return round_f16(v); }
template <> __device__ __forceinline__ float maybe_round<float>(float v) { return v; }

template <typename T> __device__ __forceinline__ void unpack(const uint4& v, float (&f)[Vec<T>::N]);
template <> __device__ __forceinline__ void unpack<__half>(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template <> __device__ __forceinline__ void unpack<float>(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the CTA; every thread receives the same value (fixed combination order).
__device__ __forceinline__ float block_sum(float v, float* red /* [kWarps] */) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; w++) t += red[w];
    __syncthreads();
    return t;
}

template <typename WT, int R, int PRO, int EPI>
__global__ void __launch_bounds__(kThreads) gemv_kernel(const GemvArgs a) {
    constexpr int VEC = Vec<WT>::N;
    constexpr int CH = 32 * VEC;  // elements one warp covers with one 128-bit load per lane
    constexpr int NMAT = (EPI == EPI_SWIGLU) ? 2 : 1;
    constexpr int U = (R * NMAT >= 16) ? 1 : (R * NMAT >= 8) ? 2 : (R * NMAT >= 4) ? 4 : 8;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float red[kWarps];
    WT* act = reinterpret_cast<WT*>(smem_raw);
    const int K = a.K;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---------------- prologue: build the activation row in shared memory ----------------
    if (PRO == PRO_COPY) {
        const uint4* src = reinterpret_cast<const uint4*>(a.vec_in);
        uint4* dst = reinterpret_cast<uint4*>(act);
        for (int i = tid; i < K / VEC; i += kThreads) dst[i] = src[i];
    } else {
        float* tmp = reinterpret_cast<float*>(smem_raw + (((size_t)K * sizeof(WT) + 15) & ~(size_t)15));
        const float* xin = a.x_in;
        if (a.tok_ptr) xin += (int64_t)(*a.tok_ptr) * K;
        float ss = 0.f;
        for (int i = tid * 4; i < K; i += kThreads * 4) {
            float4 v = *reinterpret_cast<const float4*>(xin + i);
            if (a.n_parts > 0) {
                float4 s = *reinterpret_cast<const float4*>(a.parts + i);
                for (int p = 1; p < a.n_parts; p++) {  // fixed rank order: identical on every rank
                    const float4 t = *reinterpret_cast<const float4*>(a.parts + p * a.part_stride + i);
                    s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
                }
                if (a.round_parts) {
                    s.x = round_f16(s.x); s.y = round_f16(s.y); s.z = round_f16(s.z); s.w = round_f16(s.w);
                }
                v.x += s.x; v.y += s.y; v.z += s.z; v.w += s.w;
            }
            *reinterpret_cast<float4*>(tmp + i) = v;
            if (blockIdx.x == 0 && a.x_out) *reinterpret_cast<float4*>(a.x_out + i) = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, red);
        const float scale = 1.0f / sqrtf(ss / (float)K + a.eps);
        for (int i = tid; i < K; i += kThreads) act[i] = cast_to<WT>(__fmul_rn(__fmul_rn(tmp[i], scale), a.gain[i]));
    }
    __syncthreads();

    // ---------------- main loop: R rows per warp, grid-stride over row groups -------------
    const int n_groups = a.rows / R;
    const WT* W0 = reinterpret_cast<const WT*>(a.W);
    const WT* W1 = reinterpret_cast<const WT*>(a.W2);
    for (int g = blockIdx.x * kWarps + warp; g < n_groups; g += gridDim.x * kWarps) {
        const int row0 = g * R;
        float acc[NMAT][R];
#pragma unroll
        for (int m = 0; m < NMAT; m++)
#pragma unroll
            for (int r = 0; r < R; r++) acc[m][r] = 0.f;

        const WT* wp0 = W0 + (int64_t)row0 * a.ldw;
        const WT* wp1 = NMAT == 2 ? W1 + (int64_t)row0 * a.ldw : nullptr;
        int k = lane * VEC;
        for (; k + (U - 1) * CH < K; k += U * CH) {
            uint4 wv[U][NMAT][R];
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int r = 0; r < R; r++) {
                    wv[u][0][r] = ld_stream(wp0 + (int64_t)r * a.ldw + k + u * CH);
                    if (NMAT == 2) wv[u][NMAT - 1][r] = ld_stream(wp1 + (int64_t)r * a.ldw + k + u * CH);
                }
#pragma unroll
            for (int u = 0; u < U; u++) {
                float af[VEC];
                unpack<WT>(*reinterpret_cast<const uint4*>(act + k + u * CH), af);
#pragma unroll
                for (int m = 0; m < NMAT; m++)
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        float wf[VEC];
                        unpack<WT>(wv[u][m][r], wf);
#pragma unroll
                        for (int e = 0; e < VEC; e++) acc[m][r] = fmaf(wf[e], af[e], acc[m][r]);
                    }
            }
        }
        for (; k < K; k += CH) {
            float af[VEC];
            unpack<WT>(*reinterpret_cast<const uint4*>(act + k), af);
#pragma unroll
            for (int r = 0; r < R; r++) {
                float wf[VEC];
                unpack<WT>(ld_stream(wp0 + (int64_t)r * a.ldw + k), wf);
#pragma unroll
                for (int e = 0; e < VEC; e++) acc[0][r] = fmaf(wf[e], af[e], acc[0][r]);
                if (NMAT == 2) {
                    unpack<WT>(ld_stream(wp1 + (int64_t)r * a.ldw + k), wf);
#pragma unroll
                    for (int e = 0; e < VEC; e++) acc[NMAT - 1][r] = fmaf(wf[e], af[e], acc[NMAT - 1][r]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < NMAT; m++)
#pragma unroll
            for (int r = 0; r < R; r++) acc[m][r] = warp_sum(acc[m][r]);

        // ---------------- epilogue -----------------------------------------------------------
        if (EPI == EPI_STORE) {
            WT* out = reinterpret_cast<WT*>(a.out);
#pragma unroll
            for (int r = 0; r < R; r++)
                if (lane == r) out[(int64_t)(row0 + r) * a.out_stride] = cast_to<WT>(acc[0][r]);
        } else if (EPI == EPI_F32) {
#pragma unroll
            for (int r = 0; r < R; r++)
                if (lane == r) {
                    reinterpret_cast<float*>(a.out)[(int64_t)(row0 + r) * a.out_stride] = acc[0][r];
                }
        } else if (EPI == EPI_SWIGLU) {
            WT* out = reinterpret_cast<WT*>(a.out);
#pragma unroll
            for (int r = 0; r < R; r++)
                if (lane == r) {
                    const float a1 = maybe_round<WT>(acc[0][r]);
                    const float a3 = maybe_round<WT>(acc[NMAT - 1][r]);
                    const float s = a1 / (1.0f + expf(-a1));
                    out[row0 + r] = cast_to<WT>(__fmul_rn(s, a3));
                }
        } else if (EPI == EPI_QKV) {
            if (R >= 2) {
                const int pos = *a.pos_ptr;
#pragma unroll
                for (int j = 0; j < R / 2; j++)
                    if (lane == j) {
                        const int row = row0 + 2 * j;
                        const int sec = row / a.nq, rr = row - sec * a.nq;
                        const int head = rr / a.hd, c = rr - head * a.hd;  // c is even
                        const float re = maybe_round<WT>(acc[0][2 * j]);
                        const float im = maybe_round<WT>(acc[0][2 * j + 1]);
                        const float* f = a.rope + ((int64_t)pos * (a.hd / 2) + (c >> 1)) * 2;
                        const float fr = f[0], fi = f[1];
                        // src/transformer.rs:844-847, no contraction into FMA
                        const float rr_ = __fsub_rn(__fmul_rn(re, fr), __fmul_rn(im, fi));
                        const float ri_ = __fadd_rn(__fmul_rn(re, fi), __fmul_rn(im, fr));
                        if (sec == 0) {
                            a.qbuf[rr] = rr_;
                            a.qbuf[rr + 1] = ri_;
                        } else {
                            WT* cache = reinterpret_cast<WT*>(sec == 1 ? a.kcache : a.vcache);
                            WT* dst = cache + ((int64_t)head * a.max_seq + pos) * a.hd + c;
                            dst[0] = cast_to<WT>(sec == 1 ? rr_ : re);
                            dst[1] = cast_to<WT>(sec == 1 ? ri_ : im);
                        }
                    }
            }
        }
    }

}

struct Tuning {
    int rows_per_warp = 0;  // 0 = choose from shape
    int ctas_per_sm = 0;
    bool loaded = false;
} g_tune;

void load_tuning() {
    if (g_tune.loaded) return;
    g_tune.loaded = true;
    if (const char* s = getenv("RLB_GEMV_ROWS")) g_tune.rows_per_warp = atoi(s);
    if (const char* s = getenv("RLB_GEMV_CTAS")) g_tune.ctas_per_sm = atoi(s);
}

template <typename WT, int R, int PRO, int EPI>
int launch_one(rlb_ctx* ctx, const GemvArgs& a, int ctas_per_sm) {
    static std::atomic<uint64_t> attr_set{0};
    auto kern = gemv_kernel<WT, R, PRO, EPI>;
    size_t smem = (((size_t)a.K * sizeof(WT)) + 15) & ~(size_t)15;
    if (PRO == PRO_NORM) smem += (size_t)a.K * sizeof(float);
    if (smem > 200 * 1024) return rlb_fail(RLB_ERR_LIMIT, "gemv: activation row of %d elements does not fit in shared memory", a.K);
    if (!attr_done(attr_set, ctx->device)) {
        RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_mark(attr_set, ctx->device);
    }
    const int n_groups = a.rows / R;
    int grid = (n_groups + kWarps - 1) / kWarps;
    const int max_grid = ctx->sm_count * ctas_per_sm;
    if (grid > max_grid) grid = max_grid;
    if (grid < 1) grid = 1;
    kern<<<grid, kThreads, smem, ctx->stream>>>(a);
    RLB_LAUNCH_CHECK();
    count_launch(ctx);
    return RLB_OK;
}

template <typename WT, int PRO, int EPI>
int launch_rows(rlb_ctx* ctx, const GemvArgs& a) {
    load_tuning();
    int R = g_tune.rows_per_warp;
    if (R == 0) R = (EPI == EPI_SWIGLU) ? 2 : 4;
    int unit = (EPI == EPI_QKV) ? a.nq : a.rows;  // row groups must not straddle q/k/v sections
    while (R > 1 && (unit % R != 0 || a.rows % R != 0)) R >>= 1;
    if (EPI == EPI_QKV && R < 2) return rlb_fail(RLB_ERR_INVALID, "gemv: q/k/v projection needs an even number of rows per head");
    int ctas = g_tune.ctas_per_sm ? g_tune.ctas_per_sm : 2;
    // keep shared memory per SM within reach: large activation rows lower residency anyway
    switch (R) {
        case 8: return launch_one<WT, 8, PRO, EPI>(ctx, a, ctas);
        case 4: return launch_one<WT, 4, PRO, EPI>(ctx, a, ctas);
        case 2: return launch_one<WT, 2, PRO, EPI>(ctx, a, ctas);
        default:
            if (EPI == EPI_QKV) return rlb_fail(RLB_ERR_INVALID, "gemv: bad rows per warp");
            return launch_one<WT, 1, PRO, (EPI == EPI_QKV ? EPI_F32 : EPI)>(ctx, a, ctas);
    }
}

template <typename WT>
int launch_typed(rlb_ctx* ctx, int prologue, int epilogue, const GemvArgs& a) {
    if (prologue == PRO_NORM && epilogue == EPI_QKV) return launch_rows<WT, PRO_NORM, EPI_QKV>(ctx, a);
    if (prologue == PRO_NORM && epilogue == EPI_SWIGLU) return launch_rows<WT, PRO_NORM, EPI_SWIGLU>(ctx, a);
    if (prologue == PRO_NORM && epilogue == EPI_F32) return launch_rows<WT, PRO_NORM, EPI_F32>(ctx, a);
    if (prologue == PRO_COPY && epilogue == EPI_F32) return launch_rows<WT, PRO_COPY, EPI_F32>(ctx, a);
    if (prologue == PRO_COPY && epilogue == EPI_STORE) return launch_rows<WT, PRO_COPY, EPI_STORE>(ctx, a);
    return rlb_fail(RLB_ERR_INVALID, "gemv: unsupported prologue/epilogue pair %d/%d", prologue, epilogue);
}

}  // namespace

void gemv_set_tuning(int rows_per_warp, int ctas_per_sm, int) {
    g_tune.loaded = true;
    g_tune.rows_per_warp = rows_per_warp;
    g_tune.ctas_per_sm = ctas_per_sm;
}

int launch_gemv(rlb_ctx* ctx, rlb_dtype dtype, int prologue, int epilogue, const GemvArgs& a) {
    const int vec = dtype == RLB_F16 ? 8 : 4;
    if (a.K <= 0 || a.rows <= 0 || a.K % vec != 0 || a.ldw % vec != 0 || (prologue == PRO_NORM && a.K % 4 != 0))
        return rlb_fail(RLB_ERR_INVALID, "gemv: rows %d, K %d, ldw %lld are not supported (K and the row stride must be multiples of %d)",
                        a.rows, a.K, (long long)a.ldw, vec);
    return dtype == RLB_F16 ? launch_typed<__half>(ctx, prologue, epilogue, a) : launch_typed<float>(ctx, prologue, epilogue, a);
}

// Multi-row contraction C[n][M] = A[n][K] * W[M][K]^T: Tensor::matrix_mul_transposed with
// more than one row on both sides (src/tensor.rs:999-1025, :1250-1668; OpenCL kernel
// matrix_mul_transposed_f16, src/tensor_opencl_support.rs:512-557).
//
// This file holds the exact-f32 tile kernel: operands are widened to f32, multiplied and
// accumulated in f32 (FMA), which is the reference's arithmetic up to summation order. It
// serves f32 weights (where tensor-core formats would lose the 1e-4 parity bound) and is the
// fallback shape-generic path for f16.
#include "internal.h"

#include <cstdlib>

namespace {

// The tensor-core kernel takes f16 GEMMs with at least this many rows on the token side.
constexpr int kTcMinRows = 16;
bool tc_enabled() {
    static const bool on = getenv("RLB_GEMM_TC") == nullptr || atoi(getenv("RLB_GEMM_TC")) != 0;
    return on;
}


constexpr int BM = 64;  // rows of A per CTA
constexpr int BN = 64;  // rows of W per CTA
constexpr int BK = 16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <typename T> __device__ __forceinline__ T cast_to(float v);
template <> __device__ __forceinline__ __half cast_to<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast_to<float>(float v) { return v; }

template <typename T, typename OT, bool ROUND>
__global__ void __launch_bounds__(256) gemm_nt_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W, int64_t ldw,
                                                      OT* __restrict__ C, int64_t ldc, int n, int M, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int i0 = blockIdx.y * BM, j0 = blockIdx.x * BN;
    const int ty = tid / 16, tx = tid % 16;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int gi = i0 + r, gj = j0 + r, gk = k0 + kk;
            As[kk][r] = (gi < n && gk < K) ? to_f32<T>(A[(int64_t)gi * lda + gk]) : 0.f;
            Ws[kk][r] = (gj < M && gk < K) ? to_f32<T>(W[(int64_t)gj * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float av[4], wv[4];
#pragma unroll
            for (int a = 0; a < 4; a++) av[a] = As[kk][ty * 4 + a];
#pragma unroll
            for (int b = 0; b < 4; b++) wv[b] = Ws[kk][tx * 4 + b];
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int b = 0; b < 4; b++) acc[a][b] = fmaf(av[a], wv[b], acc[a][b]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int gi = i0 + ty * 4 + a, gj = j0 + tx * 4 + b;
            if (gi < n && gj < M) {
                float v = acc[a][b];
                if (ROUND) v = __half2float(__float2half_rn(v));
                C[(int64_t)gi * ldc + gj] = cast_to<OT>(v);
            }
        }
}

}  // namespace

int launch_gemm_nt(rlb_ctx* ctx, rlb_dtype dtype, const void* A, int64_t lda, const void* W, int64_t ldw, float* C, int64_t ldc, int n,
                   int M, int K, int round_out, int* err, int w_f16_exact) {
    if (dtype == RLB_F16 && tc_enabled() && n >= kTcMinRows && gemm_tc_supported(A, lda, W, ldw, n, M, K))
        return launch_gemm_tc_f32out(ctx, A, lda, W, ldw, C, ldc, n, M, K, round_out, err ? err : ctx->d_err);
    static const bool tf32x2 = getenv("RLB_GEMM_TF32X2") == nullptr || atoi(getenv("RLB_GEMM_TF32X2")) != 0;
    if (dtype == RLB_F32 && w_f16_exact && !round_out && tf32x2 && tc_enabled() && n >= kTcMinRows &&
        gemm_tc_f32_supported(A, lda, W, ldw, n, M, K))
        return launch_gemm_tc_f32w(ctx, A, lda, W, ldw, C, ldc, n, M, K, err ? err : ctx->d_err);
    dim3 grid((M + BN - 1) / BN, (n + BM - 1) / BM);
    if (grid.y > 65535) return rlb_fail(RLB_ERR_LIMIT, "gemm: too many rows (%d)", n);
    if (dtype == RLB_F16) {
        if (round_out) gemm_nt_kernel<__half, float, true><<<grid, 256, 0, ctx->stream>>>((const __half*)A, lda, (const __half*)W, ldw, C, ldc, n, M, K);
        else gemm_nt_kernel<__half, float, false><<<grid, 256, 0, ctx->stream>>>((const __half*)A, lda, (const __half*)W, ldw, C, ldc, n, M, K);
    } else {
        gemm_nt_kernel<float, float, false><<<grid, 256, 0, ctx->stream>>>((const float*)A, lda, (const float*)W, ldw, C, ldc, n, M, K);
    }
    RLB_LAUNCH_CHECK();
    count_launch(ctx);
    return RLB_OK;
}

int launch_gemm_nt_typed(rlb_ctx* ctx, rlb_dtype dtype, const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                         int n, int M, int K) {
    if (dtype == RLB_F16 && tc_enabled() && n >= kTcMinRows && gemm_tc_supported(A, lda, W, ldw, n, M, K))
        return launch_gemm_tc_f16out(ctx, A, lda, W, ldw, C, ldc, n, M, K, ctx->d_err);
    dim3 grid((M + BN - 1) / BN, (n + BM - 1) / BM);
    if (grid.y > 65535) return rlb_fail(RLB_ERR_LIMIT, "gemm: too many rows (%d)", n);
    if (dtype == RLB_F16)
        gemm_nt_kernel<__half, __half, false><<<grid, 256, 0, ctx->stream>>>((const __half*)A, lda, (const __half*)W, ldw, (__half*)C, ldc, n, M, K);
    else
        gemm_nt_kernel<float, float, false><<<grid, 256, 0, ctx->stream>>>((const float*)A, lda, (const float*)W, ldw, (float*)C, ldc, n, M, K);
    RLB_LAUNCH_CHECK();
    count_launch(ctx);
    return RLB_OK;
}

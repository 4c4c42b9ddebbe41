// Prefill contraction on the 5th-generation tensor cores: C[n][M] = X[n][K] * W[M][K]^T for f16
// operands with f32 accumulation -- rllama's batched Tensor::matrix_mul_transposed
// (src/tensor.rs:999-1025, f16 branch :1476-1666; OpenCL kernel matrix_mul_transposed_f16,
// src/tensor_opencl_support.rs:512-557), the only dense contraction on the path.
//
// One CTA computes a 128 (weight rows) x BN (tokens) tile:
//  * operands arrive by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill outside the
//    tensor) into a shared-memory ring of 4 to 8 stages (192 KB); one thread issues the loads;
//  * when the output has few tiles (short prompts, wo / w2) K is split over blockIdx.z and a
//    second kernel adds the partial tiles in a fixed order;
//  * one thread issues tcgen05.mma (kind::f16, M 128, N BN, K 16 per instruction, four per
//    64-column stage) with the accumulator in tensor memory; tcgen05.commit releases a ring
//    slot when the MMAs that read it have finished;
//  * four warps read the accumulator back with tcgen05.ld (each warp owns 32 TMEM lanes = 32
//    weight rows), round to f16 where the reference rounds the GEMM result, and store
//    token-major so that a warp writes 128 contiguous bytes per token.
// Products of f16 values are exact in f32; only the summation order differs from the
// reference's 8-lane FMA scheme.
//
// Every mbarrier wait is bounded; on a timeout the kernel raises the error word and still
// releases its tensor memory before returning.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "internal.h"

namespace {

constexpr int BM = 128;       // weight rows per tile (MMA M)
constexpr int BK = 64;        // K columns per stage: 128 bytes of f16 = one swizzle span
constexpr int kMaxStages = 8;
constexpr int kRingBytes = 192 * 1024;  // shared memory given to the operand ring
// stages that fit the ring for a token tile of BN rows (a weight tile is always 128 x 64 f16)
constexpr int stages_for(int bn) { return (kRingBytes / (BM * BK * 2 + bn * BK * 2)) < kMaxStages ? (kRingBytes / (BM * BK * 2 + bn * BK * 2)) : kMaxStages; }
constexpr int kTcThreads = 192;  // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait; false when it ran out (the error word is raised).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* dead, int* err) {
    for (uint32_t i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *dead) return false;
    }
    *dead = 1;
    *reinterpret_cast<volatile int*>(err) = 3;  // plain store: the word may live in mapped host memory
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(dst)),
                 "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
                 : "memory");
}
// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
    d |= (uint64_t)1 << 16;                         // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset
    d |= (uint64_t)1 << 46;                         // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                         // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <typename OT> __device__ __forceinline__ OT out_cast(float v);
template <> __device__ __forceinline__ float out_cast<float>(float v) { return v; }
template <> __device__ __forceinline__ __half out_cast<__half>(float v) { return __float2half_rn(v); }

// blockIdx.z selects a K range (split-K): with more than one split every split stores its f32
// partial tile into its own [n][ldc] slab of C (slab stride `split_stride` elements) and a second
// kernel adds the slabs in a fixed order, so the result does not depend on timing.
//
// TF32 = true is the f32 form for weights whose values are f16-representable (what the checkpoint
// loader produces): operands are 32-bit, kind::tf32, 32 K columns (still 128 bytes) per stage. A weight
// with at most 11 significant bits is exact in TF32; the activations are not, so the caller passes them
// split into x = hi + lo (hi = x rounded to TF32, lo = x - hi) and every k-block is multiplied twice,
// W x hi and W x lo, into the same accumulator: all products are exact in f32 and what is dropped of lo is
// below 2^-21 of x.
template <int BN, typename OT, bool TF32>
__global__ void __launch_bounds__(kTcThreads) gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                             const __grid_constant__ CUtensorMap tm_x,
                                                             const __grid_constant__ CUtensorMap tm_x2, OT* __restrict__ C, int64_t ldc,
                                                             int n, int Mrows, int K, int round_out, int64_t split_stride, int* err) {
    constexpr int kStages = stages_for(BN);
    constexpr int BKE = TF32 ? BK / 2 : BK;   // K columns of a stage (128 bytes either way)
    constexpr int PASSES = TF32 ? 2 : 1;
    constexpr uint32_t A_BYTES = BM * BK * 2;
    constexpr uint32_t B_BYTES = BN * BK * 2;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;  // power of two >= 32

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int dead_flag;
    volatile int* dead = &dead_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BM;  // first weight row of the tile
    const int n0 = blockIdx.y * BN;  // first token of the tile
    const int nkb_total = (K + BKE - 1) / BKE;
    const int per_split = (nkb_total + (int)gridDim.z - 1) / (int)gridDim.z;
    const int kb_first = (int)blockIdx.z * per_split;
    const int nkb = max(0, min(nkb_total, kb_first + per_split) - kb_first);  // k-blocks of this split
    C += (int64_t)blockIdx.z * split_stride;

    if (threadIdx.x == 0) {
        dead_flag = 0;
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // one warp allocates the accumulator's tensor memory
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        for (int it = 0; it < nkb * PASSES; it++) {
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            const int kb = it / PASSES;
            if (!mbar_wait(&empty_bar[s], ph ^ 1u, dead, err)) break;
            unsigned char* a_s = tiles + (size_t)s * STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            tma_load_2d(a_s, &tm_w, (kb_first + kb) * BKE, m0, &full_bar[s]);  // (second pass: the same tile again, from L2)
            tma_load_2d(a_s + A_BYTES, (PASSES == 2 && (it & 1)) ? &tm_x2 : &tm_x, (kb_first + kb) * BKE, n0, &full_bar[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        // instruction descriptor: f32 accumulator, f16 A and B, both K-major, N = BN, M = 128
        // (operand format field: 0 = f16, 2 = tf32, for A at bit 7 and B at bit 10)
        const uint32_t idesc = (1u << 4) | (TF32 ? ((2u << 7) | (2u << 10)) : 0u) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        bool ok = true;
        for (int kb = 0; kb < nkb * PASSES && ok; kb++) {
            const int s = kb % kStages;
            const uint32_t ph = (kb / kStages) & 1u;
            ok = mbar_wait(&full_bar[s], ph, dead, err);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
            const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / 16; k++) {
                // one instruction covers 32 bytes of K (16 f16 or 8 tf32 columns) along the swizzled row
                if (TF32) umma_tf32(tmem_base, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
                else umma_f16(tmem_base, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[s]);  // the slot is free once these MMAs have read it
        }
        umma_commit(&done_bar);
    }

    // ---------------- epilogue: warps 2..5, one TMEM lane quarter each ----------------
    if (warp >= 2) {
        const bool ok = mbar_wait(&done_bar, 0, dead, err);
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int q = warp & 3;
        const int row = m0 + q * 32 + lane;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                      "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int token = n0 + c0 + j;
                    if (token < n && row < Mrows) {
                        float v = nkb > 0 ? __uint_as_float(r[j]) : 0.f;
                        if (round_out) v = __half2float(__float2half_rn(v));
                        C[(int64_t)token * ldc + row] = out_cast<OT>(v);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Second pass of split-K: out[i][j] = cast(round?(sum over slabs in slab order)).
template <typename OT>
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int64_t slab_stride, int splits, int64_t ld_part, OT* __restrict__ out,
                                     int64_t ldc, int n, int M, int round_out) {
    const int64_t total = (int64_t)n * M;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / M, c = i - r * M;
        float v = 0.f;
        for (int z = 0; z < splits; z++) v += part[z * slab_stride + r * ld_part + c];
        if (round_out) v = __half2float(__float2half_rn(v));
        out[r * ldc + c] = out_cast<OT>(v);
    }
}

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int load_encode() {
    if (g_encode) return RLB_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
        return rlb_fail(RLB_ERR_CUDA, "cuTensorMapEncodeTiled is not available: %s", cudaGetErrorString(e));
    g_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    return RLB_OK;
}

// Row-major [rows][K] (f16, or f32 when `f32`) with row stride ld elements; box = 128 bytes of columns x
// box_rows rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int64_t ld, int box_rows, bool f32 = false) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (f32 ? 4 : 2)};
    cuuint32_t box[2] = {(cuuint32_t)(f32 ? BK / 2 : BK), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return rlb_fail(RLB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return RLB_OK;
}

// Few output tiles: split K so that most SMs stream weights.
int pick_splits(const rlb_ctx* ctx, int tiles, int nkb) {
    int splits = 1;
    if (tiles * 5 < ctx->sm_count * 3) {
        splits = (ctx->sm_count + tiles - 1) / tiles;
        if (splits > 8) splits = 8;
        while (splits > 1 && nkb / splits < 8) splits--;
    }
    return splits;
}

// scratch_off: bytes of the context's GEMM scratch the caller already uses (the split activations).
template <int BN, typename OT, bool TF32>
int launch_bn(rlb_ctx* ctx, const CUtensorMap& tw, const CUtensorMap& tx, const CUtensorMap& tx2, OT* C, int64_t ldc, int n, int M, int K,
              int round_out, int* err, size_t scratch_off) {
    const size_t smem = (size_t)stages_for(BN) * (BM * BK * 2 + BN * BK * 2) + 1024;
    dim3 grid((M + BM - 1) / BM, (n + BN - 1) / BN, 1);
    const int splits = pick_splits(ctx, (int)(grid.x * grid.y), (K + BK - 1) / BK * (TF32 ? 2 : 1));
    if (splits == 1) {
        auto kern = gemm_tc_kernel<BN, OT, TF32>;
        static std::atomic<uint64_t> set{0};
        if (!attr_done(set, ctx->device)) {
            RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_mark(set, ctx->device);
        }
        kern<<<grid, kTcThreads, smem, ctx->stream>>>(tw, tx, tx2, C, ldc, n, M, K, round_out, 0, err);
        RLB_LAUNCH_CHECK();
        count_launch(ctx);
        return RLB_OK;
    }
    // slabs of f32 partial tiles in the context's scratch
    const size_t need = scratch_off + (size_t)splits * n * M * sizeof(float);
    if (need > ctx->gemm_scratch_bytes) return rlb_fail(RLB_ERR_STATE, "gemm: scratch of %zu bytes was not reserved", need);
    float* part = reinterpret_cast<float*>(static_cast<char*>(ctx->gemm_scratch) + scratch_off);
    auto kern = gemm_tc_kernel<BN, float, TF32>;
    static std::atomic<uint64_t> set{0};
    if (!attr_done(set, ctx->device)) {
        RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_mark(set, ctx->device);
    }
    grid.z = splits;
    kern<<<grid, kTcThreads, smem, ctx->stream>>>(tw, tx, tx2, part, (int64_t)M, n, M, K, 0, (int64_t)n * M, err);
    RLB_LAUNCH_CHECK();
    count_launch(ctx);
    const int64_t total = (int64_t)n * M;
    int rg = (int)((total + 255) / 256);
    if (rg > ctx->sm_count * 8) rg = ctx->sm_count * 8;
    splitk_reduce_kernel<OT><<<rg, 256, 0, ctx->stream>>>(part, (int64_t)n * M, splits, (int64_t)M, C, ldc, n, M, round_out);
    RLB_LAUNCH_CHECK();
    count_launch(ctx);
    return RLB_OK;
}

// Grows the context's GEMM scratch (split activations + split-K slabs) to at least `need` bytes.
int reserve_scratch(rlb_ctx* ctx, size_t need) {
    if (need <= ctx->gemm_scratch_bytes) return RLB_OK;
    RLB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->gemm_scratch) cudaFree(ctx->gemm_scratch);
    ctx->gemm_scratch = nullptr;
    ctx->gemm_scratch_bytes = 0;
    cudaError_t e = cudaMalloc(&ctx->gemm_scratch, need);
    if (e != cudaSuccess) return rlb_fail(RLB_ERR_OOM, "GEMM scratch (%zu bytes): %s", need, cudaGetErrorString(e));
    ctx->gemm_scratch_bytes = need;
    return RLB_OK;
}

// hi = x rounded to TF32 (10 explicit mantissa bits), lo = x - hi (exact in f32)
__global__ void tf32_split_kernel(const float* __restrict__ x, int64_t ldx, int n, int K, float* __restrict__ hi, float* __restrict__ lo) {
    const int64_t total = (int64_t)n * K;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / K, c = i - r * K;
        const float v = x[r * ldx + c];
        uint32_t h;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
        const float hv = __uint_as_float(h);
        hi[i] = hv;
        lo[i] = v - hv;
    }
}

template <typename OT, bool TF32>
int launch_tc(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, OT* C, int64_t ldc, int n, int M, int K, int round_out,
              int* err) {
    RLB_TRY(load_encode());
    const int bn = n > 128 ? 256 : n > 64 ? 128 : n > 32 ? 64 : 32;
    // scratch: [x hi | x lo] for the f32 form, then the split-K slabs (if any)
    const size_t xs = TF32 ? (((size_t)n * K * sizeof(float) + 255) & ~(size_t)255) : 0;
    const int splits = pick_splits(ctx, ((M + BM - 1) / BM) * ((n + bn - 1) / bn), (K + BK - 1) / BK * (TF32 ? 2 : 1));
    RLB_TRY(reserve_scratch(ctx, 2 * xs + (splits > 1 ? (size_t)splits * n * M * sizeof(float) : 0)));
    CUtensorMap tw, tx, tx2;
    RLB_TRY(make_map(&tw, W, M, K, ldw, BM, TF32));
    if (TF32) {
        float* hi = static_cast<float*>(ctx->gemm_scratch);
        float* lo = reinterpret_cast<float*>(static_cast<char*>(ctx->gemm_scratch) + xs);
        const int64_t total = (int64_t)n * K;
        int g = (int)((total + 255) / 256);
        if (g > ctx->sm_count * 16) g = ctx->sm_count * 16;
        tf32_split_kernel<<<g, 256, 0, ctx->stream>>>(static_cast<const float*>(X), ldx, n, K, hi, lo);
        RLB_LAUNCH_CHECK();
        count_launch(ctx);
        RLB_TRY(make_map(&tx, hi, n, K, K, bn, true));
        RLB_TRY(make_map(&tx2, lo, n, K, K, bn, true));
    } else {
        RLB_TRY(make_map(&tx, X, n, K, ldx, bn));
        tx2 = tx;
    }
    switch (bn) {
        case 256: return launch_bn<256, OT, TF32>(ctx, tw, tx, tx2, C, ldc, n, M, K, round_out, err, 2 * xs);
        case 128: return launch_bn<128, OT, TF32>(ctx, tw, tx, tx2, C, ldc, n, M, K, round_out, err, 2 * xs);
        case 64: return launch_bn<64, OT, TF32>(ctx, tw, tx, tx2, C, ldc, n, M, K, round_out, err, 2 * xs);
        default: return launch_bn<32, OT, TF32>(ctx, tw, tx, tx2, C, ldc, n, M, K, round_out, err, 2 * xs);
    }
}

}  // namespace

// True when the tensor-core kernel takes these operands: 16-byte aligned bases and row strides.
bool gemm_tc_supported(const void* X, int64_t ldx, const void* W, int64_t ldw, int n, int M, int K) {
    if (n < 1 || M < 1 || K < 8) return false;
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return false;
    if ((ldx * 2) % 16 != 0 || (ldw * 2) % 16 != 0) return false;
    return true;
}

int launch_gemm_tc_f32out(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, float* C, int64_t ldc, int n, int M, int K,
                          int round_out, int* err) {
    return launch_tc<float, false>(ctx, X, ldx, W, ldw, C, ldc, n, M, K, round_out, err);
}

int launch_gemm_tc_f16out(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, void* C, int64_t ldc, int n, int M, int K,
                          int* err) {
    return launch_tc<__half, false>(ctx, X, ldx, W, ldw, reinterpret_cast<__half*>(C), ldc, n, M, K, 0, err);
}

// f32 operands, weights known to hold f16-representable values: two TF32 passes (see the kernel).
bool gemm_tc_f32_supported(const void* X, int64_t ldx, const void* W, int64_t ldw, int n, int M, int K) {
    if (n < 1 || M < 1 || K < 8 || K % 4 != 0) return false;
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return false;
    if ((ldx * 4) % 16 != 0 || (ldw * 4) % 16 != 0) return false;
    return true;
}

int launch_gemm_tc_f32w(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, float* C, int64_t ldc, int n, int M, int K,
                        int* err) {
    return launch_tc<float, true>(ctx, X, ldx, W, ldw, C, ldc, n, M, K, 0, err);
}

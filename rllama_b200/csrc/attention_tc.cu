// Causal attention of a multi-token call on the tensor cores, for f16 caches and head_dim 64 / 128:
// the two dense per-head contractions of Attention::forward -- scores = q K^T / sqrt(head_dim)
// (Tensor::matrix_mul, src/tensor.rs:979-997, :1050-1115) and out = softmax(scores + mask) V
// (matrix_mul_transposed on the values, src/transformer.rs:768-779) -- with the causal mask of
// Tensor::full_triu (src/tensor.rs:496-508) as a predicate and the softmax (src/tensor.rs:479-494)
// evaluated online with the row maximum subtracted.
//
// No rounding point is added. K and V are f16 in the cache, so they are exact tensor-core inputs.
// q (f32 after RoPE) and the softmax weights p (f32) are not: each is split into two f16 halves,
// x = hi + lo with hi = f16(x) and lo = f16(x - hi), and both halves are multiplied into the same
// f32 accumulator (tcgen05.mma kind::f16; products of f16 values are exact in f32). Two halves carry
// 22 significant bits; what is dropped is below 2^-22 of x, or below 2^-25 in absolute terms where
// the low half falls into f16's subnormal range. p carries a factor 2^14 (it lies in [0, 1]; the factor is
// folded into the exponent of 2^(s - m) and cancels in o / l at the end) so that its low half stays a
// normal number down to p = 2^-17. The exponential is ex2.approx (relative error below 2^-22) on scores
// pre-multiplied by log2(e).
//
// One CTA owns 128 query rows of one head and walks the cache in tiles of 128 positions:
//  * one thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the K and V tiles
//    straight from the cache: K as the K-major B operand of the score product, V (position-major,
//    i.e. contraction index outermost) as the MN-major B operand of the output product;
//  * one thread issues the MMAs: S = Qhi K^T + Qlo K^T into one of two score buffers in tensor
//    memory (the next tile's scores are computed while the softmax of the current one runs), then
//    O_tile = Phi V + Plo V into a third buffer;
//  * eight warps do the softmax: a thread owns half a row (64 score columns, 64 output columns),
//    reads its scores with tcgen05.ld, keeps the running maximum, sum and output in registers,
//    writes the split weights to shared memory as the A operand of the output product and adds
//    the previous tile's O_tile (rescaled) to its output row.
// Every wait is bounded; when one runs out the kernel raises the error word, no later wait of the CTA
// blocks any more (the softmax warps still run their loop to its end so that every thread keeps meeting
// their named barrier), and the tensor memory is released before the CTA returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cfloat>
#include <cstdlib>

#include "internal.h"

namespace {

constexpr int QB = 128;           // query rows per CTA (MMA M)
constexpr int TK = 128;           // cache positions per tile
constexpr int kSoftmaxWarps = 8;
constexpr int kThreadsTc = (kSoftmaxWarps + 2) * 32;  // + TMA warp + MMA warp
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr float kPShift = 14.f;     // the softmax weights carry a factor 2^14 (see the file comment)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Bounded wait; false when it ran out or the CTA already gave up (the error word is raised once).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* dead, int* err) {
    for (uint32_t i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && *dead) return false;
    }
    *dead = 1;
    *reinterpret_cast<volatile int*>(err) = 3;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(dst)),
                 "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
                 : "memory");
}
// Shared-memory operand descriptors, 128-byte swizzle, 8-row groups 1024 bytes apart.
// K-major: a row of the operand (one M or N index) is 128 contiguous bytes of the contraction index.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;               // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;     // stride byte offset: next group of 8 rows
    d |= (uint64_t)1 << 46;               // descriptor version
    d |= (uint64_t)2 << 61;               // 128-byte swizzle
    return d;
}
// MN-major: a 128-byte row holds 64 consecutive M / N indices of ONE contraction index; 8 contraction
// indices form a 1024-byte group, the next group follows at the stride offset, and the next 64
// M / N indices start `lead_bytes` further on.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lead_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lead_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void softmax_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxWarps * 32) : "memory"); }

// x = hi + lo in f16 halves, eight values packed for one 16-byte shared-memory store each (packed conversions:
// two values per instruction).
__device__ __forceinline__ void split8(const float (&x)[8], uint4& hi, uint4& lo) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2 hh = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
        const float2 hf = __half22float2(hh);
        const __half2 ll = __floats2half2_rn(x[2 * i] - hf.x, x[2 * i + 1] - hf.y);
        h[i] = *reinterpret_cast<const uint32_t*>(&hh);
        l[i] = *reinterpret_cast<const uint32_t*>(&ll);
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}

struct AttnTcArgs {
    const float* q;     // n rows, row stride q_ld
    int64_t q_ld;
    __half* out;        // [n][heads * HD]
    int n, start_pos, heads, max_seq;
    int* err;
};

// Shared memory (1024-byte aligned blocks, all with the 128-byte swizzle of their operand role):
//   Qhi, Qlo  : [HD/64][128 rows][64]   A of the score product
//   K         : [HD/64][TK rows][64]    B of the score product (TMA)
//   V         : [HD/64][TK rows][64]    B of the output product, MN-major (TMA)
//   Phi, Plo  : [TK/64][128 rows][64]   A of the output product
template <int HD>
__global__ void __launch_bounds__(kThreadsTc, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                                       const __grid_constant__ CUtensorMap tm_v, const AttnTcArgs a) {
    constexpr int NB = HD / 64;                      // 64-column blocks of the head dimension
    constexpr uint32_t Q_BYTES = QB * HD * 2;        // one half (hi or lo)
    constexpr uint32_t KV_BYTES = TK * HD * 2;
    constexpr uint32_t P_BYTES = QB * TK * 2;        // one half
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t S_COL0 = 0, S_COL1 = TK, O_COL = 2 * TK;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_hi = base;
    unsigned char* q_lo = q_hi + Q_BYTES;
    unsigned char* k_s = q_lo + Q_BYTES;
    unsigned char* v_s = k_s + KV_BYTES;
    unsigned char* p_hi = v_s + KV_BYTES;
    unsigned char* p_lo = p_hi + P_BYTES;
    __shared__ __align__(8) uint64_t k_full, k_empty, v_full, v_empty, s_full[2], s_free[2], p_ready, pv_done;
    __shared__ uint32_t tmem_slot;
    __shared__ int dead_flag;
    __shared__ float xmax[2][2][QB];   // [tile parity][column half][row]: the halves' tile maxima
    __shared__ float xsum[2][QB];
    volatile int* dead = &dead_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x;
    const int qblock = (int)gridDim.y - 1 - (int)blockIdx.y;   // the longest rows first
    const int i0 = qblock * QB;
    const int rows = min(QB, a.n - i0);
    const int t_end = a.start_pos + i0 + rows;                  // positions the block's last row attends to
    const int n_tiles = (t_end + TK - 1) / TK;
    const int cache_row0 = head * a.max_seq;

    if (threadIdx.x == 0) {
        dead_flag = 0;
        mbar_init(&k_full, 1); mbar_init(&k_empty, 1); mbar_init(&v_full, 1); mbar_init(&v_empty, 1);
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(&s_free[0], kSoftmaxWarps); mbar_init(&s_free[1], kSoftmaxWarps);
        mbar_init(&p_ready, kSoftmaxWarps); mbar_init(&pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kSoftmaxWarps) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the set-up above overlaps the previous kernel's tail; q and the cache rows are its outputs
    rlb_pdl_trigger();
    rlb_pdl_wait();
    // the query block, split into halves, in the A-operand layout: row r, 16-byte chunk c of a 64-column
    // block lands at r * 128 + ((c ^ (r & 7)) * 16)
    if (warp < kSoftmaxWarps) {
        const int r = threadIdx.x >> 1, half = threadIdx.x & 1;   // two threads per row, HD / 2 columns each
        const float* src = a.q + (int64_t)(i0 + r) * a.q_ld + head * HD + half * (HD / 2);
#pragma unroll
        for (int c8 = 0; c8 < HD / 16; c8++) {
            float x[8];
            if (r < rows) {
                const float4 v0 = *reinterpret_cast<const float4*>(src + c8 * 8), v1 = *reinterpret_cast<const float4*>(src + c8 * 8 + 4);
                x[0] = v0.x; x[1] = v0.y; x[2] = v0.z; x[3] = v0.w; x[4] = v1.x; x[5] = v1.y; x[6] = v1.z; x[7] = v1.w;
            } else {
#pragma unroll
                for (int e = 0; e < 8; e++) x[e] = 0.f;
            }
            uint4 hi, lo;
            split8(x, hi, lo);
            const int col = half * (HD / 2) + c8 * 8;             // first column of this chunk
            const int blk = col >> 6, chunk = (col & 63) >> 3;
            const uint32_t off = (uint32_t)blk * (QB * 128) + (uint32_t)r * 128 + (uint32_t)((chunk ^ (r & 7)) << 4);
            *reinterpret_cast<uint4*>(q_hi + off) = hi;
            *reinterpret_cast<uint4*>(q_lo + off) = lo;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the MMA reads these through the async proxy
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    if (warp == kSoftmaxWarps) {
        // ---------------------------------- TMA producer ------------------------------------
        if (lane == 0) {
            for (int j = 0; j < n_tiles; j++) {
                const uint32_t ph = (uint32_t)j & 1u;
                if (!mbar_wait(&k_empty, ph ^ 1u, dead, a.err)) break;
                mbar_expect_tx(&k_full, KV_BYTES);
#pragma unroll
                for (int b = 0; b < NB; b++) tma_load_2d(k_s + b * (TK * 128), &tm_k, b * 64, cache_row0 + j * TK, &k_full);
                if (!mbar_wait(&v_empty, ph ^ 1u, dead, a.err)) break;
                mbar_expect_tx(&v_full, KV_BYTES);
#pragma unroll
                for (int b = 0; b < NB; b++) tma_load_2d(v_s + b * (TK * 128), &tm_v, b * 64, cache_row0 + j * TK, &v_full);
            }
        }
    } else if (warp == kSoftmaxWarps + 1) {
        // ---------------------------------- MMA issuer --------------------------------------
        if (lane == 0) {
            // f32 accumulator, f16 operands; scores: N = TK, both operands K-major; output: N = HD, B MN-major
            const uint32_t idesc_s = (1u << 4) | ((uint32_t)(TK >> 3) << 17) | ((uint32_t)(QB >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QB >> 4) << 24);
            const uint32_t qh = smem_u32(q_hi), ql = smem_u32(q_lo), ks = smem_u32(k_s), vs = smem_u32(v_s);
            const uint32_t ph_ = smem_u32(p_hi), pl_ = smem_u32(p_lo);
            auto issue_scores = [&](int j) -> bool {
                const uint32_t sb = (uint32_t)j & 1u;
                if (!mbar_wait(&k_full, (uint32_t)j & 1u, dead, a.err)) return false;
                if (j >= 2 && !mbar_wait(&s_free[sb], (uint32_t)((j >> 1) - 1) & 1u, dead, a.err)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_base + (sb ? S_COL1 : S_COL0);
                uint32_t acc = 0;
#pragma unroll
                for (int pass = 0; pass < 2; pass++)
#pragma unroll
                    for (int b = 0; b < NB; b++)
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            umma_f16(d, desc_kmajor((pass ? ql : qh) + b * (QB * 128) + k * 32), desc_kmajor(ks + b * (TK * 128) + k * 32),
                                     idesc_s, acc);
                            acc = 1;
                        }
                umma_commit(&k_empty);      // the K tile may be overwritten
                umma_commit(&s_full[sb]);   // the scores are complete
                return true;
            };
            bool ok = issue_scores(0);
            for (int j = 0; j < n_tiles && ok; j++) {
                if (j + 1 < n_tiles) ok = issue_scores(j + 1);
                if (!ok) break;
                if (!mbar_wait(&p_ready, (uint32_t)j & 1u, dead, a.err)) break;
                if (!mbar_wait(&v_full, (uint32_t)j & 1u, dead, a.err)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_base + O_COL;
                uint32_t acc = 0;
#pragma unroll
                for (int pass = 0; pass < 2; pass++)
#pragma unroll
                    for (int kb = 0; kb < TK / 16; kb++) {
                        // 16 positions per instruction: 32 bytes along a row of P, two 8-position groups of V
                        umma_f16(d, desc_kmajor((pass ? pl_ : ph_) + (kb >> 2) * (QB * 128) + (kb & 3) * 32),
                                 desc_mnmajor(vs + kb * 2048, TK * 128), idesc_o, acc);
                        acc = 1;
                    }
                umma_commit(&v_empty);
                umma_commit(&pv_done);
            }
        }
    } else {
        // ---------------------------------- softmax warps -----------------------------------
        const int quarter = warp & 3, half = warp >> 2;      // TMEM lane quarter, column half
        const int r = quarter * 32 + lane;                   // row of the query block
        const int limit = a.start_pos + i0 + r + 1;          // attends to positions below this (src/tensor.rs:496-508)
        // 1 / sqrt(head_dim) (src/transformer.rs:770) times log2(e): the softmax is evaluated with 2^x (ex2.approx, relative
        // error below 2^-22, the precision of the two-half split); softmax(s) = 2^(s c - m) / sum with c = log2(e)
        const float scale2 = (1.0f / sqrtf((float)HD)) * 1.4426950408889634f;
        constexpr int OC = HD / 2;                           // output columns of this thread
        float o[OC];
#pragma unroll
        for (int c = 0; c < OC; c++) o[c] = 0.f;
        float m_run = -FLT_MAX, l_run = 0.f, alpha_prev = 0.f;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        bool ok = true;
        // (after a wait that ran out the loop still runs to its end, without blocking: every thread must keep
        // meeting the named barrier below)
        for (int j = 0; j < n_tiles; j++) {
            const uint32_t sb = (uint32_t)j & 1u;
            ok = mbar_wait(&s_full[sb], (uint32_t)(j >> 1) & 1u, dead, a.err) && ok;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // 1. this thread's 64 scores of the tile
            float p[64];
            const uint32_t s_addr = tmem_base + lane_addr + (sb ? S_COL1 : S_COL0) + (uint32_t)half * 64;
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 32) {   // two loads of 16 columns in flight per wait
                uint32_t v[2][16];
                tmem_ld16(s_addr + c0, v[0]);
                tmem_ld16(s_addr + c0 + 16, v[1]);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 16; e++) { p[c0 + e] = __uint_as_float(v[0][e]); p[c0 + 16 + e] = __uint_as_float(v[1][e]); }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[sb]);   // the score buffer may be overwritten by tile j + 2
            const int t_first = j * TK + half * 64;
            float tmax = -FLT_MAX;
#pragma unroll
            for (int e = 0; e < 64; e++) {
                p[e] = (t_first + e < limit) ? p[e] * scale2 : -FLT_MAX;   // the causal mask; scores in units of log2(e)
                tmax = fmaxf(tmax, p[e]);
            }
            xmax[sb][half][r] = tmax;
            softmax_sync();
            const float m_new = fmaxf(m_run, fmaxf(tmax, xmax[sb][half ^ 1][r]));
            const float alpha = ex2_approx(m_run - m_new);
            // weights as 2^(s - m + 14): the factor 2^14 keeps the low f16 half normal and cancels in o / l at the end
            const float shift = kPShift - m_new;
            float psum = 0.f;
#pragma unroll
            for (int e = 0; e < 64; e++) {
                const float pv = (t_first + e < limit) ? ex2_approx(p[e] + shift) : 0.f;
                psum += pv;
                p[e] = pv;
            }
            l_run = l_run * alpha + psum;
            m_run = m_new;
            // 2. the previous tile's output product is complete: fold it into the running row, and the
            //    weight buffer is free again
            if (j > 0) {
                ok = mbar_wait(&pv_done, (uint32_t)(j - 1) & 1u, dead, a.err) && ok;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t o_addr = tmem_base + lane_addr + O_COL + (uint32_t)half * OC;
#pragma unroll
                for (int c0 = 0; c0 < OC; c0 += 32) {
                    uint32_t v[2][16];
                    tmem_ld16(o_addr + c0, v[0]);
                    tmem_ld16(o_addr + c0 + 16, v[1]);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; e++) {
                        o[c0 + e] = fmaf(o[c0 + e], alpha_prev, __uint_as_float(v[0][e]));
                        o[c0 + 16 + e] = fmaf(o[c0 + 16 + e], alpha_prev, __uint_as_float(v[1][e]));
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            alpha_prev = alpha;
            // 3. the split weights as the A operand of the output product
#pragma unroll
            for (int c8 = 0; c8 < 8; c8++) {
                float x[8];
#pragma unroll
                for (int e = 0; e < 8; e++) x[e] = p[c8 * 8 + e];
                uint4 hi, lo;
                split8(x, hi, lo);
                const uint32_t off = (uint32_t)half * (QB * 128) + (uint32_t)r * 128 + (uint32_t)((c8 ^ (r & 7)) << 4);
                *reinterpret_cast<uint4*>(p_hi + off) = hi;
                *reinterpret_cast<uint4*>(p_lo + off) = lo;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready);
        }
        if (ok && n_tiles > 0) {
            ok = mbar_wait(&pv_done, (uint32_t)(n_tiles - 1) & 1u, dead, a.err);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t o_addr = tmem_base + lane_addr + O_COL + (uint32_t)half * OC;
#pragma unroll
                for (int c0 = 0; c0 < OC; c0 += 32) {
                    uint32_t v[2][16];
                    tmem_ld16(o_addr + c0, v[0]);
                    tmem_ld16(o_addr + c0 + 16, v[1]);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 16; e++) {
                        o[c0 + e] = fmaf(o[c0 + e], alpha_prev, __uint_as_float(v[0][e]));
                        o[c0 + 16 + e] = fmaf(o[c0 + 16 + e], alpha_prev, __uint_as_float(v[1][e]));
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
        }
        // the row sum: both halves used the same maxima, so their partial sums simply add
        xsum[half][r] = l_run;
        softmax_sync();
        if (ok && r < rows) {
            const float inv = 1.0f / (xsum[0][r] + xsum[1][r]);  // (numerator and denominator both carry 2^14)
            __half* dst = a.out + (int64_t)(i0 + r) * a.heads * HD + head * HD + half * OC;
#pragma unroll
            for (int c8 = 0; c8 < OC / 8; c8++) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const __half h0 = __float2half_rn(o[c8 * 8 + 2 * e] * inv), h1 = __float2half_rn(o[c8 * 8 + 2 * e + 1] * inv);
                    w[e] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
                }
                *reinterpret_cast<uint4*>(dst + c8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kSoftmaxWarps) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

PFN_cuTensorMapEncodeTiled_v12000 g_encode_attn = nullptr;

int load_encode_attn() {
    if (g_encode_attn) return RLB_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
        return rlb_fail(RLB_ERR_CUDA, "cuTensorMapEncodeTiled is not available: %s", cudaGetErrorString(e));
    g_encode_attn = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    return RLB_OK;
}

// The cache of one layer as a 2-D tensor [heads * max_seq rows][hd] of f16; box = 64 columns x TK rows.
int cache_map(CUtensorMap* map, const void* cache, int heads, int max_seq, int hd) {
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)heads * (cuuint64_t)max_seq};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)TK};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode_attn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return rlb_fail(RLB_ERR_CUDA, "cuTensorMapEncodeTiled (KV cache) failed with code %d", (int)r);
    return RLB_OK;
}

template <int HD>
int launch_hd(rlb_ctx* ctx, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcArgs& args) {
    const size_t smem = 2 * (size_t)QB * HD * 2 + 2 * (size_t)TK * HD * 2 + 2 * (size_t)QB * TK * 2 + 1024;
    auto kern = attn_prefill_tc_kernel<HD>;
    static std::atomic<uint64_t> set{0};
    if (!attr_done(set, ctx->device)) {
        RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_mark(set, ctx->device);
    }
    dim3 grid(args.heads, (args.n + QB - 1) / QB);
    RLB_CUDA(rlb_launch(kern, grid, dim3(kThreadsTc), smem, ctx, mk, mv, args));
    count_launch(ctx);
    return RLB_OK;
}

}  // namespace

bool attn_prefill_tc_supported(rlb_dtype cache_dtype, const AttnPrefillArgs& a) {
    static const bool enabled = getenv("RLB_ATTN_TC") == nullptr || atoi(getenv("RLB_ATTN_TC")) != 0;
    if (!enabled || cache_dtype != RLB_F16) return false;
    if (a.hd != 64 && a.hd != 128) return false;
    if (a.n < 32 || a.q_ld % 4 != 0 || ((uintptr_t)a.q & 15)) return false;
    if (((uintptr_t)a.kcache & 15) || ((uintptr_t)a.vcache & 15) || ((uintptr_t)a.out & 15)) return false;
    return true;
}

int launch_attn_prefill_tc(rlb_ctx* ctx, const AttnPrefillArgs& a, int* err) {
    RLB_TRY(load_encode_attn());
    CUtensorMap mk, mv;
    RLB_TRY(cache_map(&mk, a.kcache, a.heads, a.max_seq, a.hd));
    RLB_TRY(cache_map(&mv, a.vcache, a.heads, a.max_seq, a.hd));
    AttnTcArgs args;
    args.q = a.q; args.q_ld = a.q_ld; args.out = reinterpret_cast<__half*>(a.out);
    args.n = a.n; args.start_pos = a.start_pos; args.heads = a.heads; args.max_seq = a.max_seq;
    args.err = err ? err : ctx->d_err;
    return a.hd == 128 ? launch_hd<128>(ctx, mk, mv, args) : launch_hd<64>(ctx, mk, mv, args);
}

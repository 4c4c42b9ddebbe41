// Prefill contraction on the 5th-generation tensor cores: C[n][M] = X[n][K] * W[M][K]^T for f16
// operands with f32 accumulation -- rllama's batched Tensor::matrix_mul_transposed
// (src/tensor.rs:999-1025, f16 branch :1476-1666; OpenCL kernel matrix_mul_transposed_f16,
// src/tensor_opencl_support.rs:512-557), the dense contraction of the projections.
//
// One persistent kernel, one CTA per SM. A tile is 128 tokens x TN weight rows (TN = 256; 128 for prompts of
// up to 128 tokens, where every tile is split over K and a narrower tile halves the partial results): the tokens are the
// MMA's M (tensor-memory lanes), the weight rows its N (tensor-memory columns), so a thread of the
// epilogue owns one token and reads consecutive weight rows -- consecutive addresses of the
// row-major output.
//  * Work is handed out per (tile, 64-column k-block). The first floor(tiles / CTAs) * CTAs tiles go
//    round-robin to the CTAs as whole tiles (neighbouring CTAs work on neighbouring tiles, so the
//    weight rows a group of token tiles shares are read from HBM once and then from L2); the k-blocks
//    of the remaining tiles are dealt out in equal contiguous runs over all CTAs, so every SM streams the
//    same number of bytes whatever the shape (short prompts, few tiles: this is a K split). A run that
//    does not cover a tile's whole K range leaves an f32 partial tile in scratch memory; a second kernel
//    adds the partial tiles of a tile in k order (fixed by the schedule, so results never depend on
//    timing) and applies the output rounding.
//  * Operands arrive by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill outside the tensor)
//    into a 192 KB shared-memory ring; one thread issues the loads and runs ahead across tiles.
//  * One thread issues tcgen05.mma (kind::f16, M 128, N TN, K 16 per instruction) into one of two
//    accumulators in tensor memory (2 x TN columns): the next tile's main loop runs while four warps
//    read the finished accumulator back with tcgen05.ld, round to f16 where the reference rounds the
//    GEMM result, and store 64 contiguous bytes per thread and step. Long prompts use 256-token tiles
//    (template parameter MT = 2, see the kernel): two MMAs per k-step on one weight tile.
//  * The kernel is a programmatic dependent of its predecessor: the weight tiles of the first ring
//    stages are requested before the wait for the previous kernel, the activation tiles after it.
// Products of f16 values are exact in f32; only the summation order differs from the reference's
// 8-lane FMA scheme.
//
// TF32 = true is the f32 form for weights whose values are f16-representable (what the checkpoint
// loader produces): operands are 32-bit, kind::tf32, 32 K columns (still 128 bytes) per stage. A weight
// with at most 11 significant bits is exact in TF32; the activations are not, so they are split into
// x = hi + lo (hi = x rounded to TF32, lo = x - hi), a stage carries both halves next to ONE copy of the
// weight tile, and every k-block is multiplied twice, hi W and lo W, into the same accumulator: all
// products are exact in f32 and what is dropped of lo is below 2^-21 of x.
//
// Every mbarrier wait is bounded; on a timeout the kernel raises the error word and still releases its
// tensor memory before returning.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>

#include "gemm_sched.h"
#include "round_f16.h"
#include "internal.h"

namespace {

constexpr int TM = gemm_sched::TM;   // tokens per MMA block (MMA M)
// (weight rows per tile, MMA N: template parameter TN, 256 or 128)
constexpr int BK = 64;        // K columns per stage in f16 (128 bytes = one swizzle span)
constexpr int kRingBytes = 192 * 1024;   // stage ring (224 KB gives the 128-row tiles a seventh stage and measured the same)
// threads: warp 0 TMA, warp 1 MMA, then four epilogue warps per 128-token block of a tile
constexpr int tc_threads(int mt) { return 64 + 128 * mt; }
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr uint32_t X_BYTES = TM * 128;   // one 128-token activation block of a stage
constexpr int kMaxGrid = 256;            // CTAs of the persistent kernel at most (one per SM)

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
// Bounded wait; false when it ran out (the error word is raised) or the CTA already gave up.
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
template <bool TF32>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if (TF32)
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

#ifdef RLB_GEMM_TRACE
// Timeline build (`python -m rllama_b200.build --trace`, a separate library): every CTA of the most recent GEMM launch
// leaves 16 words in g_trace, times in ns of %globaltimer: 0 entry, 1 set-up done, 2 producer past its dependency
// wait, 3 first operand stage landed, 4 last MMA committed, 5 MMA thread blocked on operand stages (total), 6 on a
// busy accumulator (total), 7 first accumulator handed to the epilogue, 8 epilogue done, 9 epilogue blocked (total),
// 10 k-blocks computed, 11 producer blocked on full ring (total), 12 producer done, 13 epilogue busy (total).
// `bench.py --gemm-trace` reads them through rlb_debug_gemm_trace.
__device__ unsigned long long g_trace[256 * 16];
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define RLB_TR(i, v) (g_trace[blockIdx.x * 16 + (i)] = (unsigned long long)(v))
#define RLB_NOW() trace_now()
#else
#define RLB_TR(i, v) ((void)0)
#define RLB_NOW() 0ull
#endif

using gemm_sched::Sched;
using gemm_sched::make_sched;
using gemm_sched::rest_begin;
using gemm_sched::Piece;
using gemm_sched::PieceIter;

template <typename OT> struct OutPack;
template <> struct OutPack<float> {
    static __device__ __forceinline__ void store16(float* dst, const float (&v)[16], bool vec, int valid_cols) {
        if (vec && valid_cols >= 16) {
#pragma unroll
            for (int j = 0; j < 4; j++) reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (j < valid_cols) dst[j] = v[j];
        }
    }
};
template <> struct OutPack<__half> {
    static __device__ __forceinline__ void store16(__half* dst, const float (&v)[16], bool vec, int valid_cols) {
        if (vec && valid_cols >= 16) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const __half2 hh = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&hh);
            }
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (j < valid_cols) dst[j] = __float2half_rn(v[j]);
        }
    }
};

// MT = 128-token blocks per tile (1 or 2). With MT = 2 a tile is 256 tokens x 256 weight rows: two MMAs per k-step share
// one weight tile (a third less shared-memory fill per flop, which is what bounds the kernel at long prompts); the two
// accumulators then take all 512 tensor-memory columns, so a tile's epilogue is not overlapped with the next main loop.
template <typename OT, bool TF32, int TN, int MT>
__global__ void __launch_bounds__(tc_threads(MT), 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_x,
                                                                const __grid_constant__ CUtensorMap tm_x2,
                                                                const __grid_constant__ CUtensorMap tm_w, OT* __restrict__ C, int64_t ldc,
                                                                int n, int Mrows, int K, int round_out, float* __restrict__ part, int* err) {
    constexpr int BKE = TF32 ? BK / 2 : BK;                      // K columns of a stage (128 bytes either way)
    constexpr int NX = TF32 ? 2 : 1;                             // activation tiles per stage (hi, lo)
    constexpr uint32_t W_BYTES = TN * 128;
    static_assert(MT == 1 || (!TF32 && TN == 256), "256-token tiles: f16, 256 weight rows");
    constexpr int TT = TM * MT;                                  // tokens per tile
    constexpr size_t kSlabFloats = (size_t)TT * TN;              // one partial tile
    constexpr uint32_t XS_BYTES = NX * MT * X_BYTES;             // activation part of a stage
    constexpr uint32_t STAGE_BYTES = XS_BYTES + W_BYTES;
    constexpr int kStages = kRingBytes / STAGE_BYTES;            // TN 256: 4 (f16), 3 (tf32, and f16 with MT 2); TN 128: 6, 4
    constexpr int NACC = MT == 1 ? 2 : 1;                        // accumulator sets in tensor memory
    constexpr uint32_t TMEM_COLS = 2 * TN;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int dead_flag;
    volatile int* dead = &dead_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) RLB_TR(0, RLB_NOW());
    const int nkb = (K + BKE - 1) / BKE;
    const Sched sched = make_sched(n, Mrows, nkb, (int)gridDim.x, TN, TT);

    if (threadIdx.x == 0) {
        dead_flag = 0;
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4 * MT);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // one warp allocates the accumulators' tensor memory
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) RLB_TR(1, RLB_NOW());
    rlb_pdl_trigger();
    if (!(warp == 0 && lane == 0)) rlb_pdl_wait();  // (the producer thread waits after its weight prefetch)

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer: runs ahead of the MMAs across pieces ----------------
        PieceIter it(sched, (int)blockIdx.x, (int)gridDim.x);
        Piece p;
        bool have = it.next(p);
        int kb = have ? p.kb0 : 0;
        auto advance = [&]() {
            if (++kb >= p.kb1) { have = it.next(p); kb = have ? p.kb0 : 0; }
        };
        // Weights do not depend on earlier kernels: the weight tiles of the first ring stages are requested BEFORE
        // the wait for the previous kernel (programmatic dependent launch), the activation tiles after it.
        int npre = 0, pre_kb[8], pre_mt[8];
        while (have && npre < kStages) {
            const int nt = p.tile / sched.n_mt, mt = p.tile - nt * sched.n_mt;
            unsigned char* st = tiles + (size_t)npre * STAGE_BYTES;
            mbar_expect_tx(&full_bar[npre], STAGE_BYTES);
            tma_load_2d(st + XS_BYTES, &tm_w, kb * BKE, nt * TN, &full_bar[npre]);
            pre_kb[npre] = kb; pre_mt[npre] = mt;
            npre++;
            advance();
        }
        rlb_pdl_wait();
        RLB_TR(2, RLB_NOW());
        unsigned long long tr_ring = 0;
        for (int i = 0; i < npre; i++) {
            unsigned char* st = tiles + (size_t)i * STAGE_BYTES;
            tma_load_2d(st, &tm_x, pre_kb[i] * BKE, pre_mt[i] * TT, &full_bar[i]);   // (one box of TT rows)
            if (TF32) tma_load_2d(st + X_BYTES, &tm_x2, pre_kb[i] * BKE, pre_mt[i] * TT, &full_bar[i]);
        }
        uint32_t cnt = (uint32_t)npre;
        while (have) {
            const int nt = p.tile / sched.n_mt, mt = p.tile - nt * sched.n_mt;
            const uint32_t s = cnt % kStages, ph = (cnt / kStages) & 1u;
            const unsigned long long tr_a = RLB_NOW();
            if (!mbar_wait(&empty_bar[s], ph ^ 1u, dead, err)) break;
            tr_ring += RLB_NOW() - tr_a;
            unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            tma_load_2d(st, &tm_x, kb * BKE, mt * TT, &full_bar[s]);
            if (TF32) tma_load_2d(st + X_BYTES, &tm_x2, kb * BKE, mt * TT, &full_bar[s]);
            tma_load_2d(st + XS_BYTES, &tm_w, kb * BKE, nt * TN, &full_bar[s]);
            cnt++;
            advance();
        }
        RLB_TR(11, tr_ring);
        RLB_TR(12, RLB_NOW());
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        // instruction descriptor: f32 accumulator, A and B both K-major, N = TN, M = TM
        // (operand format field: 0 = f16, 2 = tf32, for A at bit 7 and B at bit 10)
        const uint32_t idesc = (1u << 4) | (TF32 ? ((2u << 7) | (2u << 10)) : 0u) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
        PieceIter it(sched, (int)blockIdx.x, (int)gridDim.x);
        Piece p;
        uint32_t cnt = 0, piece = 0;
        bool ok = true;
        unsigned long long tr_starved = 0, tr_acc = 0, tr_first = 0;
        while (ok && it.next(p)) {
            const uint32_t b = NACC == 2 ? (piece & 1u) : 0u;
            const uint32_t use = NACC == 2 ? (piece >> 1) : piece;  // how often this accumulator set has been used before
            const unsigned long long tr_a = RLB_NOW();
            ok = mbar_wait(&acc_empty[b], (use & 1u) ^ 1u, dead, err);  // the epilogue has drained this accumulator
            tr_acc += RLB_NOW() - tr_a;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t d = tmem_base + b * TN;
            for (int kb = p.kb0; kb < p.kb1; kb++, cnt++) {
                const uint32_t s = cnt % kStages, ph = (cnt / kStages) & 1u;
                const unsigned long long tr_b = RLB_NOW();
                ok = mbar_wait(&full_bar[s], ph, dead, err);
                const unsigned long long tr_c = RLB_NOW();
                tr_starved += tr_c - tr_b;
                if (!tr_first) tr_first = tr_c;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t x_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                const uint32_t w_addr = x_addr + XS_BYTES;
#pragma unroll
                for (int pass = 0; pass < NX * MT; pass++)   // the hi / lo halves (tf32), or the two 128-token blocks (MT = 2)
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        // one instruction covers 32 bytes of K (16 f16 or 8 tf32 columns) along the swizzled row
                        umma<TF32>(d + (MT == 2 ? pass * TN : 0), umma_desc(x_addr + pass * X_BYTES + k * 32), umma_desc(w_addr + k * 32), idesc,
                                   (kb != p.kb0 || (MT == 1 && pass != 0) || k != 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);  // the slot is free once these MMAs have read it
            }
            if (ok) umma_commit(&acc_full[b]);
            piece++;
        }
        RLB_TR(3, tr_first); RLB_TR(4, RLB_NOW()); RLB_TR(5, tr_starved); RLB_TR(6, tr_acc); RLB_TR(10, cnt);
    } else if (warp >= 2) {
        // ---------------- epilogue: four warps per 128-token block, one TMEM lane quarter (32 tokens) each ----------------
        const int q = warp & 3, half = (warp - 2) >> 2;
        PieceIter it(sched, (int)blockIdx.x, (int)gridDim.x);
        Piece p;
        uint32_t piece = 0;
        unsigned long long tr_wait = 0, tr_busy = 0, tr_first = 0;
        const bool vec_c = ((ldc * (int64_t)sizeof(OT)) % 16 == 0) && (((uintptr_t)C & 15) == 0);
        while (it.next(p)) {
            const uint32_t b = NACC == 2 ? (piece & 1u) : 0u;
            const unsigned long long tr_a = RLB_NOW();
            const bool ok = mbar_wait(&acc_full[b], (NACC == 2 ? (piece >> 1) : piece) & 1u, dead, err);
            const unsigned long long tr_b = RLB_NOW();
            tr_wait += tr_b - tr_a;
            if (!tr_first) tr_first = tr_b;
            __syncwarp();
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int nt = p.tile / sched.n_mt, mt = p.tile - nt * sched.n_mt;
            const int token = mt * TT + half * TM + q * 32 + lane;
            const int col_base = nt * TN;
            float* slab = p.slot >= 0 ? part + ((size_t)blockIdx.x * 2 + p.slot) * kSlabFloats + (size_t)(half * TM + q * 32 + lane) * TN : nullptr;
#pragma unroll 1
            for (int c0 = 0; c0 < TN; c0 += 32) {
                if (col_base + c0 >= Mrows) break;  // (uniform over the warp)
                // two loads of 16 columns in flight before the wait
                uint32_t r[2][16];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (b + (uint32_t)half) * TN + (uint32_t)c0;
#pragma unroll
                for (int h = 0; h < 2; h++)
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                        : "=r"(r[h][0]), "=r"(r[h][1]), "=r"(r[h][2]), "=r"(r[h][3]), "=r"(r[h][4]), "=r"(r[h][5]), "=r"(r[h][6]), "=r"(r[h][7]),
                          "=r"(r[h][8]), "=r"(r[h][9]), "=r"(r[h][10]), "=r"(r[h][11]), "=r"(r[h][12]), "=r"(r[h][13]), "=r"(r[h][14]), "=r"(r[h][15])
                        : "r"(taddr + 16 * h));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int cc = c0 + 16 * h;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[h][j]);
                    if (slab) {
#pragma unroll
                        for (int j = 0; j < 4; j++) reinterpret_cast<float4*>(slab + cc)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else if (token < n && col_base + cc < Mrows) {
                        if (round_out) {
#pragma unroll
                            for (int j = 0; j < 16; j += 2) round_pair_f16(v[j], v[j + 1]);
                        }
                        OutPack<OT>::store16(C + (int64_t)token * ldc + col_base + cc, v, vec_c, Mrows - (col_base + cc));
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
            tr_busy += RLB_NOW() - tr_b;
            piece++;
        }
        if (warp == 2 && lane == 0) { RLB_TR(7, tr_first); RLB_TR(8, RLB_NOW()); RLB_TR(9, tr_wait); RLB_TR(13, tr_busy); }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Second pass for the tiles that were dealt out by k-block: out = cast(round?(sum of the tile's partial tiles
// in k order)). grid (remaining tiles, groups of 8 token rows). The CTAs whose runs meet the tile are
// found by all threads at once (thread c looks at CTA c); they are consecutive, and their order is the k order.
template <typename OT, int TN, int MT>
__global__ void __launch_bounds__(256) gemm_tc_fixup_kernel(const float* __restrict__ part, OT* __restrict__ C, int64_t ldc, int n, int Mrows,
                                                            int nkb, int grid, int round_out) {
    constexpr int TT = TM * MT;
    constexpr size_t kSlabFloats = (size_t)TT * TN;
    __shared__ int seg_slab[kMaxGrid];   // slab index (cta * 2 + slot) of CTA c's piece of this tile, or -1
    __shared__ int c_lo_s, c_hi_s;
    rlb_pdl_trigger();
    const Sched s = make_sched(n, Mrows, nkb, grid, TN, TT);
    const int j = blockIdx.x;
    if (threadIdx.x == 0) { c_lo_s = grid; c_hi_s = -1; }
    __syncthreads();
    for (int c = threadIdx.x; c < grid; c += blockDim.x) {
        const int slab = gemm_sched::partial_of(s, grid, j, c);
        if (slab >= 0) {   // CTA c's run meets the tile
            atomicMin(&c_lo_s, c);
            atomicMax(&c_hi_s, c);
        }
        seg_slab[c] = slab;
    }
    __syncthreads();
    const int c_lo = c_lo_s, c_hi = c_hi_s;
    if (c_lo >= c_hi) return;  // one CTA computed the whole tile and stored it itself
    rlb_pdl_wait();            // (the schedule above needs nothing from the GEMM; its partial tiles do)
    const int tile = s.whole + j;
    const int nt = tile / s.n_mt, mt = tile - nt * s.n_mt;
    const int row0 = blockIdx.y * 8;
    const bool vec_c = ((ldc * (int64_t)sizeof(OT)) % 16 == 0) && (((uintptr_t)C & 15) == 0);
    for (int e = threadIdx.x; e < 8 * (TN / 4); e += 256) {
        const int rr = row0 + e / (TN / 4), c4 = (e % (TN / 4)) * 4;
        const int token = mt * TT + rr, col = nt * TN + c4;
        if (token >= n || col >= Mrows) continue;
        const float* src = part + (size_t)rr * TN + c4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int c = c_lo;
        for (; c + 3 <= c_hi; c += 4) {   // four partial tiles in flight; added in k order
            float4 t[4];
#pragma unroll
            for (int k = 0; k < 4; k++)
                t[k] = seg_slab[c + k] >= 0 ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)seg_slab[c + k] * kSlabFloats)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 4; k++) { acc.x += t[k].x; acc.y += t[k].y; acc.z += t[k].z; acc.w += t[k].w; }
        }
        for (; c <= c_hi; c++)
            if (seg_slab[c] >= 0) {
                const float4 t = __ldcg(reinterpret_cast<const float4*>(src + (size_t)seg_slab[c] * kSlabFloats));
                acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
            }
        float v[4] = {acc.x, acc.y, acc.z, acc.w};
        if (round_out) {
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = __half2float(__float2half_rn(v[q]));
        }
        OT* dst = C + (int64_t)token * ldc + col;
        if (vec_c && col + 4 <= Mrows) {
            if (sizeof(OT) == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            else {
                const uint32_t w0 = (uint32_t)__half_as_ushort(__float2half_rn(v[0])) | ((uint32_t)__half_as_ushort(__float2half_rn(v[1])) << 16);
                const uint32_t w1 = (uint32_t)__half_as_ushort(__float2half_rn(v[2])) | ((uint32_t)__half_as_ushort(__float2half_rn(v[3])) << 16);
                *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
            }
        } else {
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (col + q < Mrows) {
                    if (sizeof(OT) == 4) reinterpret_cast<float*>(dst)[q] = v[q];
                    else reinterpret_cast<__half*>(dst)[q] = __float2half_rn(v[q]);
                }
        }
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

// Grows the context's GEMM scratch (split activations + partial tiles) to at least `need` bytes.
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
    rlb_pdl_trigger();
    rlb_pdl_wait();
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

template <typename OT, bool TF32, int TN, int MT>
int launch_tn(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, OT* C, int64_t ldc, int n, int M, int K, int round_out,
              int* err) {
    constexpr int BKE = TF32 ? BK / 2 : BK;
    constexpr int TT = TM * MT;
    constexpr size_t kSlabFloats = (size_t)TT * TN;
    const int nkb = (K + BKE - 1) / BKE;
    const long long units = (long long)((n + TT - 1) / TT) * ((M + TN - 1) / TN) * nkb;
    const int max_grid = ctx->sm_count < kMaxGrid ? ctx->sm_count : kMaxGrid;
    const int grid = (int)(units < max_grid ? units : max_grid);
    const Sched sched = make_sched(n, M, nkb, grid, TN, TT);
    // scratch: [x hi | x lo] for the f32 form, then two partial tiles per CTA (only touched when tiles are dealt out by k-block)
    const size_t xs = TF32 ? (((size_t)n * K * sizeof(float) + 255) & ~(size_t)255) : 0;
    const size_t slabs = sched.rest > 0 ? (size_t)grid * 2 * kSlabFloats * sizeof(float) : 0;
    RLB_TRY(reserve_scratch(ctx, 2 * xs + slabs));
    float* part = reinterpret_cast<float*>(static_cast<char*>(ctx->gemm_scratch) + 2 * xs);
    CUtensorMap tw, tx, tx2;
    RLB_TRY(make_map(&tw, W, M, K, ldw, TN, TF32));
    if (TF32) {
        float* hi = static_cast<float*>(ctx->gemm_scratch);
        float* lo = reinterpret_cast<float*>(static_cast<char*>(ctx->gemm_scratch) + xs);
        const int64_t total = (int64_t)n * K;
        int g = (int)((total + 255) / 256);
        if (g > ctx->sm_count * 16) g = ctx->sm_count * 16;
        RLB_CUDA(rlb_launch(tf32_split_kernel, dim3(g), dim3(256), 0, ctx, static_cast<const float*>(X), ldx, n, K, hi, lo));
        count_launch(ctx);
        RLB_TRY(make_map(&tx, hi, n, K, K, TM, true));
        RLB_TRY(make_map(&tx2, lo, n, K, K, TM, true));
    } else {
        RLB_TRY(make_map(&tx, X, n, K, ldx, TT));
        tx2 = tx;
    }
    const size_t smem = (size_t)kRingBytes + 1024;
    auto kern = gemm_tc_kernel<OT, TF32, TN, MT>;
    static std::atomic<uint64_t> set{0};
    if (!attr_done(set, ctx->device)) {
        RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_mark(set, ctx->device);
    }
    RLB_CUDA(rlb_launch(kern, dim3(grid), dim3(tc_threads(MT)), smem, ctx, tx, tx2, tw, C, ldc, n, M, K, round_out, part, err));
    count_launch(ctx);
    if (sched.rest > 0) {
        RLB_CUDA(rlb_launch(gemm_tc_fixup_kernel<OT, TN, MT>, dim3(sched.rest, TT / 8), dim3(256), 0, ctx, (const float*)part, C, ldc, n, M, nkb, grid,
                            round_out));
        count_launch(ctx);
    }
    return RLB_OK;
}

template <typename OT, bool TF32>
int launch_tc(rlb_ctx* ctx, const void* X, int64_t ldx, const void* W, int64_t ldw, OT* C, int64_t ldc, int n, int M, int K, int round_out,
              int* err) {
    RLB_TRY(load_encode());
    // Tile choice, from a sweep over the four models' layer shapes and prompts of 128 to 1792 tokens:
    //  - 256-token x 256-row tiles (f16 only) when whole tiles go round every SM, the token tiles pair up without
    //    padding (or the padding is under an eighth), and either K is long enough to pay for the larger epilogue
    //    or there are four rounds of tiles;
    //  - else 256-row tiles when there is a tile for every SM, or for 384 tokens and more with K up to 11008
    //    (every tile is split over K then, but the wider tile re-reads the token block half as often);
    //  - else 128-row tiles: every tile is split over K anyway and the narrower tile halves the partial results.
    const int mt = (n + TM - 1) / TM;
    const long long tiles256 = (long long)mt * ((M + 255) / 256);
    static const int force_tn = getenv("RLB_GEMM_TN") ? atoi(getenv("RLB_GEMM_TN")) : 0;  // experiments: 128, 256 or 512 (= 256-token tiles)
    if (!TF32) {
        const long long tiles_big = (long long)((n + 2 * TM - 1) / (2 * TM)) * ((M + 255) / 256);
        const bool pairs = mt % 2 == 0 || mt >= 9;
        const bool big = n > TM && pairs && tiles_big >= ctx->sm_count && (K >= 6144 || tiles_big >= 4LL * ctx->sm_count);
        if (force_tn == 512 || (force_tn == 0 && big))
            return launch_tn<OT, false, 256, 2>(ctx, X, ldx, W, ldw, C, ldc, n, M, K, round_out, err);
    }
    if (force_tn == 256) return launch_tn<OT, TF32, 256, 1>(ctx, X, ldx, W, ldw, C, ldc, n, M, K, round_out, err);
    const bool narrow = tiles256 < ctx->sm_count && !(!TF32 && n >= 3 * TM && K <= 11008);
    if (force_tn == 128 || (force_tn == 0 && narrow)) return launch_tn<OT, TF32, 128, 1>(ctx, X, ldx, W, ldw, C, ldc, n, M, K, round_out, err);
    return launch_tn<OT, TF32, 256, 1>(ctx, X, ldx, W, ldw, C, ldc, n, M, K, round_out, err);
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

#ifdef RLB_GEMM_TRACE
// (timeline build only; not part of the ABI in include/rllama_b200.h) copies the 256 x 16 trace words to `out`
extern "C" int rlb_debug_gemm_trace(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * 256 * 16);
}
#endif

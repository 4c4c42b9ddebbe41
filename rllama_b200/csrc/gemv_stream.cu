// Decode GEMV with the weight stream staged through shared memory by the bulk-copy engine.
//
// Same contraction, prologues and epilogues as gemv.cu (rllama's one-row
// Tensor::matrix_mul_transposed, src/tensor.rs:999-1025, :1250-1668), different data path:
// a GEMV at batch 1 is bound by how many bytes are in flight, and register-staged loads
// leave that to the compiler's scheduling. Here one producer warp issues `cp.async.bulk`
// copies (global -> shared, completion counted on an mbarrier) of RB weight rows x KC
// columns per stage into a ring of up to 12 stages (up to ~190 KB in flight per SM), and
// eight consumer warps read the stages from shared memory. The producer starts before the
// kernel waits for its predecessor (programmatic dependent launch): weights do not depend
// on the previous kernel, so the ring is already full when the activation row arrives.
//
// Work split: a CTA owns whole row tiles (RB rows x all of K); inside a tile the eight
// consumer warps split K. Each warp folds its lanes' partial sums with a halving exchange
// (9 shuffles for 8 rows) and hands one value per row to a tenth warp, which adds the eight
// warps in a fixed order and runs the fused epilogue, so the consumers never stop at a
// CTA-wide barrier and results do not depend on the grid size.
//
// Prologue latency is what separates consecutive kernels, so its loads are written as explicit
// batches (volatile asm): the RMSNorm gains before the dependency wait, then the residual row
// and the partial sums in one round trip through L2, all kept in registers.
//
// Every wait on an mbarrier is bounded: when a wait runs out the kernel raises an error flag
// in global memory, switches to a mode in which no wait blocks, and runs to its end.
#include "internal.h"

#include <cstdlib>

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 64;  // + one producer warp + one epilogue warp
constexpr int kPartialDepth = 2;           // tiles the epilogue warp may lag behind
constexpr int kMaxStages = 12;
constexpr uint32_t kWaitLimit = 1u << 20;

template <typename T> struct Vec;
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };

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
// Bounded wait. Returns immediately once the CTA is in "dead" mode.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* dead, int* err) {
    for (uint32_t i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 255u) == 255u && *dead) return;
    }
    *dead = 1;
    atomicExch(err, 1);
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Loads as volatile asm: the compiler keeps them where they are written (all requests of a batch
// first, uses later; nothing sinks below the dependency wait), so a batch costs one round trip.
__device__ __forceinline__ float4 ld_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cg_f4(const float* p) {  // L2 only: data published by other CTAs of this kernel
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_u4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// (private to this file) PRO_NORM whose tensor-parallel consumer gathers the whole row in every CTA
constexpr int PRO_NORM_GATHER = 2;

// Tensor-parallel exchange entries: {f32 value, u32 sequence number} in one 8-byte store.
__device__ __forceinline__ void ll_store(uint2* p, float v, uint32_t seq) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}
// Bounded poll of up to N entries (base + j * stride, j < count) until each carries `seq`. All
// pending entries are requested before any is examined, so one round costs one memory round
// trip. On a timeout the missing values read as 0, *dead is set and the error word raised.
template <int N>
__device__ __forceinline__ void ll_gather(const uint2* base, size_t stride, int count, uint32_t seq, float (&v)[N], volatile int* dead,
                                          int* err) {
    uint32_t pend = count >= N ? ((N == 32) ? 0xffffffffu : ((1u << N) - 1u)) : ((1u << count) - 1u);
#pragma unroll
    for (int j = 0; j < N; j++) v[j] = 0.f;
    for (uint32_t it = 0; pend != 0 && it < (1u << 20); it++) {
        uint32_t vv[N], ff[N];
#pragma unroll
        for (int j = 0; j < N; j++)
            if (pend & (1u << j))
                asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(vv[j]), "=r"(ff[j]) : "l"(base + (size_t)j * stride) : "memory");
#pragma unroll
        for (int j = 0; j < N; j++)
            if ((pend & (1u << j)) && ff[j] == seq) {
                v[j] = __uint_as_float(vv[j]);
                pend &= ~(1u << j);
            }
        if ((it & 255u) == 255u && *dead) return;
    }
    if (pend != 0) {
        *dead = 1;
        atomicExch(err, 2);
    }
}

// The same poll for a whole row: the thread's G groups of four consecutive entries (element tid * 4 + g * 4 * stride4)
// from `count` ranks, rank r's row at base + r * K; sum[g] = entries of rank 0 + rank 1 + ... in that order. A group is
// two 16-byte loads (four {value, sequence} entries); all pending groups of a rank are requested before any is examined.
// (Every entry was written by one aligned 8-byte store and is read inside one aligned 16-byte access, so a value is never
// seen with another store's sequence number; an entry of the pair that has not arrived yet just fails the comparison.)
template <int G>
__device__ __forceinline__ void ll_gather_row(const uint2* base, int K, int count, uint32_t seq, int tid, int stride4, float4 (&sum)[G],
                                              volatile int* dead, int* err) {
    uint32_t valid = 0;
#pragma unroll
    for (int g = 0; g < G; g++) {
        sum[g] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tid * 4 + g * 4 * stride4 < K) valid |= 1u << g;
    }
    for (int r = 0; r < count; r++) {
        const uint2* row = base + (size_t)r * K;
        uint32_t pend = valid;
        for (uint32_t it = 0; pend != 0 && it < (1u << 20); it++) {
            uint4 lo[G], hi[G];
#pragma unroll
            for (int g = 0; g < G; g++)
                if (pend & (1u << g)) {
                    const uint2* p = row + tid * 4 + g * 4 * stride4;
                    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(lo[g].x), "=r"(lo[g].y), "=r"(lo[g].z), "=r"(lo[g].w) : "l"(p) : "memory");
                    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(hi[g].x), "=r"(hi[g].y), "=r"(hi[g].z), "=r"(hi[g].w) : "l"(p + 2) : "memory");
                }
#pragma unroll
            for (int g = 0; g < G; g++)
                if ((pend & (1u << g)) && lo[g].y == seq && lo[g].w == seq && hi[g].y == seq && hi[g].w == seq) {
                    sum[g].x += __uint_as_float(lo[g].x); sum[g].y += __uint_as_float(lo[g].z);
                    sum[g].z += __uint_as_float(hi[g].x); sum[g].w += __uint_as_float(hi[g].z);
                    pend &= ~(1u << g);
                }
            if ((it & 255u) == 255u && *dead) return;
        }
        if (pend != 0) {
            *dead = 1;
            atomicExch(err, 2);
            return;
        }
    }
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
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sums N per-lane values over the warp with N - 1 + log2(32 / N) shuffles instead of 5 N: each
// halving step hands half of the values to the partner lane. Afterwards every lane holds the
// warp total of value number lane / (32 / N).
template <int N, int O = 16>
__device__ __forceinline__ float warp_fold(float (&v)[N], int lane) {
    if constexpr (N == 1) {
        float r = v[0];
#pragma unroll
        for (int o = O; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        return r;
    } else {
        const bool up = (lane & O) != 0;
        float h[N / 2];
#pragma unroll
        for (int i = 0; i < N / 2; i++) {
            const float keep = up ? v[i + N / 2] : v[i];
            const float send = up ? v[i] : v[i + N / 2];
            h[i] = keep + __shfl_xor_sync(0xffffffffu, send, O);
        }
        return warp_fold<N / 2, O / 2>(h, lane);
    }
}

struct StreamCfg {
    int n_stages;
    int* err;
};
// G: float4 groups of the activation row a consumer thread holds in the norm prologue (4: rows of up
// to 4096 elements, 8: up to 8192).
template <typename WT, int RB, int J, int PRO, int EPI, int G>
__global__ void __launch_bounds__(kThreads, 1) gemv_stream_kernel(const GemvArgs a, const StreamCfg cfg) {
    constexpr int VEC = Vec<WT>::N;
    constexpr int NMAT = (EPI == EPI_SWIGLU) ? 2 : 1;
    constexpr int SL = J * 32 * VEC;               // K elements one warp covers per stage
    constexpr int KC = kConsumerWarps * SL;        // K elements per stage
    constexpr int NSEG = NMAT * RB;                // row segments per stage
    constexpr int STAGE_ELEMS = NSEG * KC;
    constexpr size_t STAGE_BYTES = (size_t)STAGE_ELEMS * sizeof(WT);

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int K = a.K, S = cfg.n_stages;
    WT* ring = reinterpret_cast<WT*>(smem_raw);
    unsigned char* p = smem_raw + (size_t)S * STAGE_BYTES;
    WT* act = reinterpret_cast<WT*>(p);
    p += (((size_t)K * sizeof(WT)) + 15) & ~(size_t)15;
    float* partial = reinterpret_cast<float*>(p);  // [kPartialDepth][NSEG][kConsumerWarps]
    p += sizeof(float) * kPartialDepth * NSEG * kConsumerWarps;
    float* red = reinterpret_cast<float*>(p);
    p += sizeof(float) * kConsumerWarps;
    p = reinterpret_cast<unsigned char*>(((uintptr_t)p + 7) & ~(uintptr_t)7);
    uint64_t* full = reinterpret_cast<uint64_t*>(p);
    uint64_t* empty = full + kMaxStages;
    uint64_t* pfull = empty + kMaxStages;       // [kPartialDepth] consumers -> epilogue warp
    uint64_t* pempty = pfull + kPartialDepth;   // [kPartialDepth] epilogue warp -> consumers
    __shared__ int dead_flag;
    volatile int* dead = &dead_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        dead_flag = 0;
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        for (int s = 0; s < kPartialDepth; s++) {
            mbar_init(&pfull[s], kConsumerWarps);
            mbar_init(&pempty[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    const int n_tiles = a.rows / RB;
    const WT* W_a = reinterpret_cast<const WT*>(a.W);
    const WT* W_b = reinterpret_cast<const WT*>(a.W2);

    if (warp == kConsumerWarps) {
        // ------------------------------ producer warp -------------------------------------
        int s = 0;
        uint32_t ph = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const int row0 = tile * RB;
            for (int k0 = 0; k0 < K; k0 += KC) {
                mbar_wait(&empty[s], ph ^ 1u, dead, cfg.err);
                const int kn = min(KC, K - k0);
                const uint32_t nbytes = (uint32_t)kn * sizeof(WT);
                if (lane == 0) mbar_expect_tx(&full[s], nbytes * NSEG);
                __syncwarp();
                if (lane < NSEG && !*dead) {
                    const int m = lane / RB, r = lane - m * RB;
                    bulk_g2s(ring + (size_t)s * STAGE_ELEMS + (size_t)lane * KC, (m == 0 ? W_a : W_b) + (int64_t)(row0 + r) * a.ldw + k0,
                             nbytes, &full[s]);
                }
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
        return;
    }

    // RMSNorm gains never change: fetch this thread's share before waiting for the previous kernel.
    // A consumer thread owns the four elements at tid * 4 + g * 4 * kConsumers of the row, g < kRowGroups.
    constexpr int kRowGroups = G;
    constexpr bool kGainEarly = G <= 4;  // with 8 groups the registers are needed for the row itself
    float4 gain_r[kRowGroups];
    if (PRO != PRO_COPY && kGainEarly && warp < kConsumerWarps) {
#pragma unroll
        for (int g = 0; g < kRowGroups; g++) {
            const int i = tid * 4 + g * 4 * kConsumers;
            gain_r[g] = i < K ? ld_f4(a.gain + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }

    pdl_wait();  // everything below reads or overwrites what earlier kernels use

    if (warp == kConsumerWarps + 1) {
        // ------------------------------ epilogue warp -------------------------------------
        int ps = 0;
        uint32_t pph = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const int row0 = tile * RB;
            mbar_wait(&pfull[ps], pph, dead, cfg.err);
            const float* pp = partial + (size_t)ps * NSEG * kConsumerWarps;
            float mine = 0.f;  // lane i < NSEG: the dot product of row segment i
            if (lane < NSEG) {
#pragma unroll
                for (int w = 0; w < kConsumerWarps; w++) mine += pp[lane * kConsumerWarps + w];  // fixed order
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&pempty[ps]);
            if (++ps == kPartialDepth) { ps = 0; pph ^= 1u; }
            auto total = [&](int i) { return __shfl_sync(0xffffffffu, mine, i & 31); };
            if (EPI == EPI_STORE) {
                if (lane < RB) reinterpret_cast<WT*>(a.out)[(int64_t)(row0 + lane) * a.out_stride] = cast_to<WT>(mine);
            } else if (EPI == EPI_F32) {
                if (lane < RB) {
                    const float v = mine;
                    if (a.n_outs == 0) {
                        reinterpret_cast<float*>(a.out)[(int64_t)(row0 + lane) * a.out_stride] = v;
                    } else {
                        // push this partial sum, tagged with the exchange's sequence number, into every rank's inbox
                        const uint32_t seq = (uint32_t)(*a.epoch_ptr - 1) * a.seq_stride + a.out_seq_idx;
                        for (int d = 0; d < a.n_outs; d++) ll_store(a.ll_outs[d] + a.out_offset + row0 + lane, v, seq);
                    }
                }
            } else if (EPI == EPI_SWIGLU) {
                const float up3 = total(RB + lane);
                if (lane < RB) {
                    const float a1 = maybe_round<WT>(mine);
                    const float a3 = maybe_round<WT>(up3);
                    const float sg = a1 / (1.0f + expf(-a1));
                    reinterpret_cast<WT*>(a.out)[row0 + lane] = cast_to<WT>(__fmul_rn(sg, a3));
                }
            } else if (EPI == EPI_QKV) {
                const float t_re = total(2 * lane), t_im = total(2 * lane + 1);
                if (lane < RB / 2) {
                    const int pos = *a.pos_ptr;
                    const int row = row0 + 2 * lane;
                    const int sec = row / a.nq, rr = row - sec * a.nq;
                    const int head = rr / a.hd, c = rr - head * a.hd;
                    const float re = maybe_round<WT>(t_re);
                    const float im = maybe_round<WT>(t_im);
                    const float* f = a.rope + ((int64_t)pos * (a.hd / 2) + (c >> 1)) * 2;
                    const float fr = f[0], fi = f[1];
                    const float o_re = __fsub_rn(__fmul_rn(re, fr), __fmul_rn(im, fi));  // src/transformer.rs:844-847
                    const float o_im = __fadd_rn(__fmul_rn(re, fi), __fmul_rn(im, fr));
                    if (sec == 0) {
                        a.qbuf[rr] = o_re;
                        a.qbuf[rr + 1] = o_im;
                    } else {
                        WT* cache = reinterpret_cast<WT*>(sec == 1 ? a.kcache : a.vcache);
                        WT* dst = cache + ((int64_t)head * a.max_seq + pos) * a.hd + c;
                        dst[0] = cast_to<WT>(sec == 1 ? o_re : re);
                        dst[1] = cast_to<WT>(sec == 1 ? o_im : im);
                    }
                }
            }
        }
        return;
    }

    // -------------------------------- consumer warps ---------------------------------------
    if (PRO == PRO_COPY) {
        const uint4* src = reinterpret_cast<const uint4*>(a.vec_in);
        uint4* dst = reinterpret_cast<uint4*>(act);
        const int nv = K / VEC;
        for (int i0 = tid; i0 < nv; i0 += 8 * kConsumers) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (i0 + u * kConsumers < nv) v[u] = ld_u4(src + i0 + u * kConsumers);
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (i0 + u * kConsumers < nv) dst[i0 + u * kConsumers] = v[u];
        }
    } else {
        const float* xin = a.x_in;
        if (a.tok_ptr) xin += (int64_t)(*a.tok_ptr) * K;
        float ss = 0.f;
        float4 xr[kRowGroups];  // this thread's elements of the residual row
        if (PRO == PRO_NORM_GATHER && kRowGroups <= 4) {
            // Tensor-parallel push exchange, short rows: every CTA collects the whole row's partial sums from every
            // rank's entries itself (rank order, f16 rounding after the sum) and adds the residual; CTA 0 stores the new
            // residual row for the kernels that follow. No CTA waits for another one.
            constexpr int GG = kRowGroups <= 4 ? kRowGroups : 1;
            const uint32_t seq = (uint32_t)(*a.epoch_ptr - 1) * a.seq_stride + a.seq_idx;
#pragma unroll
            for (int g = 0; g < GG; g++) {
                const int i = tid * 4 + g * 4 * kConsumers;
                xr[g] = i < K ? ld_f4(xin + i) : make_float4(0.f, 0.f, 0.f, 0.f);  // requested before the poll
            }
            float4 sum[GG];
            ll_gather_row<GG>(a.ll_inbox, K, a.n_parts, seq, tid, kConsumers, sum, dead, cfg.err);
#pragma unroll
            for (int g = 0; g < GG; g++) {
                const int i = tid * 4 + g * 4 * kConsumers;
                if (i < K) {
                    float4 sacc = sum[g];
                    if (a.round_parts) {
                        sacc.x = round_f16(sacc.x); sacc.y = round_f16(sacc.y); sacc.z = round_f16(sacc.z); sacc.w = round_f16(sacc.w);
                    }
                    float4 v = xr[g];
                    v.x += sacc.x; v.y += sacc.y; v.z += sacc.z; v.w += sacc.w;
                    xr[g] = v;
                    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                    if (blockIdx.x == 0) *reinterpret_cast<float4*>(a.x_out + i) = v;
                }
            }
        } else if (a.ll_inbox != nullptr) {
            // Tensor-parallel push exchange. This CTA owns a slice of the residual row: it collects
            // that slice's partial sums from every rank's entries (rank order, f16 rounding after the
            // sum), adds the residual and publishes the result as {value, sequence} entries; then
            // every CTA reads the whole new residual from those entries. The sequence numbers carry
            // the ordering: no fence, no grid barrier.
            const uint32_t seq = (uint32_t)(*a.epoch_ptr - 1) * a.seq_stride + a.seq_idx;
            const int per = ((K + (int)gridDim.x - 1) / (int)gridDim.x + 3) & ~3;
            const int s0 = min(K, (int)blockIdx.x * per), s1 = min(K, s0 + per);
            for (int i = s0 + tid; i < s1; i += kConsumers) {
                const float xv = xin[i];  // requested before the poll, so its latency hides behind it
                float part[RLB_MAX_TP];
                ll_gather<RLB_MAX_TP>(a.ll_inbox + i, (size_t)K, a.n_parts, seq, part, dead, cfg.err);
                float sum = part[0];
#pragma unroll
                for (int q = 1; q < RLB_MAX_TP; q++)
                    if (q < a.n_parts) sum += part[q];  // fixed rank order: identical on every rank
                if (a.round_parts) sum = round_f16(sum);
                a.x_out[i] = xv + sum;
            }
            // Publish the slice with plain stores, a device-scope fence and one count per CTA; the
            // other CTAs poll that single counter (thousands of threads polling entries would
            // compete with the stores they wait for), then read the row through L2.
            __threadfence();
            consumer_sync();
            if (tid == 0) {
                atomicAdd(a.xready, 1u);
                const unsigned int target = (unsigned int)(*a.epoch_ptr) * gridDim.x;
                bool ok = false;
                for (uint32_t it = 0; it < (1u << 20) && !*dead; it++) {
                    unsigned int v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.xready) : "memory");
                    if (v >= target) { ok = true; break; }
                    __nanosleep(40);
                }
                if (!ok) { *dead = 1; atomicExch(cfg.err, 2); }
            }
            consumer_sync();
#pragma unroll
            for (int g = 0; g < kRowGroups; g++) {
                const int i = tid * 4 + g * 4 * kConsumers;
                if (i < K) xr[g] = ld_cg_f4(a.x_out + i);  // all requests first: one round trip through L2
            }
#pragma unroll
            for (int g = 0; g < kRowGroups; g++) {
                const int i = tid * 4 + g * 4 * kConsumers;
                if (i < K) {
                    const float4 v = xr[g];
                    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                }
            }
        } else {
            // all loads first (the conditional store below may alias them as far as the compiler knows,
            // which would otherwise serialise the groups: one L2 round trip each)
            float4 pr[kRowGroups];
#pragma unroll
            for (int g = 0; g < kRowGroups; g++) {
                const int i = tid * 4 + g * 4 * kConsumers;
                if (i < K) {
                    xr[g] = ld_f4(xin + i);
                    if (a.n_parts > 0) pr[g] = ld_f4(a.parts + i);
                }
            }
#pragma unroll
            for (int g = 0; g < kRowGroups; g++) {
                const int i = tid * 4 + g * 4 * kConsumers;
                if (i < K) {
                    float4 v = xr[g];
                    if (a.n_parts > 0) {
                        float4 sacc = pr[g];
                        for (int q = 1; q < a.n_parts; q++) {  // fixed rank order
                            const float4 t = *reinterpret_cast<const float4*>(a.parts + q * a.part_stride + i);
                            sacc.x += t.x; sacc.y += t.y; sacc.z += t.z; sacc.w += t.w;
                        }
                        if (a.round_parts) {
                            sacc.x = round_f16(sacc.x); sacc.y = round_f16(sacc.y); sacc.z = round_f16(sacc.z); sacc.w = round_f16(sacc.w);
                        }
                        v.x += sacc.x; v.y += sacc.y; v.z += sacc.z; v.w += sacc.w;
                    }
                    xr[g] = v;
                    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                }
            }
            if (blockIdx.x == 0 && a.x_out) {
#pragma unroll
                for (int g = 0; g < kRowGroups; g++) {
                    const int i = tid * 4 + g * 4 * kConsumers;
                    if (i < K) *reinterpret_cast<float4*>(a.x_out + i) = xr[g];
                }
            }
        }
        if (!kGainEarly) {
#pragma unroll
            for (int g = 0; g < kRowGroups; g++) {
                const int i = tid * 4 + g * 4 * kConsumers;
                if (i < K) gain_r[g] = ld_f4(a.gain + i);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        consumer_sync();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; w++) tot += red[w];
        const float scale = 1.0f / sqrtf(tot / (float)K + a.eps);
#pragma unroll
        for (int g = 0; g < kRowGroups; g++) {
            const int i = tid * 4 + g * 4 * kConsumers;
            if (i < K) {
                act[i] = cast_to<WT>(__fmul_rn(__fmul_rn(xr[g].x, scale), gain_r[g].x));
                act[i + 1] = cast_to<WT>(__fmul_rn(__fmul_rn(xr[g].y, scale), gain_r[g].y));
                act[i + 2] = cast_to<WT>(__fmul_rn(__fmul_rn(xr[g].z, scale), gain_r[g].z));
                act[i + 3] = cast_to<WT>(__fmul_rn(__fmul_rn(xr[g].w, scale), gain_r[g].w));
            }
        }
    }
    consumer_sync();

    int s = 0, ps = 0;
    uint32_t ph = 0, pph = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        float acc[NSEG];
#pragma unroll
        for (int i = 0; i < NSEG; i++) acc[i] = 0.f;
        for (int k0 = 0; k0 < K; k0 += KC) {
            mbar_wait(&full[s], ph, dead, cfg.err);
            const WT* st = ring + (size_t)s * STAGE_ELEMS;
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int kk = warp * SL + (j * 32 + lane) * VEC;
                if (k0 + kk < K) {
                    float af[VEC];
                    unpack<WT>(*reinterpret_cast<const uint4*>(act + k0 + kk), af);
#pragma unroll
                    for (int i = 0; i < NSEG; i++) {
                        float wf[VEC];
                        unpack<WT>(*reinterpret_cast<const uint4*>(st + (size_t)i * KC + kk), wf);
#pragma unroll
                        for (int e = 0; e < VEC; e++) acc[i] = fmaf(wf[e], af[e], acc[i]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (++s == S) { s = 0; ph ^= 1u; }
        }
        // fold across the warp and hand one partial sum per row segment to the epilogue warp
        const float folded = warp_fold<NSEG>(acc, lane);
        mbar_wait(&pempty[ps], pph ^ 1u, dead, cfg.err);
        if ((lane & (32 / NSEG - 1)) == 0) partial[((size_t)ps * NSEG + lane / (32 / NSEG)) * kConsumerWarps + warp] = folded;
        __syncwarp();
        if (lane == 0) mbar_arrive(&pfull[ps]);
        if (++ps == kPartialDepth) { ps = 0; pph ^= 1u; }
    }
}

struct StreamTuning {
    bool loaded = false;
    int stage_kb = 32;   // 16, 32 or 64
    int max_stages = kMaxStages;
    int pdl = 1;
    int rb = 0;          // explicit rows per tile (0 = from stage_kb)
    int smem_kb = 192;   // shared memory per CTA; the rest of the SM stays free for small co-resident CTAs
} g_st;

void load_tuning() {
    if (g_st.loaded) return;
    g_st.loaded = true;
    if (const char* s = getenv("RLB_STREAM_STAGE_KB")) { int v = atoi(s); g_st.stage_kb = v >= 64 ? 64 : v >= 32 ? 32 : 16; }
    if (const char* s = getenv("RLB_STREAM_STAGES")) { int v = atoi(s); if (v >= 2 && v <= kMaxStages) g_st.max_stages = v; }
    if (const char* s = getenv("RLB_STREAM_PDL")) g_st.pdl = atoi(s) != 0;
    if (const char* s = getenv("RLB_STREAM_RB")) g_st.rb = atoi(s);
    if (const char* s = getenv("RLB_STREAM_SMEM_KB")) { int v = atoi(s); if (v >= 48 && v <= 224) g_st.smem_kb = v; }
}

template <typename WT, int RB, int J, int PRO, int EPI, int G>
int launch_cfg(rlb_ctx* ctx, const GemvArgs& a, int* err_flag, bool pdl) {
    constexpr int VEC = Vec<WT>::N;
    constexpr int NMAT = (EPI == EPI_SWIGLU) ? 2 : 1;
    constexpr size_t STAGE_BYTES = (size_t)NMAT * RB * J * 8 * 32 * VEC * sizeof(WT);
    auto kern = gemv_stream_kernel<WT, RB, J, PRO, EPI, G>;
    size_t fixed = (((size_t)a.K * sizeof(WT)) + 15) & ~(size_t)15;
    fixed += sizeof(float) * kPartialDepth * NMAT * RB * kConsumerWarps + sizeof(float) * kConsumerWarps + 16 +
             (2 * kMaxStages + 2 * kPartialDepth) * sizeof(uint64_t);
    const size_t budget = (size_t)g_st.smem_kb * 1024;
    if (fixed + 2 * STAGE_BYTES > budget) return rlb_fail(RLB_ERR_LIMIT, "gemv: activation row of %d elements leaves no room for the weight ring", a.K);
    int stages = (int)((budget - fixed) / STAGE_BYTES);
    if (stages > g_st.max_stages) stages = g_st.max_stages;
    const size_t smem = fixed + (size_t)stages * STAGE_BYTES;
    static std::atomic<uint64_t> attr_set{0};
    if (!attr_done(attr_set, ctx->device)) {
        RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        // every kernel of the decode chain asks for the same shared-memory split, so that CTAs of
        // consecutive kernels can share an SM
        RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        attr_mark(attr_set, ctx->device);
    }
    const int n_tiles = a.rows / RB;
    const int max_grid = ctx->sm_count;
    int grid = n_tiles < max_grid ? n_tiles : max_grid;
    StreamCfg cfg;
    cfg.n_stages = stages;
    cfg.err = err_flag;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(kThreads);
    lc.dynamicSmemBytes = smem;
    lc.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = pdl ? 1 : 0;
    RLB_CUDA(cudaLaunchKernelEx(&lc, kern, a, cfg));
    count_launch(ctx);
    return RLB_OK;
}

// Rows per tile and vectors per lane for a shape; rb == 0 means "not handled here".
struct ShapeCfg { int rb; int j; };
ShapeCfg pick_cfg(int epilogue, const GemvArgs& a) {
    load_tuning();
    const int nmat = (epilogue == EPI_SWIGLU) ? 2 : 1;
    const int unit = (epilogue == EPI_QKV) ? a.nq : a.rows;
    const int J = 1;  // stage = nmat * RB * 4 KB
    int RB = g_st.rb > 0 ? g_st.rb / nmat : g_st.stage_kb / 4 / nmat / J;
    if (RB > 8) RB = 8;
    if (RB < 1) RB = 1;
    while (RB > 1 && (unit % RB != 0 || a.rows % RB != 0)) RB >>= 1;
    if (RB < 2) return ShapeCfg{0, J};
    if (nmat == 2 && RB > 4) RB = 4;
    return ShapeCfg{RB, J};
}

template <typename WT, int PRO, int EPI>
int launch_shape(rlb_ctx* ctx, const GemvArgs& a, int* err_flag, bool pdl) {
    constexpr int NMAT = (EPI == EPI_SWIGLU) ? 2 : 1;
    const ShapeCfg sc = pick_cfg(EPI, a);
    if (sc.rb == 0) return RLB_ERR_STATE;  // caller falls back to the register-staged kernel
    // (the two-vectors-per-lane variants J = 2 were measured slower at every shape and are not built)
    const bool wide = PRO != PRO_COPY && a.K > 4096;
    switch (sc.rb) {
        case 8:
            return wide ? launch_cfg<WT, (NMAT == 1 ? 8 : 4), 1, PRO, EPI, (PRO != PRO_COPY ? 8 : 4)>(ctx, a, err_flag, pdl)
                        : launch_cfg<WT, (NMAT == 1 ? 8 : 4), 1, PRO, EPI, 4>(ctx, a, err_flag, pdl);
        case 4:
            return wide ? launch_cfg<WT, 4, 1, PRO, EPI, (PRO != PRO_COPY ? 8 : 4)>(ctx, a, err_flag, pdl)
                        : launch_cfg<WT, 4, 1, PRO, EPI, 4>(ctx, a, err_flag, pdl);
        case 2:
            return wide ? launch_cfg<WT, 2, 1, PRO, EPI, (PRO != PRO_COPY ? 8 : 4)>(ctx, a, err_flag, pdl)
                        : launch_cfg<WT, 2, 1, PRO, EPI, 4>(ctx, a, err_flag, pdl);
        default: break;
    }
    return RLB_ERR_STATE;
}

template <typename WT>
int launch_typed(rlb_ctx* ctx, int prologue, int epilogue, const GemvArgs& a, int* err_flag, bool pdl) {
    // the tensor-parallel consumer that gathers the whole row in every CTA is a kernel of its own, so that the
    // single-GPU kernels carry none of its code (measured: 1.3 % on the 7B token when it was a run-time branch)
    if (prologue == PRO_NORM && a.ll_inbox != nullptr && a.gather_all && a.K <= 4096) {
        if (epilogue == EPI_QKV) return launch_shape<WT, PRO_NORM_GATHER, EPI_QKV>(ctx, a, err_flag, pdl);
        if (epilogue == EPI_SWIGLU) return launch_shape<WT, PRO_NORM_GATHER, EPI_SWIGLU>(ctx, a, err_flag, pdl);
        if (epilogue == EPI_F32) return launch_shape<WT, PRO_NORM_GATHER, EPI_F32>(ctx, a, err_flag, pdl);
    }
    if (prologue == PRO_NORM && epilogue == EPI_QKV) return launch_shape<WT, PRO_NORM, EPI_QKV>(ctx, a, err_flag, pdl);
    if (prologue == PRO_NORM && epilogue == EPI_SWIGLU) return launch_shape<WT, PRO_NORM, EPI_SWIGLU>(ctx, a, err_flag, pdl);
    if (prologue == PRO_NORM && epilogue == EPI_F32) return launch_shape<WT, PRO_NORM, EPI_F32>(ctx, a, err_flag, pdl);
    if (prologue == PRO_COPY && epilogue == EPI_F32) return launch_shape<WT, PRO_COPY, EPI_F32>(ctx, a, err_flag, pdl);
    return RLB_ERR_STATE;
}

}  // namespace

static bool stream_shape_ok(rlb_dtype dtype, int prologue, const GemvArgs& a) {
    const int vec = dtype == RLB_F16 ? 8 : 4;
    if (a.K <= 0 || a.rows < 2 || a.K % vec != 0 || a.ldw % vec != 0) return false;
    if (prologue == PRO_NORM && (a.K % 4 != 0 || a.K > 8192)) return false;  // the norm keeps the row in registers
    if ((a.ldw * (int64_t)(dtype == RLB_F16 ? 2 : 4)) % 16 != 0) return false;  // bulk copies need 16-byte aligned rows
    return true;
}

int gemv_stream_grid(rlb_ctx* ctx, rlb_dtype dtype, int prologue, int epilogue, const GemvArgs& a) {
    if (!stream_shape_ok(dtype, prologue, a)) return 0;
    const ShapeCfg sc = pick_cfg(epilogue, a);
    if (sc.rb == 0) return 0;
    const int n_tiles = a.rows / sc.rb;
    const int max_grid = ctx->sm_count;
    return n_tiles < max_grid ? n_tiles : max_grid;
}

// Returns RLB_ERR_STATE (without recording an error message) when the shape is not handled
// here, so that the caller can use the register-staged kernel instead.
int launch_gemv_stream(rlb_ctx* ctx, rlb_dtype dtype, int prologue, int epilogue, const GemvArgs& a, int* err_flag, int allow_pdl) {
    load_tuning();
    if (!stream_shape_ok(dtype, prologue, a)) return RLB_ERR_STATE;
    const bool pdl = allow_pdl && g_st.pdl;
    return dtype == RLB_F16 ? launch_typed<__half>(ctx, prologue, epilogue, a, err_flag, pdl)
                            : launch_typed<float>(ctx, prologue, epilogue, a, err_flag, pdl);
}

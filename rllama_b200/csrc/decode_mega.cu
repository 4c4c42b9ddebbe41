// One persistent kernel per decoded token.
//
// The per-layer decode chain of model.cu (q/k/v GEMV -> attention -> wo GEMV -> w1/w3 GEMV ->
// w2 GEMV, then the vocabulary head and the arg-max; rllama's Transformer::forward for one
// token, src/transformer.rs:343-382, :424-446, :536-582, :657-820) runs here as ONE cooperative
// launch of one CTA per SM that walks a table of phases. Kernel boundaries cost a drain of the
// weight stream, a launch and a fresh ramp-up for every one of the 5 L + 2 stages; inside one
// kernel
//  * the producer warp never stops: it streams the next phase's weights into the shared-memory
//    ring (cp.async.bulk + mbarrier, as in gemv_stream.cu) while the consumer warps are still in
//    the previous phase's epilogue, in attention, or waiting for other CTAs;
//  * stages that need every CTA's output of the previous stage (attention after q/k/v, wo after
//    attention, w2 after the gate) wait on a per-phase completion counter in global memory;
//  * stages that need a sum over all output rows (the norms after wo and w2, the arg-max after
//    the head) exchange 8-byte {value, sequence number} entries: the writer needs no fence and
//    the reader polls the entry itself. Under tensor parallelism the same entries are stored
//    into every rank's inbox over NVLink, so the all-reduce is fused into the projection kernel
//    and its consumer, with the sum taken in rank order on every rank.
//
// Every wait (mbarrier, completion counter, entry poll) is bounded. A wait that runs out raises
// the error word in global memory; every other wait sees the word within 256 polls and stops
// blocking, so the kernel always runs to its end.
#include "internal.h"

#include <cfloat>

namespace {

constexpr int kCW = 8;                 // consumer warps
constexpr int kConsumers = kCW * 32;
constexpr int kMegaThreads = kConsumers + 64;  // + producer warp + epilogue warp
constexpr int kSegBytes = 4096;        // one weight-row segment of a stage
constexpr int kNSeg = 8;               // row segments per stage
constexpr int kStageBytes = kSegBytes * kNSeg;
constexpr int kPartialDepth = 2;
constexpr int kMaxStages = 6;
constexpr uint32_t kWaitLimit = 1u << 20;

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
__device__ __forceinline__ bool is_dead(const int* err) { return *reinterpret_cast<const volatile int*>(err) != 0; }
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
    for (uint32_t i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 255u) == 255u && is_dead(err)) return;
    }
    atomicExch(err, 1);
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

__device__ __forceinline__ void ll_store(uint2* p, float v, uint32_t seq) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}
// Bounded poll of up to N entries (base + j * stride, j < count) until each carries `seq`.
template <int N>
__device__ __forceinline__ void ll_gather(const uint2* base, size_t stride, int count, uint32_t seq, float (&v)[N], int* err) {
    uint32_t pend = count >= N ? ((N == 32) ? 0xffffffffu : ((1u << N) - 1u)) : ((1u << count) - 1u);
#pragma unroll
    for (int j = 0; j < N; j++) v[j] = 0.f;
    for (uint32_t it = 0; pend != 0 && it < kWaitLimit; it++) {
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
        if ((it & 255u) == 255u && is_dead(err)) return;
        if (pend != 0) __nanosleep(40);
    }
    if (pend != 0) atomicExch(err, 2);
}

__device__ __forceinline__ float round_f16(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T> struct Vec;
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };
template <typename T> __device__ __forceinline__ T cast_to(float v);
template <> __device__ __forceinline__ __half cast_to<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast_to<float>(float v) { return v; }
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

struct Smem {
    unsigned char* ring;
    unsigned char* act;   // activation row of the current GEMV phase (weight dtype)
    float* tmp;           // dim floats (norm), attention merge area, arg-max scratch
    float* partial;       // [kPartialDepth][kNSeg][kConsumers]
    float* red;           // [kCW]
    uint64_t* full;
    uint64_t* empty;
    uint64_t* pfull;
    uint64_t* pempty;
};

// Consumer warps wait (bounded, with a short back-off) until a monotonic counter reaches `target`.
__device__ __forceinline__ void wait_counter(const unsigned int* ctr, uint32_t target, int* err, int code) {
    if (threadIdx.x == 0) {
        bool ok = false;
        for (uint32_t i = 0; i < kWaitLimit; i++) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
            if (v >= target) { ok = true; break; }
            if ((i & 255u) == 255u && is_dead(err)) break;
            __nanosleep(40);
        }
        if (!ok) atomicExch(err, code);
    }
    consumer_sync();
}
// Waits until every CTA has completed phase `p` of this launch.
__device__ __forceinline__ void wait_phase_done(const MegaParams& P, int p, uint32_t target) { wait_counter(P.done + p, target, P.err, 4); }

// ---------------------------------------------------------------------------------------------
// GEMV phase, consumer side: the eight warps split K inside each 32 KB stage; per-lane partial
// sums of a tile go to the epilogue warp through shared memory.
// ---------------------------------------------------------------------------------------------
template <typename WT>
__device__ __forceinline__ void consume_tiles(const int kind, const int rows, const int K, const Smem sm, int n_stages, int& s,
                                              uint32_t& par, int& ps, uint32_t& ppar, int* err) {
    constexpr int VEC = Vec<WT>::N;
    constexpr int KC = kSegBytes / (int)sizeof(WT);
    constexpr int SL = 32 * VEC;  // K elements one warp covers per stage
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nmat = kind == MK_W13 ? 2 : 1;
    const int n_tiles = rows / (kNSeg / nmat);
    const WT* act = reinterpret_cast<const WT*>(sm.act);
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        float acc[kNSeg];
#pragma unroll
        for (int i = 0; i < kNSeg; i++) acc[i] = 0.f;
        for (int k0 = 0; k0 < K; k0 += KC) {
            mbar_wait(&sm.full[s], par, err);
            const WT* st = reinterpret_cast<const WT*>(sm.ring + (size_t)s * kStageBytes);
            const int kk = warp * SL + lane * VEC;
            if (k0 + kk < K) {
                float af[VEC];
                unpack<WT>(*reinterpret_cast<const uint4*>(act + k0 + kk), af);
#pragma unroll
                for (int i = 0; i < kNSeg; i++) {
                    float wf[VEC];
                    unpack<WT>(*reinterpret_cast<const uint4*>(st + (size_t)i * KC + kk), wf);
#pragma unroll
                    for (int e = 0; e < VEC; e++) acc[i] = fmaf(wf[e], af[e], acc[i]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.empty[s]);
            if (++s == n_stages) { s = 0; par ^= 1u; }
        }
        mbar_wait(&sm.pempty[ps], ppar ^ 1u, err);
        float* mine = sm.partial + (size_t)ps * kNSeg * kConsumers + tid;
#pragma unroll
        for (int i = 0; i < kNSeg; i++) mine[i * kConsumers] = acc[i];
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.pfull[ps]);
        if (++ps == kPartialDepth) { ps = 0; ppar ^= 1u; }
    }
}

// Prologue of a GEMV phase: build the activation row in shared memory.
template <typename WT>
__device__ __noinline__ void build_activation(const MegaParams& P, const MegaPhase& ph, const Smem& sm, uint32_t seq_base, int pi,
                                              uint32_t done_target) {
    constexpr int VEC = Vec<WT>::N;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = ph.K;
    WT* act = reinterpret_cast<WT*>(sm.act);
    if (ph.kind == MK_PROJ) {
        // written by other CTAs during this launch: read through L2
        const uint4* src = reinterpret_cast<const uint4*>(ph.vec_in);
        uint4* dst = reinterpret_cast<uint4*>(act);
        for (int i = tid; i < K / VEC; i += kConsumers) dst[i] = __ldcg(src + i);
        consumer_sync();
        return;
    }
    // residual add + RMSNorm (src/transformer.rs:476-480) + cast
    const float* xin = ph.x_in;
    if (ph.use_tok) xin += (int64_t)(P.scalars[0]) * K;
    const int per = ((K + (int)gridDim.x - 1) / (int)gridDim.x + 3) & ~3;
    const int s0 = min(K, (int)blockIdx.x * per), s1 = min(K, s0 + per);
    float ss = 0.f;
    if (ph.in_seq != 0) {
        // This CTA owns rows [s0, s1) of the residual: sum the partial sums of that slice over the
        // ranks in rank order, round where the reference rounds the projection's output, add the
        // residual, publish; then read the whole new residual from the published entries.
        const uint32_t seq = seq_base + (uint32_t)ph.in_seq;
        const uint2* inbox = reinterpret_cast<const uint2*>(P.xbuf + ph.inbox_off);
        for (int i = s0 + tid; i < s1; i += kConsumers) {
            float part[RLB_MAX_TP];
            ll_gather<RLB_MAX_TP>(inbox + i, (size_t)K, P.tp, seq, part, P.err);
            float sum = part[0];
#pragma unroll
            for (int q = 1; q < RLB_MAX_TP; q++)
                if (q < P.tp) sum += part[q];
            if (P.f16) sum = round_f16(sum);
            ph.x_out[i] = xin[i] + sum;
        }
        // publish the slice: plain stores, a device-scope fence and one count per CTA; readers poll
        // a single counter instead of every entry (thousands of polling threads would starve the
        // very stores they wait for)
        __threadfence();
        consumer_sync();
        if (tid == 0) atomicAdd(P.xready + pi, 1u);
        wait_counter(P.xready + pi, done_target, P.err, 5);
        for (int i = tid * 4; i < K; i += kConsumers * 4) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(ph.x_out + i));
            *reinterpret_cast<float4*>(sm.tmp + i) = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        // first layer: the row comes straight from the embedding table
        for (int i = tid; i < K; i += kConsumers) {
            const float v = xin[i];
            sm.tmp[i] = v;
            if (i >= s0 && i < s1) ph.x_out[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) sm.red[warp] = ss;
    consumer_sync();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; w++) tot += sm.red[w];
    const float scale = 1.0f / sqrtf(tot / (float)K + P.eps);
    for (int i = tid; i < K; i += kConsumers) act[i] = cast_to<WT>(__fmul_rn(__fmul_rn(sm.tmp[i], scale), ph.gain[i]));
    consumer_sync();
}

// ---------------------------------------------------------------------------------------------
// Attention phase (consumer warps): one (head, split) item at a time, a warp per position with an
// online softmax, as attn_decode_fast_kernel in attention.cu.
// ---------------------------------------------------------------------------------------------
template <typename CT, int DPL> struct RowVec;
template <> struct RowVec<__half, 4> { typedef uint2 T; };
template <> struct RowVec<__half, 2> { typedef uint32_t T; };
template <> struct RowVec<float, 4> { typedef uint4 T; };
template <> struct RowVec<float, 2> { typedef uint2 T; };
template <typename CT, int DPL> __device__ __forceinline__ void row_unpack(const typename RowVec<CT, DPL>::T& v, float (&f)[DPL]);
template <> __device__ __forceinline__ void row_unpack<__half, 4>(const uint2& v, float (&f)[4]) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <> __device__ __forceinline__ void row_unpack<__half, 2>(const uint32_t& v, float (&f)[2]) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v));
    f[0] = a.x; f[1] = a.y;
}
template <> __device__ __forceinline__ void row_unpack<float, 4>(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void row_unpack<float, 2>(const uint2& v, float (&f)[2]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
}

template <typename CT, int HD>
__device__ __noinline__ void attention_phase(const MegaParams& P, const MegaPhase& ph, const Smem& sm) {
    constexpr int DPL = HD / 32;
    constexpr int PB = (sizeof(CT) * DPL >= 16) ? 4 : 8;  // positions per warp per batch (register budget)
    typedef typename RowVec<CT, DPL>::T RV;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* w_m = sm.tmp;              // [kCW]
    float* w_l = sm.tmp + kCW;        // [kCW]
    float* w_o = sm.tmp + 2 * kCW;    // [kCW][HD]
    unsigned int* ticket = reinterpret_cast<unsigned int*>(sm.tmp + 2 * kCW + kCW * HD);
    const int T = P.scalars[1] + 1;
    int chunk = (T + P.n_split - 1) / P.n_split;
    chunk = (chunk + 63) / 64 * 64;
    const int active = (T + chunk - 1) / chunk;
    const float scale = 1.0f / sqrtf((float)HD);  // src/transformer.rs:770
    for (int item = blockIdx.x; item < P.heads * active; item += gridDim.x) {
        const int head = item / active, split = item - head * active;
        const int t0 = split * chunk, t1 = min(T, t0 + chunk);
        const CT* kbase = reinterpret_cast<const CT*>(ph.kcache) + (int64_t)head * P.max_seq * HD + lane * DPL;
        const CT* vbase = reinterpret_cast<const CT*>(ph.vcache) + (int64_t)head * P.max_seq * HD + lane * DPL;
        float q[DPL];
#pragma unroll
        for (int d = 0; d < DPL; d++) q[d] = __ldcg(P.qbuf + head * HD + lane * DPL + d);
        float m = -FLT_MAX, l = 0.f, acc[DPL];
#pragma unroll
        for (int d = 0; d < DPL; d++) acc[d] = 0.f;
        for (int tb = t0 + warp; tb < t1; tb += kCW * PB) {
            RV kv[PB], vv[PB];
#pragma unroll
            for (int j = 0; j < PB; j++) {
                const int t = tb + j * kCW;
                if (t < t1) {
                    kv[j] = *reinterpret_cast<const RV*>(kbase + (int64_t)t * HD);
                    vv[j] = *reinterpret_cast<const RV*>(vbase + (int64_t)t * HD);
                }
            }
            float sc[PB];
#pragma unroll
            for (int j = 0; j < PB; j++) {
                float dot = 0.f;
                if (tb + j * kCW < t1) {
                    float kf[DPL];
                    row_unpack<CT, DPL>(kv[j], kf);
#pragma unroll
                    for (int d = 0; d < DPL; d++) dot = fmaf(q[d], kf[d], dot);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                sc[j] = (tb + j * kCW < t1) ? dot * scale : -FLT_MAX;
            }
            float bm = sc[0];
#pragma unroll
            for (int j = 1; j < PB; j++) bm = fmaxf(bm, sc[j]);
            const float m_new = fmaxf(m, bm);
            const float rescale = expf(m - m_new);
            l *= rescale;
#pragma unroll
            for (int d = 0; d < DPL; d++) acc[d] *= rescale;
#pragma unroll
            for (int j = 0; j < PB; j++) {
                if (tb + j * kCW < t1) {
                    const float p = expf(sc[j] - m_new);
                    l += p;
                    float vf[DPL];
                    row_unpack<CT, DPL>(vv[j], vf);
#pragma unroll
                    for (int d = 0; d < DPL; d++) acc[d] = fmaf(p, vf[d], acc[d]);
                }
            }
            m = m_new;
        }
        if (lane == 0) { w_m[warp] = m; w_l[warp] = l; }
#pragma unroll
        for (int d = 0; d < DPL; d++) w_o[warp * HD + lane * DPL + d] = acc[d];
        consumer_sync();
        float M = w_m[0];
#pragma unroll
        for (int w = 1; w < kCW; w++) M = fmaxf(M, w_m[w]);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < kCW; w++) L += w_l[w] * expf(w_m[w] - M);
        CT* out = reinterpret_cast<CT*>(P.obuf) + head * HD;
        float o = 0.f;
        const int c = tid;
        if (c < HD) {
#pragma unroll
            for (int w = 0; w < kCW; w++) o += w_o[w * HD + c] * expf(w_m[w] - M);
        }
        if (active == 1) {
            if (c < HD) out[c] = cast_to<CT>(o / L);
        } else {
            float* rec = P.attn_scratch + ((int64_t)head * P.n_split + split) * (HD + 2);
            if (c < HD) rec[c] = o;
            if (c == 0) { rec[HD] = M; rec[HD + 1] = L; }
            __threadfence();
            consumer_sync();
            if (tid == 0) *ticket = atomicAdd(P.attn_counters + head, 1u);
            consumer_sync();
            if (*ticket == (unsigned)(active - 1)) {
                __threadfence();
                const float* recs = P.attn_scratch + (int64_t)head * P.n_split * (HD + 2);
                float GM = -FLT_MAX;
                for (int s2 = 0; s2 < active; s2++) GM = fmaxf(GM, __ldcg(recs + s2 * (HD + 2) + HD));
                float GL = 0.f;
                for (int s2 = 0; s2 < active; s2++) GL += __ldcg(recs + s2 * (HD + 2) + HD + 1) * expf(__ldcg(recs + s2 * (HD + 2) + HD) - GM);
                if (c < HD) {
                    float go = 0.f;
                    for (int s2 = 0; s2 < active; s2++) go += __ldcg(recs + s2 * (HD + 2) + c) * expf(__ldcg(recs + s2 * (HD + 2) + HD) - GM);
                    out[c] = cast_to<CT>(go / GL);
                }
                if (tid == 0) P.attn_counters[head] = 0;
            }
        }
        consumer_sync();  // the merge area is reused by the next item
    }
}

// Greedy choice over the pushed logits entries (TokenSampler with top_k 1, src/token_sampler.rs:20-28):
// the lowest id among equal maxima. Runs on CTA 0's consumer warps.
__device__ __noinline__ void argmax_phase(const MegaParams& P, const Smem& sm, uint32_t seq_base) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t seq = seq_base + P.seq_stride;  // the head is the last exchange of the step
    const uint2* ll = reinterpret_cast<const uint2*>(P.xbuf + P.logits_off);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int base = tid; base < P.vocab; base += 8 * kConsumers) {
        float v8[8];
        const int cnt = min(8, (P.vocab - base + kConsumers - 1) / kConsumers);
        ll_gather<8>(ll + base, (size_t)kConsumers, cnt, seq, v8, P.err);
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (j < cnt) {
                const int i = base + j * kConsumers;
                P.logits[i] = v8[j];
                if (v8[j] > bv || (v8[j] == bv && i < bi)) { bv = v8[j]; bi = i; }
            }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    float* sv = sm.tmp;
    int* si = reinterpret_cast<int*>(sm.tmp + kCW);
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    consumer_sync();
    if (tid == 0) {
        bv = sv[0]; bi = si[0];
        for (int w = 1; w < kCW; w++)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        if (bi == 0x7fffffff) bi = 0;
        int32_t* sc = P.scalars;
        if (P.advance) {
            sc[0] = bi;
            sc[1] = sc[1] + 1;
            const int st = sc[2];
            if (st < P.tokens_cap) P.tokens_out[st] = bi;
            sc[2] = st + 1;
        } else {
            sc[3] = bi;
        }
        sc[4] = sc[4] + 1;  // exchange epoch
        sc[5] = sc[5] + 1;  // launches of this kernel
    }
}

__global__ void __launch_bounds__(kMegaThreads, 1) decode_mega_kernel(const MegaParams P) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem sm;
    sm.ring = smem_raw;
    unsigned char* p = smem_raw + (size_t)P.n_stages * kStageBytes;
    sm.act = p; p += P.act_bytes;
    sm.tmp = reinterpret_cast<float*>(p); p += P.tmp_bytes;
    sm.partial = reinterpret_cast<float*>(p); p += sizeof(float) * kPartialDepth * kNSeg * kConsumers;
    sm.red = reinterpret_cast<float*>(p); p += sizeof(float) * kCW;
    p = reinterpret_cast<unsigned char*>(((uintptr_t)p + 7) & ~(uintptr_t)7);
    sm.full = reinterpret_cast<uint64_t*>(p);
    sm.empty = sm.full + kMaxStages;
    sm.pfull = sm.empty + kMaxStages;
    sm.pempty = sm.pfull + kPartialDepth;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < P.n_stages; s++) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kCW);
        }
        for (int s = 0; s < kPartialDepth; s++) {
            mbar_init(&sm.pfull[s], kCW);
            mbar_init(&sm.pempty[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // values fixed for the whole launch (CTA 0 advances them only after the last phase, which no
    // CTA can reach before every CTA has passed its first wait)
    const uint32_t seq_base = (uint32_t)(P.scalars[4] - 1) * P.seq_stride;        // + index of the exchange (1-based)
    const uint32_t done_target = ((uint32_t)P.scalars[5] + 1u) * gridDim.x;       // completion counters are monotonic
    const int wesz = P.f16 ? 2 : 4;

    if (warp == kCW) {
        // ================================ producer warp ==================================
        int s = 0;
        uint32_t par = 0;
        for (int pi = 0; pi < P.n_phases; pi++) {
            const MegaPhase& ph = P.phases[pi];
            if (ph.kind == MK_ATTN || ph.kind == MK_ARGMAX) continue;
            const int esz = ph.kind == MK_HEAD ? 4 : wesz;
            const int nmat = ph.kind == MK_W13 ? 2 : 1;
            const int RB = kNSeg / nmat;
            const int KC = kSegBytes / esz;
            const int n_tiles = ph.rows / RB;
            const int phK = ph.K;
            const int m = lane / RB, r = lane - m * RB;
            const char* wbase = reinterpret_cast<const char*>(m == 0 ? ph.W : ph.W2);
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const int row0 = tile * RB;
                for (int k0 = 0; k0 < phK; k0 += KC) {
                    mbar_wait(&sm.empty[s], par ^ 1u, P.err);
                    const uint32_t nbytes = (uint32_t)min(KC, phK - k0) * esz;
                    if (lane == 0) mbar_expect_tx(&sm.full[s], nbytes * kNSeg);
                    __syncwarp();
                    if (lane < kNSeg)
                        bulk_g2s(sm.ring + (size_t)s * kStageBytes + (size_t)lane * kSegBytes,
                                 wbase + ((int64_t)(row0 + r) * phK + k0) * esz, nbytes, &sm.full[s]);
                    if (++s == P.n_stages) { s = 0; par ^= 1u; }
                }
            }
        }
        return;
    }

    if (warp == kCW + 1) {
        // ================================ epilogue warp ==================================
        int ps = 0;
        uint32_t ppar = 0;
        for (int pi = 0; pi < P.n_phases; pi++) {
            const MegaPhase& ph = P.phases[pi];
            if (ph.kind == MK_ATTN || ph.kind == MK_ARGMAX) continue;
            const int nmat = ph.kind == MK_W13 ? 2 : 1;
            const int RB = kNSeg / nmat;
            const int n_tiles = ph.rows / RB;
            const bool half_out = P.f16 && ph.kind != MK_HEAD;
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const int row0 = tile * RB;
                mbar_wait(&sm.pfull[ps], ppar, P.err);
                const float* pp = sm.partial + (size_t)ps * kNSeg * kConsumers;
                float tot[kNSeg];
#pragma unroll
                for (int i = 0; i < kNSeg; i++) {
                    float t = 0.f;
#pragma unroll
                    for (int w = 0; w < kCW; w++) t += pp[i * kConsumers + w * 32 + lane];  // fixed order
                    tot[i] = warp_sum(t);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.pempty[ps]);
                if (++ps == kPartialDepth) { ps = 0; ppar ^= 1u; }
                auto total = [&](int i) {
                    float t = tot[0];
#pragma unroll
                    for (int q = 1; q < kNSeg; q++) t = (i == q) ? tot[q] : t;
                    return t;
                };
                if (ph.kind == MK_PROJ || ph.kind == MK_HEAD) {
                    if (lane < RB) {  // tagged partial sum into every rank's inbox
                        const float v = total(lane);
                        const uint32_t seq = seq_base + (uint32_t)ph.out_seq;
                        for (int d = 0; d < P.tp; d++)
                            ll_store(reinterpret_cast<uint2*>(P.peer_xbuf[d] + ph.outbox_off) + ph.out_offset + row0 + lane, v, seq);
                    }
                } else if (ph.kind == MK_W13) {
                    if (lane < RB) {  // src/transformer.rs:551-565
                        float a1 = total(lane), a3 = total(RB + lane);
                        if (half_out) { a1 = round_f16(a1); a3 = round_f16(a3); }
                        const float sg = a1 / (1.0f + expf(-a1));
                        const float g = __fmul_rn(sg, a3);
                        if (half_out) reinterpret_cast<__half*>(ph.out)[row0 + lane] = __float2half_rn(g);
                        else reinterpret_cast<float*>(ph.out)[row0 + lane] = g;
                    }
                } else {  // MK_QKV: rounding, RoPE, q buffer and KV append (src/transformer.rs:719-761, :823-856)
                    if (lane < RB / 2) {
                        const int pos = P.scalars[1];
                        const int row = row0 + 2 * lane;
                        const int sec = row / P.nq, rr = row - sec * P.nq;
                        const int head = rr / P.hd, c = rr - head * P.hd;
                        float re = total(2 * lane), im = total(2 * lane + 1);
                        if (half_out) { re = round_f16(re); im = round_f16(im); }
                        const float* f = P.rope + ((int64_t)pos * (P.hd / 2) + (c >> 1)) * 2;
                        const float fr = f[0], fi = f[1];
                        const float o_re = __fsub_rn(__fmul_rn(re, fr), __fmul_rn(im, fi));
                        const float o_im = __fadd_rn(__fmul_rn(re, fi), __fmul_rn(im, fr));
                        if (sec == 0) {
                            P.qbuf[rr] = o_re;
                            P.qbuf[rr + 1] = o_im;
                        } else {
                            const int64_t idx = ((int64_t)head * P.max_seq + pos) * P.hd + c;
                            const float a0 = sec == 1 ? o_re : re, a1 = sec == 1 ? o_im : im;
                            if (half_out) {
                                __half* dst = reinterpret_cast<__half*>(sec == 1 ? ph.kcache : ph.vcache) + idx;
                                dst[0] = __float2half_rn(a0);
                                dst[1] = __float2half_rn(a1);
                            } else {
                                float* dst = reinterpret_cast<float*>(sec == 1 ? ph.kcache : ph.vcache) + idx;
                                dst[0] = a0;
                                dst[1] = a1;
                            }
                        }
                    }
                }
            }
            if (ph.kind == MK_QKV || ph.kind == MK_W13) {
                // a later phase reads this phase's plain stores: publish them, then count this CTA in
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(P.done + pi, 1u);
            }
        }
        return;
    }

    // ==================================== consumer warps =====================================
    int s = 0, ps = 0;
    uint32_t par = 0, ppar = 0;
    for (int pi = 0; pi < P.n_phases; pi++) {
        const MegaPhase& ph = P.phases[pi];
        consumer_sync();  // every warp is done with the previous phase's activation row and scratch
        if (P.trace != nullptr && blockIdx.x == 0 && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            P.trace[pi] = t;
        }
        if (ph.kind == MK_ARGMAX) {
            if (blockIdx.x == 0) argmax_phase(P, sm, seq_base);
            continue;
        }
        if (ph.wait_phase >= 0) wait_phase_done(P, ph.wait_phase, done_target);
        if (ph.kind == MK_ATTN) {
            if (P.f16) {
                if (P.hd == 128) attention_phase<__half, 128>(P, ph, sm);
                else attention_phase<__half, 64>(P, ph, sm);
            } else {
                if (P.hd == 128) attention_phase<float, 128>(P, ph, sm);
                else attention_phase<float, 64>(P, ph, sm);
            }
            __threadfence();
            consumer_sync();
            if (tid == 0) atomicAdd(P.done + pi, 1u);
            continue;
        }
        if (P.f16 && ph.kind != MK_HEAD) {
            build_activation<__half>(P, ph, sm, seq_base, pi, done_target);
            consume_tiles<__half>(ph.kind, ph.rows, ph.K, sm, P.n_stages, s, par, ps, ppar, P.err);
        } else {
            build_activation<float>(P, ph, sm, seq_base, pi, done_target);
            consume_tiles<float>(ph.kind, ph.rows, ph.K, sm, P.n_stages, s, par, ps, ppar, P.err);
        }
    }
    if (P.trace != nullptr && blockIdx.x == 0 && tid == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        P.trace[P.n_phases] = t;
    }
}

}  // namespace

size_t mega_smem_bytes(const MegaParams& P) {
    return (size_t)P.n_stages * kStageBytes + P.act_bytes + P.tmp_bytes + sizeof(float) * kPartialDepth * kNSeg * kConsumers +
           sizeof(float) * kCW + 16 + (2 * kMaxStages + 2 * kPartialDepth) * sizeof(uint64_t);
}

// Chooses the ring depth for the given activation / scratch sizes; 0 if nothing fits.
int mega_pick_stages(size_t act_bytes, size_t tmp_bytes) {
    MegaParams P;
    P.act_bytes = (int)act_bytes;
    P.tmp_bytes = (int)tmp_bytes;
    for (int s = kMaxStages; s >= 2; s--) {
        P.n_stages = s;
        if (mega_smem_bytes(P) <= 224 * 1024) return s;
    }
    return 0;
}

int launch_decode_mega(rlb_ctx* ctx, const MegaParams& P) {
    const size_t smem = mega_smem_bytes(P);
    static bool set = false;
    if (!set) {
        RLB_CUDA(cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        set = true;
    }
    void* args[] = {const_cast<MegaParams*>(&P)};
    // cooperative: every CTA waits on every other CTA, so all of them must be resident
    RLB_CUDA(cudaLaunchCooperativeKernel((const void*)decode_mega_kernel, dim3(ctx->sm_count), dim3(kMegaThreads), args, smem, ctx->stream));
    count_launch(ctx);
    return RLB_OK;
}

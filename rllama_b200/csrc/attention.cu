// Attention over the KV cache: the per-head part of Attention::forward
// (src/transformer.rs:727-781): scores = q * K / sqrt(head_dim), causal mask for multi-token
// calls (Tensor::full_triu, src/tensor.rs:496-508), softmax (src/tensor.rs:479-494),
// out = P * V. Everything is f32 arithmetic on cache values widened from their storage
// dtype, as in the reference (:762-766).
//
// The reference's softmax does not subtract the row maximum; the kernels here do (and the
// split-T decode kernel combines partial results with the usual rescaling). That is the same
// function of the inputs, evaluated without overflow; results differ by f32 rounding only.
//
// Cache layout in HBM: per layer, K and V are [head][position][head_dim] (position-major,
// one 128/256-byte row per position) instead of the reference's head_dim x max_seq_len per
// head, so that one position's vector is a single coalesced read.
#include "internal.h"

#include <atomic>
#include <cfloat>
#include <cstdlib>
#include <cstdio>

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <typename T> struct CVec;
template <> struct CVec<__half> { static constexpr int N = 8; };
template <> struct CVec<float> { static constexpr int N = 4; };

template <typename T> __device__ __forceinline__ void unpack16(const uint4& v, float* f);
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template <> __device__ __forceinline__ void unpack16<float>(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}

template <typename T> __device__ __forceinline__ T cast_out(float v);
template <> __device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float cast_out<float>(float v) { return v; }

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int w = 1; w < kWarps; w++) t = fmaxf(t, red[w]);
    __syncthreads();
    return t;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; w++) t += red[w];
    __syncthreads();
    return t;
}

// One query row against positions [t0, t1) of one head. Shared memory: q[hd], sc[t1-t0],
// acc[kThreads/tpp][hd]. Produces the unnormalised output o[hd] (in shared `o_out`), the
// running maximum m and the sum l = sum exp(s - m).
template <typename CT>
__device__ void attend_range(const float* __restrict__ q_sh, const CT* __restrict__ kbase, const CT* __restrict__ vbase,
                             int hd, int t0, int t1, float scale, float* sc, float* accbuf, float* red, float* o_out,
                             float& m_out, float& l_out) {
    constexpr int VEC = CVec<CT>::N;
    const int tid = threadIdx.x;
    const int n = t1 - t0;
    // ---- scores: a group of (hd / VEC) threads... 8 lanes per position, each lane hd/8 dims ----
    {
        const int lpp = 8;                    // lanes per position
        const int dpl = hd / lpp;             // dims per lane (multiple of VEC)
        const int sub = tid & (lpp - 1);
        const int slot = tid / lpp;           // position slot within an iteration
        const int ppi = kThreads / lpp;       // positions per iteration
        for (int i = slot; i < ((n + ppi - 1) / ppi) * ppi; i += ppi) {
            float dot = 0.f;
            if (i < n) {
                const CT* kp = kbase + (int64_t)(t0 + i) * hd + sub * dpl;
                const float* qp = q_sh + sub * dpl;
                for (int d = 0; d < dpl; d += VEC) {
                    float kf[VEC];
                    unpack16<CT>(*reinterpret_cast<const uint4*>(kp + d), kf);
#pragma unroll
                    for (int e = 0; e < VEC; e++) dot = fmaf(qp[d + e], kf[e], dot);
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            if (sub == 0 && i < n) sc[i] = dot * scale;
        }
    }
    __syncthreads();
    // ---- softmax pieces ----
    float m = -FLT_MAX;
    for (int i = tid; i < n; i += kThreads) m = fmaxf(m, sc[i]);
    m = block_reduce_max(m, red);
    float l = 0.f;
    for (int i = tid; i < n; i += kThreads) {
        const float p = expf(sc[i] - m);
        sc[i] = p;
        l += p;
    }
    l = block_reduce_sum(l, red);
    // ---- o = sum_t p[t] * V[t] : (hd / VEC) threads per position ----
    {
        const int tpp = hd / VEC;
        const int sub = tid % tpp;
        const int slot = tid / tpp;
        const int ppi = kThreads / tpp;
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) acc[e] = 0.f;
        if (slot < ppi) {
            for (int i = slot; i < n; i += ppi) {
                float vf[VEC];
                unpack16<CT>(*reinterpret_cast<const uint4*>(vbase + (int64_t)(t0 + i) * hd + sub * VEC), vf);
                const float p = sc[i];
#pragma unroll
                for (int e = 0; e < VEC; e++) acc[e] = fmaf(p, vf[e], acc[e]);
            }
#pragma unroll
            for (int e = 0; e < VEC; e++) accbuf[slot * hd + sub * VEC + e] = acc[e];
        }
        __syncthreads();
        for (int c = tid; c < hd; c += kThreads) {
            float s = 0.f;
            for (int j = 0; j < ppi; j++) s += accbuf[j * hd + c];
            o_out[c] = s;
        }
        __syncthreads();
    }
    m_out = m;
    l_out = l;
}

// grid (heads, n_split). Scratch record per (head, split): o[hd], m, l.
template <typename CT>
__global__ void __launch_bounds__(kThreads) attn_decode_kernel(const AttnDecodeArgs a) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[kWarps];
    __shared__ unsigned int ticket_sh;
    // programmatic dependent launch: let the next kernel (the wo projection) start streaming its
    // weights now; wait for the q/k/v kernel before touching its outputs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int hd = a.hd, head = blockIdx.x, split = blockIdx.y, ns = a.n_split;
    const int T = (a.pos_ptr ? *a.pos_ptr : a.pos_value) + 1;
    int chunk = (T + ns - 1) / ns;
    chunk = (chunk + 31) & ~31;
    const int t0 = min(T, split * chunk), t1 = min(T, t0 + chunk);
    float* q_sh = sm;                 // hd
    float* o_sh = q_sh + hd;          // hd
    float* accbuf = o_sh + hd;        // (kThreads / (hd / VEC)) * hd  <= kThreads * VEC
    float* sc = accbuf + kThreads * CVec<CT>::N;  // chunk (sized for max_seq / 1)
    for (int c = threadIdx.x; c < hd; c += kThreads) q_sh[c] = a.q[head * hd + c];
    __syncthreads();
    const CT* kbase = reinterpret_cast<const CT*>(a.kcache) + (int64_t)head * a.max_seq * hd;
    const CT* vbase = reinterpret_cast<const CT*>(a.vcache) + (int64_t)head * a.max_seq * hd;
    const float scale = 1.0f / sqrtf((float)hd);  // src/transformer.rs:770
    float m = -FLT_MAX, l = 0.f;
    if (t1 > t0) {
        attend_range<CT>(q_sh, kbase, vbase, hd, t0, t1, scale, sc, accbuf, red, o_sh, m, l);
    } else {
        for (int c = threadIdx.x; c < hd; c += kThreads) o_sh[c] = 0.f;
        __syncthreads();
    }
    CT* out = reinterpret_cast<CT*>(a.out) + head * hd;
    if (ns == 1) {
        for (int c = threadIdx.x; c < hd; c += kThreads) out[c] = cast_out<CT>(o_sh[c] / l);
        return;
    }
    float* rec = a.scratch + ((int64_t)head * ns + split) * (hd + 2);
    for (int c = threadIdx.x; c < hd; c += kThreads) rec[c] = o_sh[c];
    if (threadIdx.x == 0) { rec[hd] = m; rec[hd + 1] = l; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket_sh = atomicAdd(a.counters + head, 1u);
    __syncthreads();
    if (ticket_sh != (unsigned)(ns - 1)) return;
    // last CTA of this head: combine the partial results
    __threadfence();
    const float* recs = a.scratch + (int64_t)head * ns * (hd + 2);
    float M = -FLT_MAX;
    for (int s = 0; s < ns; s++) M = fmaxf(M, __ldcg(recs + s * (hd + 2) + hd));
    float L = 0.f;
    for (int s = 0; s < ns; s++) L += __ldcg(recs + s * (hd + 2) + hd + 1) * expf(__ldcg(recs + s * (hd + 2) + hd) - M);
    for (int c = threadIdx.x; c < hd; c += kThreads) {
        float o = 0.f;
        for (int s = 0; s < ns; s++) o += __ldcg(recs + s * (hd + 2) + c) * expf(__ldcg(recs + s * (hd + 2) + hd) - M);
        out[c] = cast_out<CT>(o / L);
    }
    if (threadIdx.x == 0) a.counters[head] = 0;  // ready for the next launch
}

// Prefill: grid (heads, n); one CTA per (head, query row i) attends to positions 0..start_pos+i.
template <typename CT>
__global__ void __launch_bounds__(kThreads) attn_prefill_kernel(const AttnPrefillArgs a) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[kWarps];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int hd = a.hd, head = blockIdx.x, i = blockIdx.y;
    const int T = a.start_pos + i + 1;  // mask: col >= row + start_pos + 1 is -inf
    float* q_sh = sm;
    float* o_sh = q_sh + hd;
    float* accbuf = o_sh + hd;
    float* sc = accbuf + kThreads * CVec<CT>::N;
    for (int c = threadIdx.x; c < hd; c += kThreads) q_sh[c] = a.q[(int64_t)i * a.q_ld + head * hd + c];
    __syncthreads();
    const CT* kbase = reinterpret_cast<const CT*>(a.kcache) + (int64_t)head * a.max_seq * hd;
    const CT* vbase = reinterpret_cast<const CT*>(a.vcache) + (int64_t)head * a.max_seq * hd;
    const float scale = 1.0f / sqrtf((float)hd);
    float m, l;
    attend_range<CT>(q_sh, kbase, vbase, hd, 0, T, scale, sc, accbuf, red, o_sh, m, l);
    CT* out = reinterpret_cast<CT*>(a.out) + (int64_t)i * a.heads * hd + head * hd;
    for (int c = threadIdx.x; c < hd; c += kThreads) out[c] = cast_out<CT>(o_sh[c] / l);
}

// Prefill for head_dim 64 / 128, tiled: one CTA per (head, block of 64 query rows). Tiles of 32 cache
// positions are staged in shared memory once (as f32) and shared by the 64 query rows, so the cache is
// read n / 64 times instead of n times. Scores and P.V are two small f32 FMA tile products (no tensor
// cores: q after RoPE and the softmax weights are f32 values in the reference, and rounding them to a
// tensor-core input format would add a rounding point it does not have); the softmax runs online with a
// running row maximum. Thread (r, g) = (tid / 8, tid % 8) owns the query rows r and r + 32, the score
// columns g, g + 8, g + 16, g + 24 of a tile and the output columns 4 g + 32 j ... + 3: every K or V
// value read from shared memory feeds two rows (shared-memory bandwidth, not FMA rate, bounds the kernel).
constexpr int kQB = 64;   // query rows per CTA
constexpr int kTB = 32;   // cache positions per tile

template <typename CT, int HD>
__global__ void __launch_bounds__(256) attn_prefill_tiled_kernel(const AttnPrefillArgs a) {
    constexpr int LD = HD + 4;             // padded row stride: conflict-free float4 reads
    constexpr int NJ = HD / 32;            // float4 output groups per thread and row
    constexpr int PL = kTB + 1;
    extern __shared__ __align__(16) float sm[];
    float* q_s = sm;                       // [kQB][LD]
    float* k_s = q_s + kQB * LD;           // [kTB][LD]
    float* v_s = k_s + kTB * LD;           // [kTB][HD]
    float* p_s = v_s + kTB * HD;           // [kQB][PL]
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int head = blockIdx.x, i0 = blockIdx.y * kQB;
    const int tid = threadIdx.x, r = tid >> 3, g = tid & 7;
    const int rows = min(kQB, a.n - i0);
    for (int e = tid; e < kQB * (HD / 4); e += 256) {
        const int rr = e / (HD / 4), c4 = e % (HD / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rr < rows) v = *reinterpret_cast<const float4*>(a.q + (int64_t)(i0 + rr) * a.q_ld + head * HD + c4 * 4);
        *reinterpret_cast<float4*>(q_s + rr * LD + c4 * 4) = v;
    }
    const CT* kbase = reinterpret_cast<const CT*>(a.kcache) + (int64_t)head * a.max_seq * HD;
    const CT* vbase = reinterpret_cast<const CT*>(a.vcache) + (int64_t)head * a.max_seq * HD;
    const float scale = 1.0f / sqrtf((float)HD);  // src/transformer.rs:770
    // row r + 32 h attends to the positions below limit[h] (src/tensor.rs:496-508)
    const int limit[2] = {a.start_pos + i0 + r + 1, a.start_pos + i0 + r + 33};
    const int t_end = a.start_pos + i0 + rows;    // the last row's limit
    float m[2] = {-FLT_MAX, -FLT_MAX}, l[2] = {0.f, 0.f};
    float4 o[2][NJ];
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int j = 0; j < NJ; j++) o[h][j] = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int t0 = 0; t0 < t_end; t0 += kTB) {
        __syncthreads();  // the previous tile has been consumed (and q_s is complete)
        for (int e = tid; e < kTB * (HD / 4); e += 256) {
            const int tt = e / (HD / 4), c4 = e % (HD / 4);
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (t0 + tt < t_end) {
                const CT* kp = kbase + (int64_t)(t0 + tt) * HD + c4 * 4;
                const CT* vp = vbase + (int64_t)(t0 + tt) * HD + c4 * 4;
                if constexpr (sizeof(CT) == 2) {
                    const uint2 kr = *reinterpret_cast<const uint2*>(kp), vr = *reinterpret_cast<const uint2*>(vp);
                    const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kr.x)), k1 = __half22float2(*reinterpret_cast<const __half2*>(&kr.y));
                    const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&vr.x)), v1 = __half22float2(*reinterpret_cast<const __half2*>(&vr.y));
                    kv = make_float4(k0.x, k0.y, k1.x, k1.y);
                    vv = make_float4(v0.x, v0.y, v1.x, v1.y);
                } else {
                    kv = *reinterpret_cast<const float4*>(kp);
                    vv = *reinterpret_cast<const float4*>(vp);
                }
            }
            *reinterpret_cast<float4*>(k_s + tt * LD + c4 * 4) = kv;
            *reinterpret_cast<float4*>(v_s + tt * HD + c4 * 4) = vv;
        }
        __syncthreads();
        // scores of rows r, r + 32 against the tile's positions g, g + 8, g + 16, g + 24
        float s4[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
        for (int d = 0; d < HD; d += 4) {
            const float4 q0 = *reinterpret_cast<const float4*>(q_s + r * LD + d);
            const float4 q1 = *reinterpret_cast<const float4*>(q_s + (r + 32) * LD + d);
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float4 kv = *reinterpret_cast<const float4*>(k_s + (g + 8 * c) * LD + d);
                s4[0][c] = fmaf(q0.x, kv.x, s4[0][c]); s4[0][c] = fmaf(q0.y, kv.y, s4[0][c]); s4[0][c] = fmaf(q0.z, kv.z, s4[0][c]); s4[0][c] = fmaf(q0.w, kv.w, s4[0][c]);
                s4[1][c] = fmaf(q1.x, kv.x, s4[1][c]); s4[1][c] = fmaf(q1.y, kv.y, s4[1][c]); s4[1][c] = fmaf(q1.z, kv.z, s4[1][c]); s4[1][c] = fmaf(q1.w, kv.w, s4[1][c]);
            }
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float tmax = -FLT_MAX;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                s4[h][c] = (t0 + g + 8 * c < limit[h]) ? s4[h][c] * scale : -FLT_MAX;  // the causal mask
                tmax = fmaxf(tmax, s4[h][c]);
            }
            // the eight threads of a row sit in one warp, next to each other
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
            const float m_new = fmaxf(m[h], tmax);
            const float rescale = expf(m[h] - m_new);
            float psum = 0.f;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float pv = (t0 + g + 8 * c < limit[h]) ? expf(s4[h][c] - m_new) : 0.f;
                p_s[(r + 32 * h) * PL + g + 8 * c] = pv;
                psum += pv;
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            psum += __shfl_xor_sync(0xffffffffu, psum, 4);
            l[h] = l[h] * rescale + psum;
            m[h] = m_new;
#pragma unroll
            for (int j = 0; j < NJ; j++) { o[h][j].x *= rescale; o[h][j].y *= rescale; o[h][j].z *= rescale; o[h][j].w *= rescale; }
        }
        __syncwarp();  // a row's weights are written and read by the same warp
#pragma unroll 4
        for (int tt = 0; tt < kTB; tt++) {
            const float p0 = p_s[r * PL + tt], p1 = p_s[(r + 32) * PL + tt];
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const float4 vv = *reinterpret_cast<const float4*>(v_s + tt * HD + g * 4 + 32 * j);
                o[0][j].x = fmaf(p0, vv.x, o[0][j].x); o[0][j].y = fmaf(p0, vv.y, o[0][j].y); o[0][j].z = fmaf(p0, vv.z, o[0][j].z); o[0][j].w = fmaf(p0, vv.w, o[0][j].w);
                o[1][j].x = fmaf(p1, vv.x, o[1][j].x); o[1][j].y = fmaf(p1, vv.y, o[1][j].y); o[1][j].z = fmaf(p1, vv.z, o[1][j].z); o[1][j].w = fmaf(p1, vv.w, o[1][j].w);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int rr = r + 32 * h;
        if (rr < rows) {
            CT* out = reinterpret_cast<CT*>(a.out) + (int64_t)(i0 + rr) * a.heads * HD + head * HD;
            const float inv = 1.0f / l[h];
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const int c = g * 4 + 32 * j;
                out[c] = cast_out<CT>(o[h][j].x * inv); out[c + 1] = cast_out<CT>(o[h][j].y * inv);
                out[c + 2] = cast_out<CT>(o[h][j].z * inv); out[c + 3] = cast_out<CT>(o[h][j].w * inv);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Decode attention, low-latency form for head_dim 64 / 128: one warp per position, online softmax.
//
// A warp owns positions t0 + warp, t0 + warp + 8, ...; its 32 lanes split head_dim (DPL = HD / 32
// values each), so one position's K (or V) row is one coalesced warp load. K and V rows of a
// batch of PB positions are all requested before any arithmetic: one memory round trip per batch,
// none of it waiting on the softmax state. The running (max, sum, output) triple is per warp; the
// eight warps are merged once through shared memory, and the splits of a head are merged by the
// last CTA to arrive (as in the general kernel above). Only CTAs whose range is not empty take
// part, and a head with a single live split writes its output directly.
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

constexpr int kFastMinChunk = 64;  // positions per CTA at least (a multiple of kWarps)
constexpr int kMaxCluster = 16;    // splits of a head that may form one thread-block cluster (beyond 8: non-portable size)

__host__ __device__ inline int fast_chunk(int T, int ns) {
    int chunk = (T + ns - 1) / ns;
    chunk = (chunk + kFastMinChunk - 1) / kFastMinChunk * kFastMinChunk;
    return chunk;
}

// Distributed shared memory of a thread-block cluster: address of `addr` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t cluster_map(const void* addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(addr)), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_store(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// CL = false: the splits of a head meet through records in global memory and a ticket counter; the
// CTA that draws the last ticket merges them. CL = true: the n_split (<= 8) CTAs of a head form a
// thread-block cluster, send their partial result into the shared memory of the cluster's first
// CTA and meet at the cluster barrier: no global round trips on the way to the merged row.
// PB = positions per warp per batch (8 or 16): a CTA requests 8 PB cache rows of K and of V at once, and the
// first batch before the dependency wait; 16 is chosen when a CTA may own more than 64 positions (long contexts).
template <typename CT, int HD, bool CL, int PB>
__global__ void __launch_bounds__(kThreads) attn_decode_fast_kernel(const AttnDecodeArgs a) {
    constexpr int DPL = HD / 32;
    typedef typename RowVec<CT, DPL>::T RV;
    __shared__ float w_m[kWarps], w_l[kWarps];
    __shared__ float w_o[kWarps][HD];
    __shared__ unsigned int ticket_sh;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // A CTA's shared memory may be written by its cluster peers only once that CTA is running: every CTA
    // announces itself here and waits for all of them just before its first remote store.
    if constexpr (CL) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    // Before waiting for the projection kernel: the position (only the last kernel of a decode step
    // changes it) and the cache rows of earlier positions (written by earlier steps) are already
    // final, so the first batch of K and V rows is requested now and its latency overlaps the wait.
    const int head = blockIdx.x, split = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int T = (a.pos_ptr ? *a.pos_ptr : a.pos_value) + 1;
    const int chunk = fast_chunk(T, a.n_split);
    const int active = (T + chunk - 1) / chunk;  // splits with at least one position
    const bool work = split < active;
    if (!CL && !work) return;  // (in a cluster every CTA goes on to the barrier; its loops below are empty)
    const int t0 = split * chunk, t1 = min(T, t0 + chunk);
    const CT* kbase = reinterpret_cast<const CT*>(a.kcache) + (int64_t)head * a.max_seq * HD + lane * DPL;
    const CT* vbase = reinterpret_cast<const CT*>(a.vcache) + (int64_t)head * a.max_seq * HD + lane * DPL;
    RV kv[PB], vv[PB];
#pragma unroll
    for (int j = 0; j < PB; j++) {
        const int t = t0 + warp + j * kWarps;
        if (t < t1 && t < T - 1) {
            kv[j] = *reinterpret_cast<const RV*>(kbase + (int64_t)t * HD);
            vv[j] = *reinterpret_cast<const RV*>(vbase + (int64_t)t * HD);
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float q[DPL];
#pragma unroll
    for (int d = 0; d < DPL; d++) q[d] = a.q[head * HD + lane * DPL + d];
    const float scale = 1.0f / sqrtf((float)HD);  // src/transformer.rs:770
    float m = -FLT_MAX, l = 0.f, acc[DPL];
#pragma unroll
    for (int d = 0; d < DPL; d++) acc[d] = 0.f;

    for (int tb = t0 + warp; tb < t1; tb += kWarps * PB) {
        const bool first = tb == t0 + warp;
#pragma unroll
        for (int j = 0; j < PB; j++) {
            const int t = tb + j * kWarps;
            if (t < t1 && (!first || t == T - 1)) {  // the newest row, and every batch after the first
                kv[j] = *reinterpret_cast<const RV*>(kbase + (int64_t)t * HD);
                vv[j] = *reinterpret_cast<const RV*>(vbase + (int64_t)t * HD);
            }
        }
        float sc[PB];
#pragma unroll
        for (int j = 0; j < PB; j++) {
            float dot = 0.f;
            if (tb + j * kWarps < t1) {
                float kf[DPL];
                row_unpack<CT, DPL>(kv[j], kf);
#pragma unroll
                for (int d = 0; d < DPL; d++) dot = fmaf(q[d], kf[d], dot);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            sc[j] = (tb + j * kWarps < t1) ? dot * scale : -FLT_MAX;
        }
        float bm = sc[0];
#pragma unroll
        for (int j = 1; j < PB; j++) bm = fmaxf(bm, sc[j]);
        const float m_new = fmaxf(m, bm);
        const float rescale = expf(m - m_new);  // first batch: exp(-huge) = 0 against zero state
        l *= rescale;
#pragma unroll
        for (int d = 0; d < DPL; d++) acc[d] *= rescale;
#pragma unroll
        for (int j = 0; j < PB; j++) {
            if (tb + j * kWarps < t1) {
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
    // merge the eight warps
    if (lane == 0) { w_m[warp] = m; w_l[warp] = l; }
#pragma unroll
    for (int d = 0; d < DPL; d++) w_o[warp][lane * DPL + d] = acc[d];
    __syncthreads();
    float M = w_m[0];
#pragma unroll
    for (int w = 1; w < kWarps; w++) M = fmaxf(M, w_m[w]);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; w++) L += w_l[w] * expf(w_m[w] - M);
    CT* out = reinterpret_cast<CT*>(a.out) + head * HD;
    float o = 0.f;
    const int c = threadIdx.x;
    if (c < HD) {
#pragma unroll
        for (int w = 0; w < kWarps; w++) o += w_o[w][c] * expf(w_m[w] - M);
    }
    if constexpr (CL) {
        __shared__ float r_o[kMaxCluster][HD];
        __shared__ float r_m[kMaxCluster], r_l[kMaxCluster];
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // every CTA of the cluster has started
        if (work) {
            if (c < HD) cluster_store(cluster_map(&r_o[split][c], 0), o);
            if (c == 0) {
                cluster_store(cluster_map(&r_m[split], 0), M);
                cluster_store(cluster_map(&r_l[split], 0), L);
            }
        }
        cluster_sync();
        if (split != 0) return;
        float GM = r_m[0];
        for (int s = 1; s < active; s++) GM = fmaxf(GM, r_m[s]);
        float GL = 0.f, go = 0.f;
        for (int s = 0; s < active; s++) {
            const float w = expf(r_m[s] - GM);
            GL += r_l[s] * w;
            if (c < HD) go += r_o[s][c] * w;
        }
        if (c < HD) out[c] = cast_out<CT>(go / GL);
        return;
    }
    if (active == 1) {
        if (c < HD) out[c] = cast_out<CT>(o / L);
        return;
    }
    float* rec = a.scratch + ((int64_t)head * a.n_split + split) * (HD + 2);
    if (c < HD) rec[c] = o;
    if (c == 0) { rec[HD] = M; rec[HD + 1] = L; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket_sh = atomicAdd(a.counters + head, 1u);
    __syncthreads();
    if (ticket_sh != (unsigned)(active - 1)) return;
    // last CTA of this head: merge the splits. The record columns are requested together with the
    // per-split maxima and sums (one round trip through L2), eight splits at a time.
    __threadfence();
    __shared__ float sp_m[64], sp_w[64];
    const float* recs = a.scratch + (int64_t)head * a.n_split * (HD + 2);
    constexpr int MB = 8;
    float rv[MB];
#pragma unroll
    for (int s = 0; s < MB; s++) rv[s] = (c < HD && s < active) ? __ldcg(recs + s * (HD + 2) + c) : 0.f;
    if (threadIdx.x < active) {
        sp_m[threadIdx.x] = __ldcg(recs + threadIdx.x * (HD + 2) + HD);
        sp_w[threadIdx.x] = __ldcg(recs + threadIdx.x * (HD + 2) + HD + 1);
    }
    __syncthreads();
    float GM = -FLT_MAX;
    for (int s = 0; s < active; s++) GM = fmaxf(GM, sp_m[s]);
    float GL = 0.f;
    for (int s = 0; s < active; s++) GL += sp_w[s] * expf(sp_m[s] - GM);
    __syncthreads();
    if (threadIdx.x < active) sp_w[threadIdx.x] = expf(sp_m[threadIdx.x] - GM) / GL;
    __syncthreads();
    if (c < HD) {
        float go = 0.f;
#pragma unroll
        for (int s = 0; s < MB; s++)
            if (s < active) go += rv[s] * sp_w[s];
#pragma unroll 4
        for (int s = MB; s < active; s++) go += __ldcg(recs + s * (HD + 2) + c) * sp_w[s];
        out[c] = cast_out<CT>(go);
    }
    if (threadIdx.x == 0) a.counters[head] = 0;  // ready for the next launch
}

size_t attn_smem_bytes(int hd, int vec, int max_positions) {
    return sizeof(float) * ((size_t)2 * hd + (size_t)kThreads * vec + (size_t)max_positions);
}

}  // namespace

size_t attn_decode_scratch_floats(int heads, int hd, int n_split) { return (size_t)heads * n_split * (hd + 2); }

int launch_attn_decode(rlb_ctx* ctx, rlb_dtype cache_dtype, const AttnDecodeArgs& a, int allow_pdl) {
    const int vec = cache_dtype == RLB_F16 ? 8 : 4;
    if (a.hd % 8 != 0 || (a.hd / 8) % vec != 0 || a.hd / vec > kThreads)
        return rlb_fail(RLB_ERR_INVALID, "attention: head_dim %d is not supported", a.hd);
    int chunk = (a.max_seq + a.n_split - 1) / a.n_split;
    chunk = (chunk + 31) & ~31;
    const size_t smem = attn_smem_bytes(a.hd, vec, chunk);
    if (smem > 200 * 1024) return rlb_fail(RLB_ERR_LIMIT, "attention: %d positions per CTA do not fit in shared memory", chunk);
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(a.heads, a.n_split);
    lc.blockDim = dim3(kThreads);
    lc.dynamicSmemBytes = smem;
    lc.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = allow_pdl ? 1 : 0;
    static const bool use_fast = getenv("RLB_ATTN_FAST") == nullptr || atoi(getenv("RLB_ATTN_FAST")) != 0;
    static const bool use_cluster = getenv("RLB_ATTN_CLUSTER") == nullptr || atoi(getenv("RLB_ATTN_CLUSTER")) != 0;
    if (use_fast && (a.hd == 64 || a.hd == 128)) {
        lc.dynamicSmemBytes = 0;
        // the splits of a head as one thread-block cluster (sizes beyond 8 are non-portable and need an opt-in)
        const bool cluster = use_cluster && a.n_split <= kMaxCluster;
        if (cluster) {
            cudaLaunchAttribute& ca = attr[lc.numAttrs++];
            ca.id = cudaLaunchAttributeClusterDimension;
            ca.val.clusterDim.x = 1;
            ca.val.clusterDim.y = (unsigned)a.n_split;
            ca.val.clusterDim.z = 1;
        }
        // A CTA that may own more than 128 positions takes 16 per warp and batch -- but only while the grid is at most one
        // CTA per SM (few local heads, i.e. tensor parallelism). Measured on 8 local heads at context 1800: 8 splits 33.4 us
        // per layer, 8 splits with 16 per batch 31.0, 16 splits 30.2, 16 splits with 16 per batch 32.6 (the larger register
        // footprint costs more than the shorter chain of batches saves; 65B on one GPU: 22.0 -> 23.5 ms/token with it).
        static const int wide_env = getenv("RLB_ATTN_WIDE") ? atoi(getenv("RLB_ATTN_WIDE")) : -1;  // experiments: force off / on
        const bool wide = wide_env >= 0 ? wide_env != 0 : (fast_chunk(a.max_seq, a.n_split) > 128 && a.heads * a.n_split <= ctx->sm_count);
        const void* kern;
#define RLB_ATTN_PICK(CT, HD) (cluster ? (wide ? (const void*)attn_decode_fast_kernel<CT, HD, true, 16> : (const void*)attn_decode_fast_kernel<CT, HD, true, 8>) \
                                       : (wide ? (const void*)attn_decode_fast_kernel<CT, HD, false, 16> : (const void*)attn_decode_fast_kernel<CT, HD, false, 8>))
        if (cache_dtype == RLB_F16) kern = a.hd == 128 ? RLB_ATTN_PICK(__half, 128) : RLB_ATTN_PICK(__half, 64);
        else kern = a.hd == 128 ? RLB_ATTN_PICK(float, 128) : RLB_ATTN_PICK(float, 64);
#undef RLB_ATTN_PICK
        if (cluster && a.n_split > 8) RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        // same shared-memory split as the projection kernels before and after this one, so that their
        // CTAs (which prefetch weights while they wait for this kernel) can share an SM with these
        RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        void* kargs[] = {(void*)&a};
        RLB_CUDA(cudaLaunchKernelExC(&lc, kern, kargs));
    } else if (cache_dtype == RLB_F16) {
        static std::atomic<uint64_t> set{0};
        if (!attr_done(set, ctx->device)) { RLB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr_mark(set, ctx->device); }
        RLB_CUDA(cudaLaunchKernelEx(&lc, attn_decode_kernel<__half>, a));
    } else {
        static std::atomic<uint64_t> set{0};
        if (!attr_done(set, ctx->device)) { RLB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr_mark(set, ctx->device); }
        RLB_CUDA(cudaLaunchKernelEx(&lc, attn_decode_kernel<float>, a));
    }
    count_launch(ctx);
    return RLB_OK;
}

int launch_attn_prefill(rlb_ctx* ctx, rlb_dtype cache_dtype, const AttnPrefillArgs& a) {
    const int vec = cache_dtype == RLB_F16 ? 8 : 4;
    if (a.hd % 8 != 0 || (a.hd / 8) % vec != 0 || a.hd / vec > kThreads)
        return rlb_fail(RLB_ERR_INVALID, "attention: head_dim %d is not supported", a.hd);
    if (a.allow_tc && attn_prefill_tc_supported(cache_dtype, a)) return launch_attn_prefill_tc(ctx, a, a.err);
    static const bool use_tiled = getenv("RLB_ATTN_TILED") == nullptr || atoi(getenv("RLB_ATTN_TILED")) != 0;
    if (use_tiled && a.n >= 8 && (a.hd == 64 || a.hd == 128) && a.q_ld % 4 == 0) {
        const size_t smem = sizeof(float) * ((size_t)kQB * (a.hd + 4) + (size_t)kTB * (a.hd + 4) + (size_t)kTB * a.hd + (size_t)kQB * (kTB + 1));
        dim3 grid(a.heads, (a.n + kQB - 1) / kQB);
        const void* kern;
        if (cache_dtype == RLB_F16) kern = a.hd == 128 ? (const void*)attn_prefill_tiled_kernel<__half, 128> : (const void*)attn_prefill_tiled_kernel<__half, 64>;
        else kern = a.hd == 128 ? (const void*)attn_prefill_tiled_kernel<float, 128> : (const void*)attn_prefill_tiled_kernel<float, 64>;
        RLB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cudaLaunchConfig_t lc = {};
        lc.gridDim = grid; lc.blockDim = dim3(256); lc.dynamicSmemBytes = smem; lc.stream = ctx->stream;
        cudaLaunchAttribute pattr[1];
        pattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        pattr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = pattr; lc.numAttrs = ctx->pdl_chain ? 1 : 0;
        void* kargs[] = {(void*)&a};
        RLB_CUDA(cudaLaunchKernelExC(&lc, kern, kargs));
        count_launch(ctx);
        return RLB_OK;
    }
    const size_t smem = attn_smem_bytes(a.hd, vec, a.start_pos + a.n);
    if (smem > 200 * 1024) return rlb_fail(RLB_ERR_LIMIT, "attention: %d positions do not fit in shared memory", a.start_pos + a.n);
    dim3 grid(a.heads, a.n);
    if (cache_dtype == RLB_F16) {
        static std::atomic<uint64_t> set{0};
        if (!attr_done(set, ctx->device)) { RLB_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr_mark(set, ctx->device); }
        attn_prefill_kernel<__half><<<grid, kThreads, smem, ctx->stream>>>(a);
    } else {
        static std::atomic<uint64_t> set{0};
        if (!attr_done(set, ctx->device)) { RLB_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr_mark(set, ctx->device); }
        attn_prefill_kernel<float><<<grid, kThreads, smem, ctx->stream>>>(a);
    }
    RLB_LAUNCH_CHECK();
    count_launch(ctx);
    return RLB_OK;
}


// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the standalone attention op.
//
// Some hosts of this library cannot let it allocate device memory while tokens are being
// generated: an inference server that has already divided all of HBM between weights and KV
// caches has nothing left for cudaMalloc to hand out, and a worker thread on the token path
// cannot afford cudaMalloc / cudaFree, which stall every stream of the device while they run.
// For those callers the split-attention kernel's scratch (per-split partial outputs and the
// per-head arrival counters) lives in the fixed array below instead of
// in memory obtained at call time. Every GPU that loads the library holds the array
// (kStaticBytes) until the process exits.
//
// Limits and rules:
//  * heads <= kStaticMaxHeads and heads * n_split * (head_dim + 2) floats <= kStaticRecordFloats,
//    otherwise the call fails with RLB_ERR_LIMIT;
//  * all calls on a device share the one array and it keeps the last call's contents: the words
//    that must start at zero are cleared on every call, and two calls that overlap on the GPU
//    (different streams or contexts of the same device) race on it -- serialise them;
//  * the first call on each device looks up the array's device address
//    (cudaGetSymbolAddress); make that first call before any stream capture begins.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kStaticMaxHeads = 256;
constexpr size_t kStaticHeaderFloats = 64 + kStaticMaxHeads;      // one unused 256-byte line + counters
constexpr size_t kStaticRecordFloats = 256 * 1024;                // 1 MiB of partial records
constexpr size_t kStaticFloats = kStaticHeaderFloats + kStaticRecordFloats;
constexpr size_t kStaticBytes = kStaticFloats * sizeof(float);

// In host code this name is only a handle for the runtime's symbol lookup, never an address a
// kernel could use; the device address is obtained once per device below.
static __device__ __align__(256) float g_attn_static[kStaticFloats];

constexpr int kMaxDevices = 64;
float* g_attn_static_addr[kMaxDevices] = {nullptr};
std::mutex g_attn_static_mu;

int static_scratch_address(int device, float** out) {
    if (device < 0 || device >= kMaxDevices) return rlb_fail(RLB_ERR_LIMIT, "attention (static scratch): device index %d is beyond %d", device, kMaxDevices);
    std::lock_guard<std::mutex> g(g_attn_static_mu);
    if (!g_attn_static_addr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static);  // the caller made `device` current
        if (e != cudaSuccess || !p) return rlb_fail(RLB_ERR_CUDA, "cudaGetSymbolAddress(static attention scratch): %s", cudaGetErrorString(e));
        g_attn_static_addr[device] = static_cast<float*>(p);
    }
    *out = g_attn_static_addr[device];
    return RLB_OK;
}

}  // namespace

extern "C" int rlb_attention_decode_static(rlb_tensor* out, const rlb_tensor* q, const rlb_tensor* kcache, const rlb_tensor* vcache,
                                           int32_t heads, int32_t max_seq_len, int32_t pos, int32_t n_split) {
    int hd = 0;
    RLB_TRY(attention_check(out, q, kcache, vcache, heads, max_seq_len, pos, n_split, &hd));
    if (heads > kStaticMaxHeads)
        return rlb_fail(RLB_ERR_LIMIT, "attention (static scratch): %d heads exceed the maximum of %d", heads, kStaticMaxHeads);
    const size_t need = attn_decode_scratch_floats(heads, hd, n_split);
    if (need > kStaticRecordFloats)
        return rlb_fail(RLB_ERR_LIMIT, "attention (static scratch): heads %d x n_split %d x (head_dim %d + 2) = %zu floats exceed the fixed %zu",
                        heads, n_split, hd, need, kStaticRecordFloats);
    rlb_ctx* ctx = out->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    float* base = nullptr;
    RLB_TRY(static_scratch_address(ctx->device, &base));
    // the arrival counters must start from zero on every call (an earlier call that was cut short may
    // have left some behind); the position travels by value in the kernel's arguments
    RLB_CUDA(cudaMemsetAsync(base, 0, kStaticHeaderFloats * sizeof(float), ctx->stream));
    AttnDecodeArgs a;
    a.q = (const float*)q->d; a.kcache = kcache->d; a.vcache = vcache->d; a.out = out->d;
    a.pos_ptr = nullptr; a.pos_value = pos;
    a.heads = heads; a.hd = hd; a.max_seq = max_seq_len; a.n_split = n_split;
    a.counters = reinterpret_cast<unsigned int*>(base + 64);
    a.scratch = base + kStaticHeaderFloats;
    RLB_TRY(launch_attn_decode(ctx, kcache->dtype, a, 0));
    RLB_CUDA(cudaEventRecord(out->ready, ctx->stream));
    return RLB_OK;
}

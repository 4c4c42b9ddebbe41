// Model-level path: what rllama's Transformer::from_unpickled / make_caches / forward
// (src/transformer.rs:242-382) become on one B200 or on a tensor-parallel group of them.
//
// Decode (one token) is a fixed chain of fused kernels per layer, replayed as a CUDA graph:
//   1. [residual add + attention RMSNorm] -> Wq|Wk|Wv GEMV -> f16 round -> RoPE -> KV append
//   2. single-query attention over the cache (split over positions, combined in-kernel)
//   3. Wo GEMV -> f32 partial sums
//   4. [residual add + FFN RMSNorm] -> W1,W3 GEMV -> SiLU gate -> f16 round
//   5. W2 GEMV -> f32 partial sums
// and, after the last layer, [residual add + final RMSNorm] -> f32 vocabulary head -> arg-max.
// The "residual add" of step 1/4/head consumes the partial sums of step 5/3: it sums them in
// rank order (one term without tensor parallelism), rounds the sum to f16 where the reference
// rounds the projection's output (src/transformer.rs:570, :819) and adds it to the residual
// stream (src/transformer.rs:442-445).
//
// Prefill (n > 1 tokens) runs the same stages as row-wise kernels around a tiled GEMM.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "internal.h"
#include "tp.h"

namespace {

struct LayerW {
    void* wqkv = nullptr;  // [3 * nq][dim]   (q rows, then k rows, then v rows of this rank's heads)
    void* wo = nullptr;    // [dim][nq]
    void* w1 = nullptr;    // [F_local][dim]
    void* w3 = nullptr;    // [F_local][dim]
    void* w2 = nullptr;    // [dim][F_local]
    float* attn_norm = nullptr;
    float* ffn_norm = nullptr;
    // Layer not resident in HBM (percentage_to_gpu < 1): its five matrices wait here, in pinned host
    // memory, laid out like the model's HBM staging buffer, which the pointers above then address.
    char* host = nullptr;
};

struct ProfSlot {
    cudaEvent_t ev = nullptr;
    int cls = -1;  // class of the kernel that FOLLOWS this event
};

enum ProfClass { PC_QKV = 0, PC_ATTN, PC_WO, PC_W13, PC_W2, PC_HEAD, PC_ARGMAX, PC_COMM, PC_COUNT };
const char* kProfNames[PC_COUNT] = {"qkv", "attn", "wo", "w13", "w2", "head", "argmax", "comm"};

}  // namespace

struct rlb_model {
    rlb_ctx* ctx = nullptr;
    rlb_model_params p{};
    int hd = 0, tp = 1, rank = 0;
    int head0 = 0, nh = 0, nq = 0;  // this rank's heads
    int f0 = 0, F = 0;              // this rank's FFN slice
    int v0 = 0, V = 0;              // this rank's vocabulary slice
    rlb_dtype wdt = RLB_F32;
    size_t wsz = 4;
    bool finalized = false;

    float* tok_emb = nullptr;
    float* norm = nullptr;
    float* output = nullptr;
    float* rope = nullptr;
    std::vector<LayerW> L;
    std::vector<uint8_t> have;  // [n_layers * 12 + kind] flags
    int gpu_layers = 0;         // layers 0 .. gpu_layers-1 are resident in HBM (src/transformer.rs:262-274)
    char* stage = nullptr;      // HBM staging buffer for the matrices of one non-resident layer
    size_t layer_bytes = 0;     // wqkv | wo | w1 w3 | w2 of one layer

    // decode buffers
    float* xa = nullptr;
    float* xb = nullptr;
    float* qbuf = nullptr;
    void* obuf = nullptr;   // attention output, weight dtype
    void* gbuf = nullptr;   // gated FFN activation, weight dtype
    float* part_wo = nullptr;   // [tp][dim]
    float* part_w2 = nullptr;   // [tp][dim]
    float* logits_local = nullptr;  // [V]
    float* logits = nullptr;        // [vocab]
    int32_t* scalars = nullptr;     // device: tok, pos, step, next
    int32_t* tokens_out = nullptr;  // device [tokens_cap]
    int tokens_cap = 0;
    float* attn_scratch = nullptr;
    unsigned int* attn_counters = nullptr;
    int n_split = 1;
    int32_t* h_scalars = nullptr;  // pinned
    float* h_logits = nullptr;     // pinned [vocab]
    int32_t* h_tokens = nullptr;   // pinned [tokens_cap]

    // prefill buffers (grown on demand)
    int pf_cap = 0;
    int32_t* pf_tokens = nullptr;
    float* pf_x = nullptr;
    void* pf_a = nullptr;
    float* pf_qkv = nullptr;
    void* pf_o = nullptr;
    float* pf_p = nullptr;
    float* pf_g1 = nullptr;
    void* pf_g = nullptr;
    float* pf_last = nullptr;

    // tensor parallel
    TpNccl nccl;
    int tp_mode = 0;                 // 0: NCCL collectives, 1: fused one-shot push over peer memory
    // push mode: one exchange buffer per rank, mapped into every peer; all of it is 8-byte
    // {f32 value, u32 sequence} entries:
    //   [inbox_wo : tp*dim][inbox_w2 : tp*dim][logits : vocab][x_a : dim][x_b : dim]
    char* xbuf = nullptr;
    size_t xbuf_bytes = 0;
    char* peer_xbuf[RLB_MAX_TP] = {nullptr};  // peer_xbuf[rank] == xbuf
    bool peers_open = false;
    bool peers_ipc = false;          // the peer buffers were mapped from IPC handles (and must be unmapped)
    uint64_t graph_gen = 0;          // bumped when captured graphs become stale

    // options / statistics
    bool w_f16_exact = true;  // every projection matrix arrived as f16 (or was checked): its f32 copy is exact in TF32
    bool use_graph = true;
    bool use_stream = true;  // bulk-copy staged GEMV kernels (gemv_stream.cu)
    bool use_pdl = true;     // programmatic dependent launch between the decode kernels
    bool profile = false;
    double prof_ms[PC_COUNT] = {0};
    int prof_steps = 0;
    std::vector<ProfSlot> prof_slots;
    size_t prof_used = 0;
    uint64_t kernels_per_step = 0;
};

struct rlb_caches {
    rlb_model* m = nullptr;
    void* k = nullptr;  // [n_layers][nh][max_seq][hd]
    void* v = nullptr;
    size_t layer_elems = 0;
    cudaGraphExec_t graph = nullptr;      // decode step that leaves the arg-max in scalars[3]
    cudaGraphExec_t graph_adv = nullptr;  // decode step with on-device token feedback
    uint64_t graph_gen = 0;               // model->graph_gen the graphs were captured under
    bool warmed = false;
};

namespace {

size_t cache_bytes(const rlb_model* m) { return (size_t)m->p.n_layers * m->nh * m->p.max_seq_len * m->hd * m->wsz; }

int dev_alloc(void** p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) return rlb_fail(RLB_ERR_OOM, "cudaMalloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
    return RLB_OK;
}
template <typename T> int dev_alloc_t(T** p, size_t count) { return dev_alloc((void**)p, count * sizeof(T)); }

void split_even(int total, int parts, int idx, int* start, int* count) {
    const int base = total / parts, rem = total % parts;
    *count = base + (idx < rem ? 1 : 0);
    *start = idx * base + (idx < rem ? idx : rem);
}

void prof_mark(rlb_model* m, int cls) {
    if (!m->profile) return;
    if (m->prof_used >= m->prof_slots.size()) {
        ProfSlot s;
        cudaEventCreate(&s.ev);
        m->prof_slots.push_back(s);
    }
    ProfSlot& s = m->prof_slots[m->prof_used++];
    s.cls = cls;
    cudaEventRecord(s.ev, m->ctx->stream);
}

void prof_collect(rlb_model* m) {
    if (!m->profile || m->prof_used < 2) { m->prof_used = 0; return; }
    cudaEventSynchronize(m->prof_slots[m->prof_used - 1].ev);
    for (size_t i = 0; i + 1 < m->prof_used; i++) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, m->prof_slots[i].ev, m->prof_slots[i + 1].ev);
        if (m->prof_slots[i].cls >= 0) m->prof_ms[m->prof_slots[i].cls] += ms;
    }
    m->prof_used = 0;
    m->prof_steps++;
}

// Exchange-buffer layout (push mode), byte offsets.
size_t xb_inbox_wo(const rlb_model*) { return 0; }
size_t xb_inbox_w2(const rlb_model* m) { return (size_t)m->tp * m->p.dim * 8; }
size_t xb_logits(const rlb_model* m) { return 2 * (size_t)m->tp * m->p.dim * 8; }
size_t xb_x(const rlb_model* m, int which) { return xb_logits(m) + (size_t)m->p.vocab_size * 8 + (size_t)which * m->p.dim * 8; }
size_t xb_ready(const rlb_model* m, int idx) { return ((xb_x(m, 2) + 127) & ~(size_t)127) + (size_t)idx * 128; }  // one line per exchange
size_t xb_total(const rlb_model* m) { return xb_ready(m, 2 * m->p.n_layers + 2); }
bool push_mode(const rlb_model* m) { return m->tp > 1 && m->tp_mode == 1; }

// All-reduce of the partial sums of one projection when the NCCL mode is active.
int tp_reduce(rlb_model* m, float* part, size_t count, bool decode = true) {
    if (m->tp == 1 || (decode && push_mode(m))) return RLB_OK;
    prof_mark(m, PC_COMM);
    return nccl_allreduce_f32(&m->nccl, part, count, m->ctx->stream);
}

// Decode GEMV: the bulk-copy staged kernel where the shape allows, else the register-staged one.
// after_copy: the kernel follows a copy on the stream, not a kernel, so it is launched as an ordinary dependent.
int gemv_decode(rlb_model* m, rlb_dtype dtype, int prologue, int epilogue, const GemvArgs& a, bool after_copy = false) {
    if (m->use_stream) {
        const int s = launch_gemv_stream(m->ctx, dtype, prologue, epilogue, a, m->scalars + 8, m->use_pdl && !m->profile && !after_copy);
        if (s != RLB_ERR_STATE) return s;
    }
    if (a.ll_inbox != nullptr || a.n_outs > 0)
        return rlb_fail(RLB_ERR_STATE, "the tensor-parallel push exchange needs the staged GEMV kernel, which does not take this shape (rows %d, K %d)", a.rows, a.K);
    return launch_gemv(m->ctx, dtype, prologue, epilogue, a);
}

// ---- the decode step (enqueue only; runs eagerly or under stream capture) -----------------
int enqueue_decode_step(rlb_model* m, rlb_caches* c, bool advance) {
    rlb_ctx* ctx = m->ctx;
    const int d = m->p.dim;
    const int32_t* tok = m->scalars + 0;
    const int32_t* pos = m->scalars + 1;
    const bool f16 = m->wdt == RLB_F16;
    const bool push = push_mode(m);
    const float* parts_wo = m->part_wo;
    const float* parts_w2 = m->part_w2;
    const uint32_t seq_stride = 2u * (uint32_t)m->p.n_layers + 1u;  // exchanges per decode step

    // Producer side of an exchange (push mode): tagged partial sums go into every rank's inbox.
    auto push_out = [&](GemvArgs& a, size_t inbox_off, int64_t offset, uint32_t idx) {
        a.n_outs = m->tp;
        a.out_offset = offset;
        a.out_seq_idx = idx + 1;
        a.seq_stride = seq_stride;
        a.epoch_ptr = m->scalars + 4;
        for (int r = 0; r < m->tp; r++) a.ll_outs[r] = (uint2*)(m->peer_xbuf[r] + inbox_off);
    };
    // Consumer side: poll this rank's inbox for exchange `idx`, publish the new residual in x buffer `which`.
    auto push_in = [&](GemvArgs& a, size_t inbox_off, uint32_t idx, int which) {
        a.ll_inbox = (const uint2*)(m->xbuf + inbox_off);
        a.xready = (unsigned int*)(m->xbuf + xb_ready(m, (int)idx));
        a.n_parts = m->tp;
        a.seq_idx = idx + 1;
        a.seq_stride = seq_stride;
        a.epoch_ptr = m->scalars + 4;
        // Short rows on few ranks: every CTA polls the whole row's entries itself (tp * dim * 8 bytes through L2 per
        // CTA) and the slice publication with its fence, counter and second L2 round trip falls away.
        static const int gather_kb = getenv("RLB_TP_GATHER_KB") ? atoi(getenv("RLB_TP_GATHER_KB")) : 64;
        // (two ranks only: the case that was measured and is covered by the 2-GPU tests)
        a.gather_all = m->tp == 2 && d <= 4096 && (size_t)m->tp * (size_t)d * 8 <= (size_t)gather_kb * 1024;
    };

    for (int l = 0; l < m->p.n_layers; l++) {
        const LayerW& W = m->L[l];
        char* kc = (char*)c->k + (size_t)l * c->layer_elems * m->wsz;
        char* vc = (char*)c->v + (size_t)l * c->layer_elems * m->wsz;
        if (W.host)  // not resident: bring the layer's matrices into the staging buffer (stream order keeps the previous layer's reads ahead of it)
            RLB_CUDA(cudaMemcpyAsync(m->stage, W.host, m->layer_bytes, cudaMemcpyHostToDevice, ctx->stream));
        {   // 1. norm + q/k/v projection + RoPE + cache append
            GemvArgs a;
            a.W = W.wqkv; a.rows = 3 * m->nq; a.K = d; a.ldw = d;
            if (l == 0) { a.x_in = m->tok_emb; a.tok_ptr = tok; }
            else {
                a.x_in = m->xb; a.parts = parts_w2; a.n_parts = 1; a.part_stride = d; a.round_parts = f16;
                if (push) push_in(a, xb_inbox_w2(m), 2u * (l - 1) + 1u, 0);
            }
            a.x_out = m->xa; a.gain = W.attn_norm; a.eps = m->p.norm_eps;
            a.qbuf = m->qbuf; a.kcache = kc; a.vcache = vc; a.rope = m->rope; a.pos_ptr = pos;
            a.nq = m->nq; a.hd = m->hd; a.max_seq = m->p.max_seq_len;
            prof_mark(m, PC_QKV);
            RLB_TRY(gemv_decode(m, m->wdt, PRO_NORM, EPI_QKV, a, W.host != nullptr));
        }
        {   // 2. attention
            AttnDecodeArgs a;
            a.q = m->qbuf; a.kcache = kc; a.vcache = vc; a.out = m->obuf; a.pos_ptr = pos;
            a.heads = m->nh; a.hd = m->hd; a.max_seq = m->p.max_seq_len; a.n_split = m->n_split;
            a.scratch = m->attn_scratch; a.counters = m->attn_counters;
            prof_mark(m, PC_ATTN);
            RLB_TRY(launch_attn_decode(ctx, m->wdt, a, m->use_stream && m->use_pdl && !m->profile));
        }
        {   // 3. wo
            GemvArgs a;
            a.W = W.wo; a.rows = d; a.K = m->nq; a.ldw = m->nq; a.vec_in = m->obuf; a.out = m->part_wo;
            if (push) {
                push_out(a, xb_inbox_wo(m), (int64_t)m->rank * d, 2u * l);
                if (gemv_stream_grid(ctx, m->wdt, PRO_COPY, EPI_F32, a) == 0)
                    return rlb_fail(RLB_ERR_STATE, "push mode needs the staged GEMV kernel for the wo projection");
            }
            prof_mark(m, PC_WO);
            RLB_TRY(gemv_decode(m, m->wdt, PRO_COPY, EPI_F32, a));
            RLB_TRY(tp_reduce(m, m->part_wo, d));
        }
        {   // 4. residual + norm + w1/w3 + SiLU gate
            GemvArgs a;
            a.W = W.w1; a.W2 = W.w3; a.rows = m->F; a.K = d; a.ldw = d;
            a.x_in = m->xa; a.parts = parts_wo; a.n_parts = 1; a.part_stride = d; a.round_parts = f16;
            if (push) push_in(a, xb_inbox_wo(m), 2u * l, 1);
            a.x_out = m->xb; a.gain = W.ffn_norm; a.eps = m->p.norm_eps; a.out = m->gbuf;
            prof_mark(m, PC_W13);
            RLB_TRY(gemv_decode(m, m->wdt, PRO_NORM, EPI_SWIGLU, a));
        }
        {   // 5. w2
            GemvArgs a;
            a.W = W.w2; a.rows = d; a.K = m->F; a.ldw = m->F; a.vec_in = m->gbuf; a.out = m->part_w2;
            if (push) {
                push_out(a, xb_inbox_w2(m), (int64_t)m->rank * d, 2u * l + 1u);
                if (gemv_stream_grid(ctx, m->wdt, PRO_COPY, EPI_F32, a) == 0)
                    return rlb_fail(RLB_ERR_STATE, "push mode needs the staged GEMV kernel for the w2 projection");
            }
            prof_mark(m, PC_W2);
            RLB_TRY(gemv_decode(m, m->wdt, PRO_COPY, EPI_F32, a));
            RLB_TRY(tp_reduce(m, m->part_w2, d));
        }
    }
    {   // final norm + f32 head (src/transformer.rs:378-381)
        GemvArgs a;
        a.W = m->output; a.rows = m->V; a.K = d; a.ldw = d;
        a.x_in = m->xb; a.parts = parts_w2; a.n_parts = 1; a.part_stride = d; a.round_parts = f16;
        if (push) push_in(a, xb_inbox_w2(m), 2u * (m->p.n_layers - 1) + 1u, 0);
        a.x_out = m->xa;  // the final residual row (the push exchange publishes it there)
        a.gain = m->norm; a.eps = m->p.norm_eps;
        a.out = m->tp == 1 ? m->logits : m->logits_local;
        if (push) {
            push_out(a, xb_logits(m), (int64_t)m->v0, 2u * m->p.n_layers);
            if (gemv_stream_grid(ctx, RLB_F32, PRO_NORM, EPI_F32, a) == 0)
                return rlb_fail(RLB_ERR_STATE, "push mode needs the staged GEMV kernel for the output head");
        }
        prof_mark(m, PC_HEAD);
        RLB_TRY(gemv_decode(m, RLB_F32, PRO_NORM, EPI_F32, a));
        if (m->tp > 1 && !push) {
            prof_mark(m, PC_COMM);
            RLB_TRY(nccl_allgather_f32(&m->nccl, m->logits_local, m->logits, (size_t)m->V, ctx->stream));
        }
    }
    StepSync sy;
    sy.err = m->scalars + 8;
    if (push) {
        sy.epoch = m->scalars + 4;  // counts the decode steps run in push mode (starts at 1)
        sy.ll_logits = (const uint2*)(m->xbuf + xb_logits(m));
        sy.dense_out = m->logits;
        sy.seq_idx = 2u * m->p.n_layers + 1u;
        sy.seq_stride = seq_stride;
    }
    prof_mark(m, PC_ARGMAX);
    if (advance)
        RLB_TRY(launch_argmax_advance(ctx, m->logits, m->p.vocab_size, m->scalars + 0, m->scalars + 1, m->scalars + 2, m->tokens_out,
                                      m->tokens_cap, sy));
    else
        RLB_TRY(launch_argmax(ctx, m->logits, m->p.vocab_size, m->scalars + 3, sy));
    prof_mark(m, -1);
    return RLB_OK;
}

// Runs one decode step: eagerly the first time on a cache object (which also loads every
// kernel before any capture), then as a replayed CUDA graph.
int run_decode_step(rlb_model* m, rlb_caches* c, bool advance, cudaGraphExec_t* slot) {
    rlb_ctx* ctx = m->ctx;
    if (!m->use_graph || m->profile || !c->warmed) {
        const uint64_t before = ctx->launches;
        RLB_TRY(enqueue_decode_step(m, c, advance));
        m->kernels_per_step = ctx->launches - before;
        c->warmed = true;
        if (m->profile) prof_collect(m);
        return RLB_OK;
    }
    if (c->graph_gen != m->graph_gen) {  // the exchange mode changed since these graphs were captured
        if (c->graph) cudaGraphExecDestroy(c->graph);
        if (c->graph_adv) cudaGraphExecDestroy(c->graph_adv);
        c->graph = c->graph_adv = nullptr;
        c->graph_gen = m->graph_gen;
    }
    if (!*slot) {
        const uint64_t before = ctx->launches;
        cudaGraph_t graph = nullptr;
        RLB_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        int s = enqueue_decode_step(m, c, advance);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
        m->kernels_per_step = ctx->launches - before;
        ctx->launches = before;  // capture records, it does not run
        if (s != RLB_OK) {
            if (graph) cudaGraphDestroy(graph);
            return s;
        }
        if (e != cudaSuccess) return rlb_fail(RLB_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
        e = cudaGraphInstantiate(slot, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return rlb_fail(RLB_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    RLB_CUDA(cudaGraphLaunch(*slot, ctx->stream));
    ctx->launches += m->kernels_per_step;
    return RLB_OK;
}

int ensure_prefill_buffers(rlb_model* m, int n) {
    if (n <= m->pf_cap) return RLB_OK;
    cudaStreamSynchronize(m->ctx->stream);
    void** ptrs[] = {(void**)&m->pf_tokens, (void**)&m->pf_x, &m->pf_a, (void**)&m->pf_qkv, &m->pf_o, (void**)&m->pf_p,
                     (void**)&m->pf_g1, &m->pf_g, (void**)&m->pf_last};
    for (void** p : ptrs) { if (*p) cudaFree(*p); *p = nullptr; }
    m->pf_cap = 0;
    const size_t N = (size_t)n, d = m->p.dim;
    RLB_TRY(dev_alloc_t(&m->pf_tokens, N));
    RLB_TRY(dev_alloc_t(&m->pf_x, N * d));
    RLB_TRY(dev_alloc(&m->pf_a, N * d * m->wsz));
    RLB_TRY(dev_alloc_t(&m->pf_qkv, N * 3 * m->nq));
    RLB_TRY(dev_alloc(&m->pf_o, N * m->nq * m->wsz));
    RLB_TRY(dev_alloc_t(&m->pf_p, N * d));
    RLB_TRY(dev_alloc_t(&m->pf_g1, N * 2 * m->F));
    RLB_TRY(dev_alloc(&m->pf_g, N * m->F * m->wsz));
    RLB_TRY(dev_alloc_t(&m->pf_last, d));
    m->pf_cap = n;
    return RLB_OK;
}

// Multi-token forward: tokens are in m->pf_tokens. Leaves the logits of the last token in m->logits.
int enqueue_prefill(rlb_model* m, rlb_caches* c, int n, int start_pos) {
    rlb_ctx* ctx = m->ctx;
    const int d = m->p.dim, nq = m->nq, F = m->F;
    const bool f16 = m->wdt == RLB_F16;
    const int round_proj = (f16 && m->tp == 1) ? 1 : 0;  // with tensor parallelism the rounding follows the reduction
    // the kernels of this chain are launched as programmatic dependents of one another (see rlb_launch)
    struct ChainGuard { rlb_ctx* c; ~ChainGuard() { c->pdl_chain = false; } } chain_guard{ctx};
    ctx->pdl_chain = m->use_pdl && n <= 512;  // (beyond that the kernels run for hundreds of microseconds and nothing is gained)
    RLB_TRY(launch_embed(ctx, m->tok_emb, m->pf_tokens, n, d, m->pf_x));

    // The residual add of a projection's output (src/transformer.rs:442-445) is folded into the RMSNorm that follows
    // it: `pending` says that pf_p holds a projection output not yet added to the residual rows.
    bool pending = false;
    const int round_add = (f16 && !round_proj) ? 1 : 0;
    for (int l = 0; l < m->p.n_layers; l++) {
        const LayerW& W = m->L[l];
        char* kc = (char*)c->k + (size_t)l * c->layer_elems * m->wsz;
        char* vc = (char*)c->v + (size_t)l * c->layer_elems * m->wsz;
        if (W.host) RLB_CUDA(cudaMemcpyAsync(m->stage, W.host, m->layer_bytes, cudaMemcpyHostToDevice, ctx->stream));
        RLB_TRY(launch_add_norm_rows(ctx, m->pf_x, pending ? m->pf_p : nullptr, round_add, n, d, W.attn_norm, m->p.norm_eps, m->wdt, m->pf_a));
        // q, k and v in one GEMM: row i of the result is [q_i | k_i | v_i]
        RLB_TRY(launch_gemm_nt(ctx, m->wdt, m->pf_a, d, W.wqkv, d, m->pf_qkv, 3 * nq, n, 3 * nq, d, f16, m->scalars + 8, m->w_f16_exact));
        RLB_TRY(launch_rope_append(ctx, m->pf_qkv, m->pf_qkv + nq, m->pf_qkv + 2 * nq, 3 * nq, n, start_pos, m->nh, m->hd,
                                   m->p.max_seq_len, m->rope, m->wdt, kc, vc));
        AttnPrefillArgs aa;
        aa.q = m->pf_qkv; aa.q_ld = 3 * nq; aa.kcache = kc; aa.vcache = vc; aa.out = m->pf_o; aa.n = n; aa.start_pos = start_pos;
        aa.heads = m->nh; aa.hd = m->hd; aa.max_seq = m->p.max_seq_len; aa.err = m->scalars + 8;
        RLB_TRY(launch_attn_prefill(ctx, m->wdt, aa));
        RLB_TRY(launch_gemm_nt(ctx, m->wdt, m->pf_o, nq, W.wo, nq, m->pf_p, d, n, d, nq, round_proj, m->scalars + 8, m->w_f16_exact));
        RLB_TRY(tp_reduce(m, m->pf_p, (size_t)n * d, false));
        RLB_TRY(launch_add_norm_rows(ctx, m->pf_x, m->pf_p, round_add, n, d, W.ffn_norm, m->p.norm_eps, m->wdt, m->pf_a));
        // w1 and w3 (stored back to back) in one GEMM: row i of the result is [w1 x_i | w3 x_i]
        RLB_TRY(launch_gemm_nt(ctx, m->wdt, m->pf_a, d, W.w1, d, m->pf_g1, 2 * F, n, 2 * F, d, f16, m->scalars + 8, m->w_f16_exact));
        RLB_TRY(launch_swiglu_rows(ctx, m->pf_g1, m->pf_g1 + F, 2 * F, n, F, m->wdt, m->pf_g));
        RLB_TRY(launch_gemm_nt(ctx, m->wdt, m->pf_g, F, W.w2, F, m->pf_p, d, n, d, F, round_proj, m->scalars + 8, m->w_f16_exact));
        RLB_TRY(tp_reduce(m, m->pf_p, (size_t)n * d, false));
        pending = true;
    }
    // the last layer's FFN output still has to be added; only the last row is needed from here on
    RLB_TRY(launch_add_rows(ctx, m->pf_x + (size_t)(n - 1) * d, m->pf_p + (size_t)(n - 1) * d, d, round_add));
    // only the last row gets logits (src/transformer.rs:378-381)
    RLB_TRY(launch_rmsnorm_rows(ctx, m->pf_x + (size_t)(n - 1) * d, 1, d, m->norm, m->p.norm_eps, RLB_F32, m->pf_last));
    GemvArgs a;
    a.W = m->output; a.rows = m->V; a.K = d; a.ldw = d; a.vec_in = m->pf_last;
    a.out = m->tp == 1 ? m->logits : m->logits_local;
    {   // the staged GEMV where it takes the shape (the head is the largest single matrix), else the register-staged one
        int s = m->use_stream ? launch_gemv_stream(ctx, RLB_F32, PRO_COPY, EPI_F32, a, m->scalars + 8, 0) : RLB_ERR_STATE;
        if (s == RLB_ERR_STATE) s = launch_gemv(ctx, RLB_F32, PRO_COPY, EPI_F32, a);
        RLB_TRY(s);
    }
    if (m->tp > 1) RLB_TRY(nccl_allgather_f32(&m->nccl, m->logits_local, m->logits, (size_t)m->V, ctx->stream));
    return RLB_OK;
}

// The decode kernels raise scalars[8] when a bounded wait ran out; h points at its host copy.
int check_device_flag(const int32_t* h) {
    if (*h == 3) return rlb_fail(RLB_ERR_CUDA, "a prefill kernel (GEMM or attention) gave up waiting on a shared-memory barrier (results are invalid)");
    if (*h == 2) return rlb_fail(RLB_ERR_COMM, "a decode kernel gave up waiting for another rank's partial sums (results are invalid)");
    if (*h != 0) return rlb_fail(RLB_ERR_CUDA, "a decode kernel gave up waiting on a shared-memory barrier (results are invalid)");
    return RLB_OK;
}

int check_forward_args(rlb_model* m, rlb_caches* c, const int32_t* tokens, int n, int start_pos) {
    if (!m || !c || !tokens) return rlb_fail(RLB_ERR_INVALID, "forward: null pointer");
    if (!m->finalized) return rlb_fail(RLB_ERR_STATE, "forward: model is not finalized");
    if (c->m != m) return rlb_fail(RLB_ERR_INVALID, "forward: caches belong to another model");
    if (n < 1 || start_pos < 0 || start_pos + n > m->p.max_seq_len)
        return rlb_fail(RLB_ERR_INVALID, "forward: %d tokens at position %d exceed max_seq_len %d", n, start_pos, m->p.max_seq_len);
    for (int i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= m->p.vocab_size)
            return rlb_fail(RLB_ERR_INVALID, "forward: token id %d is outside the vocabulary of %d", tokens[i], m->p.vocab_size);
    return RLB_OK;
}

// Enqueues the forward pass; the last token's logits end up in m->logits and, when want_argmax,
// the greedy choice in m->scalars[3].
int forward_common(rlb_model* m, rlb_caches* c, const int32_t* tokens, int n, int start_pos, bool want_argmax) {
    rlb_ctx* ctx = m->ctx;
    if (n == 1) {
        m->h_scalars[0] = tokens[0];
        m->h_scalars[1] = start_pos;
        RLB_CUDA(cudaMemcpyAsync(m->scalars, m->h_scalars, 2 * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        RLB_TRY(run_decode_step(m, c, false, &c->graph));
        return RLB_OK;
    }
    RLB_TRY(ensure_prefill_buffers(m, n));
    RLB_CUDA(cudaMemcpyAsync(m->pf_tokens, tokens, (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
    RLB_TRY(enqueue_prefill(m, c, n, start_pos));
    if (want_argmax) RLB_TRY(launch_argmax(ctx, m->logits, m->p.vocab_size, m->scalars + 3));
    return RLB_OK;
}

}  // namespace

extern "C" {

int rlb_model_create(rlb_ctx* ctx, const rlb_model_params* p, rlb_model** out) {
    if (!ctx || !p || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_model_create: null pointer");
    *out = nullptr;
    if (p->dim <= 0 || p->n_layers <= 0 || p->n_heads <= 0 || p->ffn_dim <= 0 || p->vocab_size <= 0 || p->max_seq_len <= 0)
        return rlb_fail(RLB_ERR_INVALID, "rlb_model_create: non-positive model dimension");
    if (p->dim % p->n_heads != 0) return rlb_fail(RLB_ERR_INVALID, "dim %d is not divisible by n_heads %d", p->dim, p->n_heads);
    const int tp = p->tp_size <= 0 ? 1 : p->tp_size;
    if (tp > RLB_MAX_TP || p->tp_rank < 0 || p->tp_rank >= tp) return rlb_fail(RLB_ERR_INVALID, "bad tensor-parallel rank %d of %d", p->tp_rank, tp);
    const int hd = p->dim / p->n_heads;
    if (p->dim % 16 != 0 || hd % 8 != 0) return rlb_fail(RLB_ERR_INVALID, "dim must be a multiple of 16 and head_dim of 8");
    if (p->ffn_dim % tp != 0 || (p->ffn_dim / tp) % 8 != 0)
        return rlb_fail(RLB_ERR_INVALID, "ffn_dim %d cannot be split %d ways in multiples of 8", p->ffn_dim, tp);
    if (p->vocab_size % tp != 0) return rlb_fail(RLB_ERR_INVALID, "vocab_size %d is not divisible by tp_size %d", p->vocab_size, tp);
    if (p->n_heads < tp) return rlb_fail(RLB_ERR_INVALID, "fewer heads (%d) than tensor-parallel ranks (%d)", p->n_heads, tp);

    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    rlb_model* m = new rlb_model();
    m->ctx = ctx; m->p = *p; m->p.tp_size = tp; m->tp = tp; m->rank = p->tp_rank; m->hd = hd;
    split_even(p->n_heads, tp, m->rank, &m->head0, &m->nh);
    m->nq = m->nh * hd;
    m->F = p->ffn_dim / tp; m->f0 = m->rank * m->F;
    m->V = p->vocab_size / tp; m->v0 = m->rank * m->V;
    m->wdt = p->force_f16 ? RLB_F16 : RLB_F32;
    m->wsz = dtype_size(m->wdt);
    m->L.resize(p->n_layers);
    m->have.assign((size_t)p->n_layers * 12 + 12, 0);

    const size_t d = p->dim;
    int s = RLB_OK;
    auto A = [&](void** ptr, size_t bytes) { if (s == RLB_OK) s = dev_alloc(ptr, bytes); };
    A((void**)&m->tok_emb, (size_t)p->vocab_size * d * 4);
    A((void**)&m->norm, d * 4);
    A((void**)&m->output, (size_t)m->V * d * 4);
    A((void**)&m->rope, (size_t)p->max_seq_len * (hd / 2) * 2 * 4);
    // DataSettings::percentage_to_gpu (src/transformer.rs:91-103) and the rule of :262-274, in f32 as there
    float pct = p->has_percentage_to_gpu ? p->percentage_to_gpu : 1.0f;
    if (pct >= 1.0f) pct = 1.0f;
    if (pct < 0.0f) pct = 0.0f;
    if (pct != pct) pct = 0.0f;
    m->gpu_layers = std::min(p->n_layers, (int)roundf(pct * (float)(p->n_layers - 1)) + 1);
    const size_t b_qkv = (size_t)3 * m->nq * d * m->wsz, b_wo = d * m->nq * m->wsz, b_w13 = (size_t)2 * m->F * d * m->wsz,
                 b_w2 = d * m->F * m->wsz;
    m->layer_bytes = b_qkv + b_wo + b_w13 + b_w2;
    if (m->gpu_layers < p->n_layers) A((void**)&m->stage, m->layer_bytes);
    for (int l = 0; l < p->n_layers; l++) {
        LayerW& W = m->L[l];
        if (l < m->gpu_layers) {
            A(&W.wqkv, b_qkv);
            A(&W.wo, b_wo);
            A(&W.w1, b_w13);  // w1 and w3 back to back: one GEMM serves both at prefill
            A(&W.w2, b_w2);
        } else if (s == RLB_OK) {
            cudaError_t e = cudaHostAlloc((void**)&W.host, m->layer_bytes, cudaHostAllocMapped | cudaHostAllocPortable);
            if (e != cudaSuccess) s = rlb_fail(RLB_ERR_OOM, "pinned host memory for layer %d (%zu bytes): %s", l, m->layer_bytes, cudaGetErrorString(e));
            W.wqkv = m->stage; W.wo = m->stage + b_qkv; W.w1 = m->stage + b_qkv + b_wo; W.w2 = m->stage + b_qkv + b_wo + b_w13;
        }
        if (W.w1) W.w3 = (char*)W.w1 + (size_t)m->F * d * m->wsz;
        A((void**)&W.attn_norm, d * 4);
        A((void**)&W.ffn_norm, d * 4);
    }
    A((void**)&m->xa, d * 4); A((void**)&m->xb, d * 4);
    A((void**)&m->qbuf, (size_t)m->nq * 4);
    A(&m->obuf, (size_t)m->nq * m->wsz);
    A(&m->gbuf, (size_t)m->F * m->wsz);
    A((void**)&m->part_wo, (size_t)tp * d * 4);
    A((void**)&m->part_w2, (size_t)tp * d * 4);
    A((void**)&m->logits_local, (size_t)m->V * 4);
    A((void**)&m->logits, (size_t)p->vocab_size * 4);
    A((void**)&m->scalars, 16 * sizeof(int32_t));
    m->tokens_cap = p->max_seq_len;
    A((void**)&m->tokens_out, (size_t)m->tokens_cap * sizeof(int32_t));
    // split attention over positions (64 per CTA at least) so that about three small CTAs per SM are busy
    int ns = (3 * ctx->sm_count + m->nh - 1) / m->nh;
    const int max_ns = (p->max_seq_len + 63) / 64;
    if (ns > max_ns) ns = max_ns;
    if (ns > 32) ns = 32;
    // up to 16 splits run as one thread-block cluster per head and merge through distributed shared memory
    if (ns > 16 && (getenv("RLB_ATTN_CLUSTER") == nullptr || atoi(getenv("RLB_ATTN_CLUSTER")) != 0)) ns = 16;
    if (ns < 1) ns = 1;
    if (const char* e = getenv("RLB_ATTN_SPLIT")) { int v = atoi(e); if (v >= 1 && v <= 64) ns = v; }
    m->n_split = ns;
    A((void**)&m->attn_scratch, attn_decode_scratch_floats(m->nh, hd, ns) * 4);
    A((void**)&m->attn_counters, (size_t)m->nh * sizeof(unsigned int));
    if (s == RLB_OK) {
        cudaError_t e = cudaMallocHost((void**)&m->h_scalars, 16 * sizeof(int32_t));
        if (e == cudaSuccess) e = cudaMallocHost((void**)&m->h_logits, (size_t)p->vocab_size * 4);
        if (e == cudaSuccess) e = cudaMallocHost((void**)&m->h_tokens, (size_t)m->tokens_cap * sizeof(int32_t));
        if (e == cudaSuccess) e = cudaMemsetAsync(m->attn_counters, 0, (size_t)m->nh * sizeof(unsigned int), ctx->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(m->scalars, 0, 16 * sizeof(int32_t), ctx->stream);
        if (e == cudaSuccess) {  // scalars[4]: decode-step epoch, starts at 1
            m->h_scalars[4] = 1;
            e = cudaMemcpyAsync(m->scalars + 4, m->h_scalars + 4, sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream);
        }
        if (e != cudaSuccess) s = rlb_fail(RLB_ERR_CUDA, "model buffers: %s", cudaGetErrorString(e));
    }
    if (s != RLB_OK) {
        rlb_model_free(m);
        return s;
    }
    if (const char* e = getenv("RLB_STREAM")) m->use_stream = atoi(e) != 0;
    if (const char* e = getenv("RLB_PDL")) m->use_pdl = atoi(e) != 0;
    if (const char* e = getenv("RLB_GRAPH")) m->use_graph = atoi(e) != 0;
    if (ctx->verbose)
        printf("model: dim %d layers %d heads %d (local %d from %d) ffn %d (local %d) vocab %d (local %d) %s tp %d/%d attn split %d\n", p->dim,
               p->n_layers, p->n_heads, m->nh, m->head0, p->ffn_dim, m->F, p->vocab_size, m->V, m->wdt == RLB_F16 ? "f16" : "f32", m->rank, tp,
               m->n_split);
    *out = m;
    return RLB_OK;
}

int rlb_model_set_tensor(rlb_model* m, rlb_tensor_kind kind, int32_t layer, const void* data, int64_t rows, int64_t cols,
                         int64_t capacity_cols, rlb_dtype dtype) {
    if (!m || !data) return rlb_fail(RLB_ERR_INVALID, "rlb_model_set_tensor: null pointer");
    if (dtype != RLB_F16 && dtype != RLB_F32) return rlb_fail(RLB_ERR_INVALID, "rlb_model_set_tensor: bad dtype");
    if (capacity_cols < cols) return rlb_fail(RLB_ERR_INVALID, "rlb_model_set_tensor: capacity_cols < cols");
    const bool per_layer = kind >= RLB_WQ && kind <= RLB_FFN_NORM;
    if (per_layer && (layer < 0 || layer >= m->p.n_layers)) return rlb_fail(RLB_ERR_INVALID, "layer %d out of range", layer);
    if (!per_layer) layer = 0;
    rlb_ctx* ctx = m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    const int64_t d = m->p.dim, F = m->p.ffn_dim, Vv = m->p.vocab_size;
    int64_t er = 0, ec = 0;             // expected full shape
    int64_t r0 = 0, nr = 0, c0 = 0, nc = 0;  // slice kept by this rank
    void* dst = nullptr; int64_t dst_ld = 0; rlb_dtype ddt = m->wdt;
    LayerW* W = per_layer ? &m->L[layer] : nullptr;
    // f32 data may carry more than f16's 11 significant bits: the prefill then keeps the exact f32 FMA GEMM
    if (kind >= RLB_WQ && kind <= RLB_W3 && dtype == RLB_F32) m->w_f16_exact = false;
    switch (kind) {
        case RLB_TOK_EMBEDDINGS: er = Vv; ec = d; nr = Vv; nc = d; dst = m->tok_emb; dst_ld = d; ddt = RLB_F32; break;
        case RLB_OUTPUT: er = Vv; ec = d; r0 = m->v0; nr = m->V; nc = d; dst = m->output; dst_ld = d; ddt = RLB_F32; break;
        case RLB_NORM: er = 1; ec = d; nr = 1; nc = d; dst = m->norm; dst_ld = d; ddt = RLB_F32; break;
        case RLB_ATTENTION_NORM: er = 1; ec = d; nr = 1; nc = d; dst = W->attn_norm; dst_ld = d; ddt = RLB_F32; break;
        case RLB_FFN_NORM: er = 1; ec = d; nr = 1; nc = d; dst = W->ffn_norm; dst_ld = d; ddt = RLB_F32; break;
        case RLB_WQ: case RLB_WK: case RLB_WV:
            er = d; ec = d; r0 = (int64_t)m->head0 * m->hd; nr = m->nq; nc = d;
            dst = (char*)W->wqkv + (size_t)(kind - RLB_WQ) * m->nq * d * m->wsz; dst_ld = d; break;
        case RLB_WO: er = d; ec = d; nr = d; c0 = (int64_t)m->head0 * m->hd; nc = m->nq; dst = W->wo; dst_ld = m->nq; break;
        case RLB_W1: er = F; ec = d; r0 = m->f0; nr = m->F; nc = d; dst = W->w1; dst_ld = d; break;
        case RLB_W3: er = F; ec = d; r0 = m->f0; nr = m->F; nc = d; dst = W->w3; dst_ld = d; break;
        case RLB_W2: er = d; ec = F; nr = d; c0 = m->f0; nc = m->F; dst = W->w2; dst_ld = m->F; break;
        default: return rlb_fail(RLB_ERR_INVALID, "unknown tensor kind %d", (int)kind);
    }
    // a matrix of a layer that is not resident in HBM goes to its place in the layer's pinned host block
    if (W && W->host && kind >= RLB_WQ && kind <= RLB_W3) dst = W->host + ((char*)dst - m->stage);
    // 1-D gains may arrive as [1][dim] or [dim][1]-like flat rows
    if (er == 1 && rows * cols == d) { rows = 1; cols = d; if (capacity_cols < d) capacity_cols = d; }
    if (rows != er || cols != ec)
        return rlb_fail(RLB_ERR_INVALID, "tensor kind %d layer %d: expected %lldx%lld, got %lldx%lld", (int)kind, layer, (long long)er,
                        (long long)ec, (long long)rows, (long long)cols);
    const size_t ssz = dtype_size(dtype);
    const char* src = (const char*)data + ((size_t)r0 * capacity_cols + c0) * ssz;
    if (dtype == ddt) {
        RLB_CUDA(cudaMemcpy2DAsync(dst, dst_ld * ssz, src, capacity_cols * ssz, (size_t)nc * ssz, (size_t)nr, cudaMemcpyDefault, ctx->stream));
        RLB_CUDA(cudaStreamSynchronize(ctx->stream));
    } else {
        void* tmp = nullptr;
        RLB_TRY(dev_alloc(&tmp, (size_t)nr * nc * ssz));
        cudaError_t e = cudaMemcpy2DAsync(tmp, nc * ssz, src, capacity_cols * ssz, (size_t)nc * ssz, (size_t)nr, cudaMemcpyDefault, ctx->stream);
        int s = RLB_OK;
        if (e != cudaSuccess) s = rlb_fail(RLB_ERR_CUDA, "set_tensor copy: %s", cudaGetErrorString(e));
        if (s == RLB_OK) s = launch_convert(ctx, tmp, dtype, nc, dst, ddt, dst_ld, nr, nc);
        cudaStreamSynchronize(ctx->stream);
        cudaFree(tmp);
        RLB_TRY(s);
    }
    m->have[(size_t)layer * 12 + kind] = 1;
    return RLB_OK;
}

int rlb_model_finalize(rlb_model* m) {
    if (!m) return rlb_fail(RLB_ERR_INVALID, "rlb_model_finalize: null model");
    rlb_ctx* ctx = m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    static const char* names[12] = {"tok_embeddings", "wq", "wk", "wv", "wo", "w1", "w2", "w3", "attention_norm", "ffn_norm", "norm", "output"};
    for (int k : {RLB_TOK_EMBEDDINGS, RLB_NORM, RLB_OUTPUT})
        if (!m->have[k]) return rlb_fail(RLB_ERR_STATE, "missing tensor %s", names[k]);  // UnpicklingError::MissingField
    for (int l = 0; l < m->p.n_layers; l++)
        for (int k = RLB_WQ; k <= RLB_FFN_NORM; k++)
            if (!m->have[(size_t)l * 12 + k]) return rlb_fail(RLB_ERR_STATE, "missing tensor layers.%d.%s", l, names[k]);
    // compute_freqs_cis (src/transformer.rs:858-885): f64 table, narrowed to f32 where it is applied
    const int hd = m->hd, T = m->p.max_seq_len;
    std::vector<float> tab((size_t)T * (hd / 2) * 2);
    for (int pos = 0; pos < T; pos++)
        for (int i = 0; i < hd / 2; i++) {
            const double freq = 1.0 / pow(10000.0, (double)i * 2.0 / (double)hd);
            const double ang = freq * (double)pos;
            tab[((size_t)pos * (hd / 2) + i) * 2 + 0] = (float)cos(ang);
            tab[((size_t)pos * (hd / 2) + i) * 2 + 1] = (float)sin(ang);
        }
    RLB_CUDA(cudaMemcpyAsync(m->rope, tab.data(), tab.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    RLB_CUDA(cudaStreamSynchronize(ctx->stream));
    m->finalized = true;
    return RLB_OK;
}

int rlb_model_free(rlb_model* m) {
    if (!m) return RLB_OK;
    rlb_ctx* ctx = m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    nccl_destroy(&m->nccl);
    for (int r = 0; r < m->tp; r++)
        if (m->peers_open && m->peers_ipc && r != m->rank && m->peer_xbuf[r]) cudaIpcCloseMemHandle(m->peer_xbuf[r]);
    if (m->xbuf) cudaFree(m->xbuf);
    void* ptrs[] = {m->tok_emb, m->norm, m->output, m->rope, m->xa, m->xb, m->qbuf, m->obuf, m->gbuf, m->part_wo, m->part_w2,
                    m->logits_local, m->logits, m->scalars, m->tokens_out, m->attn_scratch, m->attn_counters, m->pf_tokens, m->pf_x,
                    m->pf_a, m->pf_qkv, m->pf_o, m->pf_p, m->pf_g1, m->pf_g, m->pf_last};
    for (void* p : ptrs) if (p) cudaFree(p);
    for (auto& W : m->L) {
        if (W.host) {  // the matrix pointers address the shared staging buffer
            cudaFreeHost(W.host);
            W.wqkv = W.wo = W.w1 = W.w2 = nullptr;
        }
        void* lp[] = {W.wqkv, W.wo, W.w1, W.w2, W.attn_norm, W.ffn_norm};
        for (void* p : lp) if (p) cudaFree(p);
    }
    if (m->stage) cudaFree(m->stage);
    if (m->h_scalars) cudaFreeHost(m->h_scalars);
    if (m->h_logits) cudaFreeHost(m->h_logits);
    if (m->h_tokens) cudaFreeHost(m->h_tokens);
    for (auto& s : m->prof_slots) if (s.ev) cudaEventDestroy(s.ev);
    delete m;
    return RLB_OK;
}

int rlb_tp_nccl_unique_id(void* id128) {
    if (!id128) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_nccl_unique_id: null pointer");
    return nccl_unique_id(id128);
}

int rlb_tp_nccl_init(rlb_model* m, const void* id128) {
    if (!m || !id128) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_nccl_init: null pointer");
    std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
    RLB_CUDA(cudaSetDevice(m->ctx->device));
    if (m->tp == 1) return RLB_OK;
    return nccl_init(&m->nccl, id128, m->rank, m->tp);
}

int rlb_tp_peer_export(rlb_model* m, void* handle128) {
    if (!m || !handle128) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_peer_export: null pointer");
    std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
    RLB_CUDA(cudaSetDevice(m->ctx->device));
    if (m->tp == 1) return rlb_fail(RLB_ERR_STATE, "rlb_tp_peer_export: the model is not tensor parallel");
    if (!m->xbuf) {
        m->xbuf_bytes = xb_total(m);
        RLB_TRY(dev_alloc((void**)&m->xbuf, m->xbuf_bytes));
        RLB_CUDA(cudaMemset(m->xbuf, 0, m->xbuf_bytes));
    }
    static_assert(sizeof(cudaIpcMemHandle_t) <= RLB_TP_HANDLE_BYTES, "handle does not fit");
    cudaIpcMemHandle_t h;
    RLB_CUDA(cudaIpcGetMemHandle(&h, m->xbuf));
    memset(handle128, 0, RLB_TP_HANDLE_BYTES);
    memcpy(handle128, &h, sizeof(h));
    return RLB_OK;
}

int rlb_tp_peer_import(rlb_model* m, const void* handles, int32_t n_handles) {
    if (!m || !handles) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_peer_import: null pointer");
    std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
    RLB_CUDA(cudaSetDevice(m->ctx->device));
    if (n_handles != m->tp) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_peer_import: %d handles for %d ranks", n_handles, m->tp);
    if (!m->xbuf) return rlb_fail(RLB_ERR_STATE, "rlb_tp_peer_import: call rlb_tp_peer_export first");
    if (m->peers_open) return RLB_OK;
    for (int r = 0; r < m->tp; r++) {
        if (r == m->rank) { m->peer_xbuf[r] = m->xbuf; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)r * RLB_TP_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return rlb_fail(RLB_ERR_COMM, "cannot map the exchange buffer of rank %d: %s", r, cudaGetErrorString(e));
        m->peer_xbuf[r] = (char*)p;
    }
    m->peers_open = true;
    m->peers_ipc = true;
    return RLB_OK;
}

int rlb_tp_peer_import_local(rlb_model* m, rlb_model* const* peers, int32_t n_peers) {
    if (!m || !peers) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_peer_import_local: null pointer");
    if (n_peers != m->tp) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_peer_import_local: %d models for %d ranks", n_peers, m->tp);
    if (m->tp == 1) return rlb_fail(RLB_ERR_STATE, "rlb_tp_peer_import_local: the model is not tensor parallel");
    if (m->peers_open) return RLB_OK;
    for (int r = 0; r < m->tp; r++) {
        rlb_model* p = r == m->rank ? m : peers[r];
        if (!p) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_peer_import_local: no model for rank %d", r);
        if (p->tp != m->tp || p->rank != r || p->p.dim != m->p.dim || p->p.n_layers != m->p.n_layers || p->p.vocab_size != m->p.vocab_size)
            return rlb_fail(RLB_ERR_INVALID, "rlb_tp_peer_import_local: model %d is not rank %d of the same %d-way model", r, r, m->tp);
        {   // the peer's exchange buffer, allocated on its own device
            std::lock_guard<std::recursive_mutex> g(p->ctx->mu);
            RLB_CUDA(cudaSetDevice(p->ctx->device));
            if (!p->xbuf) {
                p->xbuf_bytes = xb_total(p);
                RLB_TRY(dev_alloc((void**)&p->xbuf, p->xbuf_bytes));
                RLB_CUDA(cudaMemset(p->xbuf, 0, p->xbuf_bytes));
            }
        }
        std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
        RLB_CUDA(cudaSetDevice(m->ctx->device));
        if (p->ctx->device != m->ctx->device) {
            int can = 0;
            RLB_CUDA(cudaDeviceCanAccessPeer(&can, m->ctx->device, p->ctx->device));
            if (!can) return rlb_fail(RLB_ERR_COMM, "device %d cannot access the memory of device %d", m->ctx->device, p->ctx->device);
            cudaError_t e = cudaDeviceEnablePeerAccess(p->ctx->device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (e != cudaSuccess) return rlb_fail(RLB_ERR_COMM, "cudaDeviceEnablePeerAccess(%d): %s", p->ctx->device, cudaGetErrorString(e));
        }
        m->peer_xbuf[r] = p->xbuf;
    }
    m->peers_open = true;
    m->peers_ipc = false;
    return RLB_OK;
}

int rlb_tp_set_mode(rlb_model* m, int32_t mode) {
    if (!m) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_set_mode: null model");
    std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
    if (mode != 0 && mode != 1) return rlb_fail(RLB_ERR_INVALID, "rlb_tp_set_mode: unknown mode %d", mode);
    if (mode == 1 && m->tp > 1 && !m->peers_open) return rlb_fail(RLB_ERR_STATE, "rlb_tp_set_mode: peer exchange buffers are not imported");
    if (mode == 1 && !m->use_stream) return rlb_fail(RLB_ERR_STATE, "rlb_tp_set_mode: the push mode needs the staged GEMV kernels");
    if (m->tp_mode != mode) m->graph_gen++;
    m->tp_mode = mode;
    return RLB_OK;
}

int rlb_caches_create(rlb_model* m, rlb_caches** out) {
    if (!m || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_caches_create: null pointer");
    *out = nullptr;
    rlb_ctx* ctx = m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    rlb_caches* c = new rlb_caches();
    c->m = m;
    c->layer_elems = (size_t)m->nh * m->p.max_seq_len * m->hd;
    const size_t bytes = cache_bytes(m);
    int s = dev_alloc(&c->k, bytes);
    if (s == RLB_OK) s = dev_alloc(&c->v, bytes);
    if (s == RLB_OK) {
        cudaError_t e = cudaMemsetAsync(c->k, 0, bytes, ctx->stream);  // Tensor::zeros (src/transformer.rs:144-153)
        if (e == cudaSuccess) e = cudaMemsetAsync(c->v, 0, bytes, ctx->stream);
        if (e != cudaSuccess) s = rlb_fail(RLB_ERR_CUDA, "cache memset: %s", cudaGetErrorString(e));
    }
    if (s != RLB_OK) {
        rlb_caches_free(c);
        return s;
    }
    *out = c;
    return RLB_OK;
}

int rlb_caches_true_clone(rlb_caches* src, rlb_caches** out) {
    if (!src || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_caches_true_clone: null pointer");
    RLB_TRY(rlb_caches_create(src->m, out));
    rlb_ctx* ctx = src->m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    const size_t bytes = cache_bytes(src->m);
    RLB_CUDA(cudaMemcpyAsync((*out)->k, src->k, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    RLB_CUDA(cudaMemcpyAsync((*out)->v, src->v, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return RLB_OK;
}

int rlb_caches_shift_left(rlb_caches* c, int32_t shifts) {
    if (!c) return rlb_fail(RLB_ERR_INVALID, "rlb_caches_shift_left: null pointer");
    if (shifts < 0) return rlb_fail(RLB_ERR_INVALID, "rlb_caches_shift_left: negative shift");
    rlb_model* m = c->m;
    std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
    RLB_CUDA(cudaSetDevice(m->ctx->device));
    const int64_t heads = (int64_t)m->p.n_layers * m->nh;
    RLB_TRY(launch_cache_shift_left(m->ctx, c->k, m->wdt, heads, m->p.max_seq_len, m->hd, shifts));
    RLB_TRY(launch_cache_shift_left(m->ctx, c->v, m->wdt, heads, m->p.max_seq_len, m->hd, shifts));
    return RLB_OK;
}

int rlb_caches_free(rlb_caches* c) {
    if (!c) return RLB_OK;
    rlb_ctx* ctx = c->m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (c->graph) cudaGraphExecDestroy(c->graph);
    if (c->graph_adv) cudaGraphExecDestroy(c->graph_adv);
    if (c->k) cudaFree(c->k);
    if (c->v) cudaFree(c->v);
    delete c;
    return RLB_OK;
}

int rlb_caches_read(rlb_caches* c, int32_t which, int32_t layer, int32_t head, int32_t pos, float* out) {
    if (!c || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_caches_read: null pointer");
    rlb_model* m = c->m;
    if (layer < 0 || layer >= m->p.n_layers || head < 0 || head >= m->nh || pos < 0 || pos >= m->p.max_seq_len || (which != 0 && which != 1))
        return rlb_fail(RLB_ERR_INVALID, "rlb_caches_read: index out of range");
    std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
    RLB_CUDA(cudaSetDevice(m->ctx->device));
    const char* base = (const char*)(which == 0 ? c->k : c->v);
    const size_t off = ((size_t)layer * c->layer_elems + ((size_t)head * m->p.max_seq_len + pos) * m->hd) * m->wsz;
    std::vector<uint16_t> tmp(m->hd * 2);
    RLB_CUDA(cudaStreamSynchronize(m->ctx->stream));
    RLB_CUDA(cudaMemcpy(tmp.data(), base + off, (size_t)m->hd * m->wsz, cudaMemcpyDeviceToHost));
    if (m->wdt == RLB_F16) {
        for (int i = 0; i < m->hd; i++) {
            __half_raw r;
            r.x = tmp[i];
            out[i] = __half2float(__half(r));
        }
    } else {
        memcpy(out, tmp.data(), (size_t)m->hd * 4);
    }
    return RLB_OK;
}

int rlb_forward(rlb_model* m, rlb_caches* c, const int32_t* tokens, int32_t n, int32_t start_pos, float* logits_out) {
    RLB_TRY(check_forward_args(m, c, tokens, n, start_pos));
    if (!logits_out) return rlb_fail(RLB_ERR_INVALID, "forward: null logits pointer");
    rlb_ctx* ctx = m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    RLB_TRY(forward_common(m, c, tokens, n, start_pos, false));
    RLB_CUDA(cudaMemcpyAsync(m->h_logits, m->logits, (size_t)m->p.vocab_size * 4, cudaMemcpyDeviceToHost, ctx->stream));
    RLB_CUDA(cudaMemcpyAsync(m->h_scalars + 9, m->scalars + 8, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    RLB_CUDA(cudaStreamSynchronize(ctx->stream));
    RLB_TRY(check_device_flag(m->h_scalars + 9));
    memcpy(logits_out, m->h_logits, (size_t)m->p.vocab_size * 4);
    return RLB_OK;
}

int rlb_forward_greedy(rlb_model* m, rlb_caches* c, const int32_t* tokens, int32_t n, int32_t start_pos, int32_t* next_token) {
    RLB_TRY(check_forward_args(m, c, tokens, n, start_pos));
    if (!next_token) return rlb_fail(RLB_ERR_INVALID, "forward_greedy: null output pointer");
    rlb_ctx* ctx = m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    RLB_TRY(forward_common(m, c, tokens, n, start_pos, true));
    RLB_CUDA(cudaMemcpyAsync(m->h_scalars + 8, m->scalars + 3, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    RLB_CUDA(cudaMemcpyAsync(m->h_scalars + 9, m->scalars + 8, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    RLB_CUDA(cudaStreamSynchronize(ctx->stream));
    RLB_TRY(check_device_flag(m->h_scalars + 9));
    *next_token = m->h_scalars[8];
    return RLB_OK;
}

int rlb_decode_greedy(rlb_model* m, rlb_caches* c, int32_t first_token, int32_t start_pos, int32_t n_steps, int32_t* tokens_out,
                      float* elapsed_ms) {
    RLB_TRY(check_forward_args(m, c, &first_token, 1, start_pos));
    if (!tokens_out || n_steps < 1) return rlb_fail(RLB_ERR_INVALID, "decode_greedy: bad arguments");
    if (start_pos + n_steps > m->p.max_seq_len) return rlb_fail(RLB_ERR_INVALID, "decode_greedy: %d steps from %d exceed max_seq_len %d", n_steps, start_pos, m->p.max_seq_len);
    if (n_steps > m->tokens_cap) return rlb_fail(RLB_ERR_LIMIT, "decode_greedy: more than %d steps", m->tokens_cap);
    rlb_ctx* ctx = m->ctx;
    std::lock_guard<std::recursive_mutex> g(ctx->mu);
    RLB_CUDA(cudaSetDevice(ctx->device));
    static thread_local cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (!e0) { RLB_CUDA(cudaEventCreate(&e0)); RLB_CUDA(cudaEventCreate(&e1)); }
    m->h_scalars[0] = first_token; m->h_scalars[1] = start_pos; m->h_scalars[2] = 0; m->h_scalars[3] = 0;
    RLB_CUDA(cudaMemcpyAsync(m->scalars, m->h_scalars, 4 * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
    cudaGraphExec_t& slot = c->graph_adv;
    int done = 0;
    // Not part of the timed region: the eager first step on fresh caches and, under tensor parallelism, one
    // step after which the ranks are aligned by the exchange itself (else the skew the host left between
    // the ranks' launches is timed)
    if (!c->warmed || (m->tp > 1 && n_steps > 1)) {
        RLB_TRY(run_decode_step(m, c, true, &slot));
        done = 1;
    }
    RLB_CUDA(cudaEventRecord(e0, ctx->stream));
    for (int i = done; i < n_steps; i++) RLB_TRY(run_decode_step(m, c, true, &slot));
    RLB_CUDA(cudaEventRecord(e1, ctx->stream));
    RLB_CUDA(cudaMemcpyAsync(m->h_tokens, m->tokens_out, (size_t)n_steps * sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    RLB_CUDA(cudaMemcpyAsync(m->h_scalars + 9, m->scalars + 8, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    RLB_CUDA(cudaStreamSynchronize(ctx->stream));
    RLB_TRY(check_device_flag(m->h_scalars + 9));
    memcpy(tokens_out, m->h_tokens, (size_t)n_steps * sizeof(int32_t));
    if (elapsed_ms) {
        float ms = 0.f;
        RLB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        *elapsed_ms = (n_steps - done) > 0 ? ms * (float)n_steps / (float)(n_steps - done) : 0.f;
    }
    return RLB_OK;
}

int rlb_model_set_option(rlb_model* m, const char* name, int64_t value) {
    if (!m || !name) return rlb_fail(RLB_ERR_INVALID, "rlb_model_set_option: null pointer");
    std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
    if (!strcmp(name, "graph")) { m->use_graph = value != 0; return RLB_OK; }
    if (!strcmp(name, "stream_gemv")) { m->use_stream = value != 0; return RLB_OK; }
    if (!strcmp(name, "pdl")) { m->use_pdl = value != 0; return RLB_OK; }
    if (!strcmp(name, "profile")) {
        m->profile = value != 0;
        for (double& v : m->prof_ms) v = 0;
        m->prof_steps = 0;
        m->prof_used = 0;
        return RLB_OK;
    }
    if (!strcmp(name, "gemv_rows")) { gemv_set_tuning((int)value, 0, 0); return RLB_OK; }
    return rlb_fail(RLB_ERR_INVALID, "unknown option %s", name);
}

int rlb_model_get_stat(rlb_model* m, const char* name, double* value) {
    if (!m || !name || !value) return rlb_fail(RLB_ERR_INVALID, "rlb_model_get_stat: null pointer");
    std::lock_guard<std::recursive_mutex> g(m->ctx->mu);
    if (!strcmp(name, "kernels_per_step")) { *value = (double)m->kernels_per_step; return RLB_OK; }
    if (!strcmp(name, "attn_split")) { *value = m->n_split; return RLB_OK; }
    if (!strcmp(name, "prof_steps")) { *value = m->prof_steps; return RLB_OK; }
    if (!strcmp(name, "local_heads")) { *value = m->nh; return RLB_OK; }
    if (!strcmp(name, "layers_on_gpu")) { *value = m->gpu_layers; return RLB_OK; }
    if (!strcmp(name, "first_head")) { *value = m->head0; return RLB_OK; }
    if (!strcmp(name, "local_ffn")) { *value = m->F; return RLB_OK; }
    if (!strcmp(name, "local_vocab")) { *value = m->V; return RLB_OK; }
    if (!strcmp(name, "vocab_size")) { *value = m->p.vocab_size; return RLB_OK; }
    if (!strcmp(name, "ffn_dim")) { *value = m->p.ffn_dim; return RLB_OK; }
    if (!strncmp(name, "prof_ms_", 8)) {
        for (int i = 0; i < PC_COUNT; i++)
            if (!strcmp(name + 8, kProfNames[i])) { *value = m->prof_ms[i]; return RLB_OK; }
    }
    return rlb_fail(RLB_ERR_INVALID, "unknown statistic %s", name);
}

}  // extern "C"

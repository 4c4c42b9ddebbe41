/*
 * rllama_b200.h -- C ABI of the B200 (sm_100a) backend for rllama's decode / prefill path.
 *
 * The library replaces rllama's OpenCL backend (src/tensor_opencl_support.rs) and the
 * CPU arithmetic below Transformer::forward (src/transformer.rs:343-382). It is what a
 * Rust `extern "C"` block built from build.rs would bind. Plain pointers and sizes only.
 *
 * Conventions
 *  - every function returns an int status: 0 = RLB_OK, otherwise an rlb_status code; no
 *    function aborts. rlb_last_error() gives the message of the last failure on the
 *    calling thread.
 *  - f16 values cross the boundary as uint16_t bit patterns; matrices are row-major and
 *    are described by (rows, cols, capacity_cols, dtype) exactly as rllama's Tensor
 *    describes them (src/tensor.rs:103-112): capacity_cols is the row stride in elements.
 *  - handles are opaque. Functions may be called from any host thread; calls that touch
 *    the same model are serialised inside the library.
 *  - there is no CPU fallback: without a usable sm_100 device rlb_ctx_create fails.
 */
#ifndef RLLAMA_B200_H
#define RLLAMA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum rlb_status {
    RLB_OK = 0,
    RLB_ERR_INVALID = 1,  /* bad argument, shape or dtype (the reference panics here)   */
    RLB_ERR_CUDA = 2,     /* a CUDA runtime call failed                                  */
    RLB_ERR_NO_DEVICE = 3,/* no usable device / wrong architecture                       */
    RLB_ERR_OOM = 4,      /* device allocation failed                                    */
    RLB_ERR_STATE = 5,    /* call order violated (e.g. forward before finalize)          */
    RLB_ERR_COMM = 6,     /* tensor-parallel exchange failed or timed out                */
    RLB_ERR_LIMIT = 7     /* a size is beyond a documented maximum                       */
} rlb_status;

typedef enum rlb_dtype {  /* TensorDType (src/tensor.rs:81-101) */
    RLB_F32 = 0,
    RLB_F16 = 1
} rlb_dtype;

typedef struct rlb_ctx rlb_ctx;        /* replaces `OpenCL`       (src/tensor_opencl_support.rs:30-37) */
typedef struct rlb_tensor rlb_tensor;  /* replaces `OpenCLTensor` (src/tensor_opencl_support.rs:39-52) */
typedef struct rlb_event rlb_event;    /* replaces `OpenCLEvent`  (src/tensor_opencl_support.rs:54-57) */
typedef struct rlb_model rlb_model;    /* `Transformer`           (src/transformer.rs:22-36)           */
typedef struct rlb_caches rlb_caches;  /* `TransformerCaches`     (src/transformer.rs:111-113)         */

/* Message of the last failure on the calling thread ("" if none). Never NULL. */
const char* rlb_last_error(void);

/* Number of CUDA devices visible to the process. */
int rlb_device_count(int* count);

/* ------------------------------------------------------------------------------------
 * Tier 1: op-level mirror of OpenCLTensor, so tensor.rs can swap backends one to one.
 * ---------------------------------------------------------------------------------- */

/* OpenCL::new(verbose, nth_device) (src/tensor_opencl_support.rs:86-128). Selects the
 * nth CUDA device, checks that it is compute capability 10.x, creates the stream.     */
int rlb_ctx_create(int verbose, int nth_device, rlb_ctx** out);
int rlb_ctx_destroy(rlb_ctx* ctx);
/* OpenCL::flush (src/tensor_opencl_support.rs:130-132): waits for all queued work.    */
int rlb_ctx_flush(rlb_ctx* ctx);
/* How many kernels this library has launched on ctx so far (graph replays count every
 * kernel node they run).                                                              */
int rlb_ctx_kernel_launches(rlb_ctx* ctx, uint64_t* count);

/* OpenCL::data_u16_to_gpu (src/tensor_opencl_support.rs:134-169), for f16 and f32.
 * The copy is asynchronous: `host` must stay valid until rlb_tensor_wait returns.     */
int rlb_tensor_upload(rlb_ctx* ctx, const void* host, int64_t rows, int64_t cols,
                      int64_t capacity_cols, rlb_dtype dtype, rlb_tensor** out);
/* A zero-filled device tensor (the reference uploads a zeroed host tensor for results,
 * src/tensor.rs:1016-1021).                                                           */
int rlb_tensor_zeros(rlb_ctx* ctx, int64_t rows, int64_t cols, int64_t capacity_cols,
                     rlb_dtype dtype, rlb_tensor** out);
/* OpenCLTensor::wait_until_ready (src/tensor_opencl_support.rs:177-196).              */
int rlb_tensor_wait(rlb_tensor* t);
/* OpenCLTensor::data_u16_from_gpu (src/tensor_opencl_support.rs:198-212): asynchronous
 * read of rows*capacity_cols elements into `host`; complete after rlb_event_wait.     */
int rlb_tensor_download(rlb_tensor* t, void* host, rlb_event** out_event);
/* OpenCLEvent::wait (src/tensor_opencl_support.rs:409-412); also frees the event.     */
int rlb_event_wait(rlb_event* ev);
/* Drop for OpenCLTensor (src/tensor_opencl_support.rs:59-75).                         */
int rlb_tensor_free(rlb_tensor* t);

/* OpenCLTensor::copy_inplace (src/tensor_opencl_support.rs:215-232): dst <- src.      */
int rlb_copy_inplace(rlb_tensor* dst, const rlb_tensor* src);
/* OpenCLTensor::transpose_from (src/tensor_opencl_support.rs:234-256): dst <- src^T.  */
int rlb_transpose_from(rlb_tensor* dst, const rlb_tensor* src);
/* OpenCLTensor::hadamard_product_inplace (src/tensor_opencl_support.rs:258-281).      */
int rlb_hadamard_product_inplace(rlb_tensor* dst, const rlb_tensor* other);
/* OpenCLTensor::silu_inplace (src/tensor_opencl_support.rs:283-299).                  */
int rlb_silu_inplace(rlb_tensor* t);
/* OpenCLTensor::matrix_mul_inplace_transposed (src/tensor_opencl_support.rs:301-407):
 * dst[i][j] = sum_k src[i][k] * other[j][k]; f32 accumulation; f16 operands give an
 * f16-rounded result. Dispatches on the row counts: a one-row operand takes the
 * bandwidth-bound GEMV kernel, otherwise the tiled GEMM (tcgen05 for f16).            */
int rlb_matrix_mul_inplace_transposed(rlb_tensor* dst, const rlb_tensor* src, const rlb_tensor* other);

/* Single-query attention over a position-major KV cache: the per-head part of
 * Attention::forward at decode (src/transformer.rs:727-781) as a standalone op.
 *   q       1 x (heads*head_dim) f32, already rotated
 *   kcache  (heads*max_seq_len) x head_dim, f16 or f32, capacity_cols == head_dim:
 *   vcache  row (h*max_seq_len + t) holds head h, position t
 *   out     1 x (heads*head_dim) in the cache dtype (f16 results are rounded once)
 * Attends to positions 0..pos. n_split > 1 splits the positions of each head over that
 * many CTAs and combines their partial results (1..64). Scratch for the partial results
 * is owned by the context and grown on demand.                                        */
int rlb_attention_decode(rlb_tensor* out, const rlb_tensor* q, const rlb_tensor* kcache, const rlb_tensor* vcache,
                         int32_t heads, int32_t max_seq_len, int32_t pos, int32_t n_split);

/* The same per-head attention for a multi-token call (the prefill half of Attention::forward,
 * src/transformer.rs:727-781, with the causal mask of Tensor::full_triu, src/tensor.rs:496-508):
 *   q    n x (heads*head_dim) f32, already rotated; row i attends to positions 0..start_pos+i
 *   out  n x (heads*head_dim) in the cache dtype, no row padding
 * f16 caches with head_dim 64 or 128 and n >= 32 run on the tensor cores (q and the softmax
 * weights split into two f16 halves, so no rounding point is added); tensor_cores = 0 keeps
 * the call on the CUDA-core kernel (for comparisons).                                    */
int rlb_attention_prefill(rlb_tensor* out, const rlb_tensor* q, const rlb_tensor* kcache, const rlb_tensor* vcache,
                          int32_t heads, int32_t max_seq_len, int32_t start_pos, int32_t tensor_cores);

/* rlb_attention_decode without any allocation (no counterpart in the reference). For hosts
 * that cannot let the library allocate on the token path: a server whose HBM is already
 * split between weights and KV caches, or a latency-critical thread that must not stall the
 * device in cudaMalloc / cudaFree. The split-attention scratch is a fixed 1 MiB (+ 1.25 KiB
 * header) array inside the library, held by every GPU that loads it until the process ends.
 * Same arguments and results as rlb_attention_decode. Fails with RLB_ERR_LIMIT when
 * heads > 256 or heads * n_split * (head_dim + 2) > 262144 floats. All calls on one device
 * share the array: calls that overlap on the GPU race, so serialise them. The first call on
 * a device resolves the array's device address; make it before any stream capture.      */
int rlb_attention_decode_static(rlb_tensor* out, const rlb_tensor* q, const rlb_tensor* kcache, const rlb_tensor* vcache,
                                int32_t heads, int32_t max_seq_len, int32_t pos, int32_t n_split);

/* ------------------------------------------------------------------------------------
 * Tier 2: the fused model-level path (what Transformer::forward becomes).
 * ---------------------------------------------------------------------------------- */

typedef enum rlb_tensor_kind {  /* checkpoint tensors rllama looks up */
    RLB_TOK_EMBEDDINGS = 0,     /* tok_embeddings.weight (src/embedding.rs:17)           */
    RLB_WQ = 1,                 /* layers.N.attention.wq.weight (src/transformer.rs:594) */
    RLB_WK = 2,
    RLB_WV = 3,
    RLB_WO = 4,                 /* (src/transformer.rs:612)                              */
    RLB_W1 = 5,                 /* layers.N.feed_forward.w1.weight (:489)                */
    RLB_W2 = 6,
    RLB_W3 = 7,
    RLB_ATTENTION_NORM = 8,     /* layers.N.attention_norm.weight (:400-413)             */
    RLB_FFN_NORM = 9,
    RLB_NORM = 10,              /* norm.weight (:296-301)                                */
    RLB_OUTPUT = 11             /* output.weight, always kept in f32 (:302-308)          */
} rlb_tensor_kind;

typedef struct rlb_model_params {
    int32_t dim;          /* ModelParams.dim        (src/model_params.rs:4-14)           */
    int32_t n_layers;
    int32_t n_heads;
    int32_t ffn_dim;      /* rows of w1; the reference infers it from the tensor         */
    int32_t vocab_size;
    int32_t max_seq_len;  /* --max-seq-len (src/rllama_main.rs:247)                      */
    float norm_eps;
    int32_t force_f16;    /* DataSettings::force_f16 (src/transformer.rs:105-108): the 7
                             per-layer matrices and the KV cache are f16; else f32      */
    int32_t tp_rank;      /* tensor-parallel rank of this process, 0 <= rank < tp_size   */
    int32_t tp_size;      /* 1, 2, 4 or 8; heads and FFN columns are split               */
    int32_t has_percentage_to_gpu;  /* 0: every layer is resident in HBM (the default, 1.0)  */
    float percentage_to_gpu;  /* DataSettings::percentage_to_gpu (src/transformer.rs:91-103,
                             --percentage-to-gpu): clamped to [0, 1], NaN -> 0; layer i is
                             resident in HBM iff i <= round(p * (n_layers - 1)) (:262-274).
                             There is no CPU path: the other layers' matrices stay in pinned
                             host memory and are copied into one HBM staging buffer, layer by
                             layer, inside every forward call (same kernels, same results). */
} rlb_model_params;

/* Transformer::from_unpickled (src/transformer.rs:242-326), construction half.        */
int rlb_model_create(rlb_ctx* ctx, const rlb_model_params* params, rlb_model** out);
/* One checkpoint tensor, given WHOLE (all tensor-parallel ranks pass the same data);
 * the library keeps this rank's slice along the axis the reference concatenates shards
 * on: rows for wq wk wv w1 w3 output, columns for wo w2 (src/transformer.rs:489-506,
 * :594-617, :302-307). `data` may be host or device memory, f16 or f32; it is converted
 * to the model's weight dtype as the reference does (always widened, then to f16 under
 * force_f16). Synchronous: `data` may be reused on return.                             */
int rlb_model_set_tensor(rlb_model* m, rlb_tensor_kind kind, int32_t layer, const void* data,
                         int64_t rows, int64_t cols, int64_t capacity_cols, rlb_dtype dtype);
/* Checks that every tensor was given, builds the RoPE table (src/transformer.rs:858-885). */
int rlb_model_finalize(rlb_model* m);
/* Frees the model. Its caches (rlb_caches_*) refer to it: free them first.                */
int rlb_model_free(rlb_model* m);

/* Tensor-parallel wiring, one process per GPU. Either
 *  (a) NCCL: every rank passes the same 128-byte ncclUniqueId (rank 0 obtains it with
 *      rlb_tp_nccl_unique_id and the caller broadcasts it), or
 *  (b) peer memory: every rank exports a handle to its exchange buffer, the caller
 *      all-gathers the handles and gives every rank the full list.
 * Both can be active; rlb_tp_set_mode picks which one forward uses. No counterpart in
 * the reference, which is single-device (src/transformer.rs:254-256).                  */
#define RLB_TP_HANDLE_BYTES 128
int rlb_tp_nccl_unique_id(void* id128);
int rlb_tp_nccl_init(rlb_model* m, const void* id128);
int rlb_tp_peer_export(rlb_model* m, void* handle128);
int rlb_tp_peer_import(rlb_model* m, const void* handles, int32_t n_handles);
/* (b) for ranks that live in ONE process (one host thread or several, one context per GPU): the
 * models of all ranks, indexed by rank (the entry of m's own rank may be m or NULL). Exchange
 * buffers are allocated as needed and peer access between the devices is enabled. No counterpart
 * in the reference.                                                                       */
int rlb_tp_peer_import_local(rlb_model* m, rlb_model* const* peers, int32_t n_peers);
/* mode: 0 = NCCL all-reduce / all-gather, 1 = fused push exchange over peer memory (needs
 * rlb_tp_peer_import; prefill keeps using NCCL). Every rank must switch at the same step. */
int rlb_tp_set_mode(rlb_model* m, int32_t mode);

/* Transformer::make_caches (src/transformer.rs:328-341).                              */
int rlb_caches_create(rlb_model* m, rlb_caches** out);
/* TransformerCaches::true_clone (src/transformer.rs:207-213).                         */
int rlb_caches_true_clone(rlb_caches* src, rlb_caches** out);
/* TransformerCaches::shift_left (src/transformer.rs:200-205).                         */
int rlb_caches_shift_left(rlb_caches* c, int32_t shifts);
int rlb_caches_free(rlb_caches* c);
/* Reads this rank's cached K (which = 0) or V (1) values for one layer/head/position
 * into out[head_dim] as f32 (inspection; the reference exposes its cache tensors).    */
int rlb_caches_read(rlb_caches* c, int32_t which, int32_t layer, int32_t head, int32_t pos, float* out);

/* Transformer::forward(tokens, start_pos, caches) (src/transformer.rs:343-382):
 * n >= 1 tokens at positions start_pos..start_pos+n, returns the vocab_size f32 logits
 * of the LAST token in host memory. n == 1 is the decode step; n > 1 the prefill.
 * (The reference panics for n > 1 with start_pos > 0; here that is a causal chunk.)    */
int rlb_forward(rlb_model* m, rlb_caches* c, const int32_t* tokens, int32_t n, int32_t start_pos,
                float* logits_out);
/* Same, but only the arg-max token id comes back (greedy, TokenSampler with top_k 1,
 * src/token_sampler.rs:20-28): the lowest id among equal maxima.                       */
int rlb_forward_greedy(rlb_model* m, rlb_caches* c, const int32_t* tokens, int32_t n, int32_t start_pos,
                       int32_t* next_token);
/* Greedy generation with the token fed back on the device: starting from `first_token`
 * at position start_pos, runs n_steps decode steps (the loop of
 * src/rllama_main.rs:821-901 with sampling reduced to arg-max). tokens_out[n_steps]
 * receives the generated ids; *elapsed_ms (may be NULL) the device time of the loop
 * measured with events on the model's stream.                                          */
int rlb_decode_greedy(rlb_model* m, rlb_caches* c, int32_t first_token, int32_t start_pos, int32_t n_steps,
                      int32_t* tokens_out, float* elapsed_ms);

/* ------------------------------------------------------------------------------------
 * Checkpoint loading (host side): the unzipped Meta LLaMA layout rllama reads.
 * ---------------------------------------------------------------------------------- */
typedef struct rlb_data_source rlb_data_source;  /* `DataSource::LLaMASource` (src/data_source.rs:22-30) */

/* DataSource::from_llama_source (src/data_source.rs:166-196): unpickles
 * <model_path>/consolidated.NN/data.pkl for NN = 00, 01, ... until one is missing.      */
int rlb_data_source_open(const char* model_path, rlb_data_source** out);
int rlb_data_source_free(rlb_data_source* ds);
int rlb_data_source_shards(rlb_data_source* ds, int32_t* n_shards);
/* Shape of a named tensor after concatenating its shards. direction: 0 = along rows,
 * 1 = along columns (FromPiecesDirection, src/tensor.rs:2340-2343), 2 = first shard only
 * (Tensor::from_unpickled_pieces1, src/tensor.rs:309-329).                               */
int rlb_data_source_tensor_shape(rlb_data_source* ds, const char* name, int32_t direction, int64_t* rows, int64_t* cols);
/* TensorBuilder::load_from_pieces (src/tensor.rs:2388-2545): reads the f16 rows of every
 * shard from consolidated.NN/data/<key> into out[rows][cols] (dense, f16 bit patterns).  */
int rlb_data_source_read_f16(rlb_data_source* ds, const char* name, int32_t direction, uint16_t* out, int64_t rows, int64_t cols);
/* DataSource::from_vicuna_source (src/data_source.rs:206-215): a HuggingFace directory
 * (config.json, pytorch_model.bin.index.json, *.bin torch.save archives read in place).   */
int rlb_data_source_open_vicuna(const char* model_path, rlb_data_source** out);
/* DataSource::from_inferred_source (src/data_source.rs:188-204): params.json -> Meta's
 * layout, pytorch_model.bin.index.json -> HuggingFace's, else "Unknown source".           */
int rlb_data_source_open_inferred(const char* model_path, rlb_data_source** out);
/* DataSource::need_to_do_antitranspose (src/data_source.rs:223-228).                      */
int rlb_data_source_need_antitranspose(rlb_data_source* ds, int32_t* yes);
/* Tensor::huggingface_llama_model_antitranspose (src/tensor.rs:841-909) on dense f16 rows:
 * dst row h*hd + 2j + t = src row h*hd + t*hd/2 + j, hd = rows / n_heads.                 */
int rlb_huggingface_antitranspose_f16(const uint16_t* src, uint16_t* dst, int64_t rows, int64_t cols, int32_t n_heads);
/* ModelParams from params.json (src/model_params.rs:4-14, src/rllama_main.rs:201-241):
 * fills dim, n_heads, n_layers, norm_eps, vocab_size (HF aliases accepted); the other
 * fields of *out are left untouched.                                                     */
int rlb_model_params_from_json(const char* path, rlb_model_params* out);
/* Transformer::from_unpickled (src/transformer.rs:242-326) with Embedding::from_unpickled
 * (src/embedding.rs:13-48): creates the model and loads every tensor by its Meta name.
 * ffn_dim and vocab_size of *params are ignored: they come from the w1 and embedding
 * tensors, as in the reference. Every tensor-parallel rank reads the whole checkpoint and
 * keeps its slice.                                                                       */
int rlb_model_from_llama_source(rlb_ctx* ctx, rlb_data_source* ds, const rlb_model_params* params, rlb_model** out);

/* ------------------------------------------------------------------------------------
 * Host-side callers of the path: tokenizer and sampler of the generation loop
 * (src/rllama_main.rs:814-901).
 * ---------------------------------------------------------------------------------- */
typedef struct rlb_tokenizer rlb_tokenizer;  /* `Tokenizer` (src/tokenizer.rs:11-14) */
typedef struct rlb_sampler rlb_sampler;      /* `TokenSampler` (src/token_sampler.rs:6-11) */

/* Tokenizer::load (src/tokenizer.rs:46-96): a SentencePiece ModelProto file.          */
int rlb_tokenizer_load(const char* path, rlb_tokenizer** out);
int rlb_tokenizer_free(rlb_tokenizer* tk);
/* Number of pieces in the model file (indices run 0 .. n-1; pieces without text and
 * earlier duplicates of a text have no entry).                                          */
int rlb_tokenizer_n_pieces(rlb_tokenizer* tk, int32_t* n);
/* Tokenizer::id_to_str (src/tokenizer.rs:100-108). The reference panics on an unknown
 * id; this returns RLB_ERR_INVALID. *out stays valid until rlb_tokenizer_free.          */
int rlb_tokenizer_id_to_str(rlb_tokenizer* tk, int32_t id, const char** out);
/* Tokenizer::str_to_id (src/tokenizer.rs:111-118): *id = -1 when there is no such piece. */
int rlb_tokenizer_str_to_id(rlb_tokenizer* tk, const char* s, int32_t* id);
/* Tokenizer::tokenize_to_ids (src/tokenizer.rs:166-178): start token 1, then the greedy
 * longest-prefix pieces of "\u2581" + text with spaces replaced by "\u2581". *n receives
 * the count; ids may be NULL to query it, else RLB_ERR_LIMIT when cap is too small.      */
int rlb_tokenizer_tokenize_to_ids(rlb_tokenizer* tk, const char* text, int32_t* ids, int32_t cap, int32_t* n);

/* TokenSampler::new (src/token_sampler.rs:20-28): temperature 0.2, top_p 1.0, top_k 1,
 * repetition_penalty 0.8.                                                               */
int rlb_sampler_create(rlb_sampler** out);
int rlb_sampler_free(rlb_sampler* s);
/* The four builder setters / getters (src/token_sampler.rs:30-66) in one call each.     */
int rlb_sampler_set(rlb_sampler* s, float temperature, float top_p, int32_t top_k, float repetition_penalty);
int rlb_sampler_get(rlb_sampler* s, float* temperature, float* top_p, int32_t* top_k, float* repetition_penalty);
/* No counterpart in the reference (it draws from rand::thread_rng): seeds the draw.     */
int rlb_sampler_seed(rlb_sampler* s, uint64_t seed);
/* TokenSampler::sample (src/token_sampler.rs:83-174) on `vocab` f32 logits: *token and
 * its probability among the candidates kept by top-k / top-p.                           */
int rlb_sampler_sample(rlb_sampler* s, const float* logits, int32_t vocab, const int32_t* existing_tokens, int32_t n_existing,
                       int32_t* token, float* prob);
/* The candidate list `sample` draws from (descending probability, after top-k and
 * top-p): up to cap entries are written, *n receives the list's length. No counterpart
 * in the reference; it makes the sampler testable without statistics.                   */
int rlb_sampler_candidates(rlb_sampler* s, const float* logits, int32_t vocab, const int32_t* existing_tokens, int32_t n_existing,
                           int32_t* tokens, float* probs, int32_t cap, int32_t* n);

/* Tuning and inspection. Options: "graph" (replay the decode step as a CUDA graph, default 1),
 * "stream_gemv" (bulk-copy staged GEMV kernels, default 1), "pdl" (programmatic dependent launch,
 * default 1), "profile" (time every kernel class of the decode step). Statistics: "kernels_per_step", "attn_split", "local_heads", "layers_on_gpu",
 * "first_head", "local_ffn", "local_vocab", "vocab_size", "ffn_dim", "prof_steps", "prof_ms_<qkv|attn|wo|w13|w2|head|argmax|comm>". */
int rlb_model_set_option(rlb_model* m, const char* name, int64_t value);
int rlb_model_get_stat(rlb_model* m, const char* name, double* value);

#ifdef __cplusplus
}
#endif
#endif /* RLLAMA_B200_H */

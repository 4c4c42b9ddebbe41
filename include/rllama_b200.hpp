// Header-only C++ mirror of rllama's model surface over the C ABI of rllama_b200.h:
// Transformer (src/transformer.rs:22-36, :240-383), TransformerCaches (:111-113, :200-214),
// DataSettings (:38-109), ModelParams, DataSource, Tokenizer and TokenSampler, with the
// reference's method names and argument order. Errors, which
// the reference turns into panics or Err values, become rllama::Error exceptions.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "rllama_b200.h"

namespace rllama {

struct Error : std::runtime_error {
    int status;
    Error(int s, const char* msg) : std::runtime_error(msg), status(s) {}
};

inline void check(int status) {
    if (status != RLB_OK) throw Error(status, rlb_last_error());
}

// OpenCL::new(verbose, nth_device) (src/tensor_opencl_support.rs:86-128)
class Cuda {
  public:
    explicit Cuda(bool verbose = false, int nth_device = 0) { check(rlb_ctx_create(verbose ? 1 : 0, nth_device, &h_)); }
    ~Cuda() { rlb_ctx_destroy(h_); }
    Cuda(const Cuda&) = delete;
    Cuda& operator=(const Cuda&) = delete;
    void flush() { check(rlb_ctx_flush(h_)); }
    rlb_ctx* handle() const { return h_; }
  private:
    rlb_ctx* h_ = nullptr;
};

struct DataSettings {
    Cuda* cl = nullptr;
    bool force_f16_ = false;
    float percentage_to_gpu_ = 1.0f;  // layers beyond round(p * (n_layers - 1)) wait in pinned host memory (no CPU path)
    DataSettings force_f16() const { DataSettings d = *this; d.force_f16_ = true; return d; }
    DataSettings percentage_to_gpu(float p) const {
        DataSettings d = *this;
        if (p != p) p = 0.0f;  // NaN -> 0 (src/transformer.rs:91-103)
        d.percentage_to_gpu_ = p < 0.0f ? 0.0f : (p > 1.0f ? 1.0f : p);
        return d;
    }
};

class Transformer;

class TransformerCaches {
  public:
    ~TransformerCaches() { rlb_caches_free(h_); }
    TransformerCaches(TransformerCaches&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    TransformerCaches(const TransformerCaches&) = delete;
    TransformerCaches true_clone() const {
        rlb_caches* c = nullptr;
        check(rlb_caches_true_clone(h_, &c));
        return TransformerCaches(c);
    }
    void shift_left(int shifts) { check(rlb_caches_shift_left(h_, shifts)); }
    rlb_caches* handle() const { return h_; }
  private:
    friend class Transformer;
    explicit TransformerCaches(rlb_caches* h) : h_(h) {}
    rlb_caches* h_ = nullptr;
};

class Transformer {
  public:
    // The dimension arguments of Transformer::from_unpickled (src/transformer.rs:242-251); tensors
    // follow through set_tensor (what from_unpickled pulls out of the data source), then finalize().
    Transformer(int dim, int n_layers, int n_heads, int ffn_dim, int vocab_size, int max_seq_len, double eps,
                const DataSettings& data_settings, int tp_rank = 0, int tp_size = 1)
        : vocab_size_(vocab_size) {
        if (!data_settings.cl) throw Error(RLB_ERR_INVALID, "DataSettings without a CUDA context");
        rlb_model_params p{};
        p.dim = dim; p.n_layers = n_layers; p.n_heads = n_heads; p.ffn_dim = ffn_dim; p.vocab_size = vocab_size;
        p.max_seq_len = max_seq_len; p.norm_eps = (float)eps; p.force_f16 = data_settings.force_f16_ ? 1 : 0;
        p.tp_rank = tp_rank; p.tp_size = tp_size;
        p.has_percentage_to_gpu = 1; p.percentage_to_gpu = data_settings.percentage_to_gpu_;
        check(rlb_model_create(data_settings.cl->handle(), &p, &h_));
    }
    ~Transformer() { rlb_model_free(h_); }
    Transformer(const Transformer&) = delete;
    Transformer& operator=(const Transformer&) = delete;

    void set_tensor(rlb_tensor_kind kind, int layer, const void* data, int64_t rows, int64_t cols, int64_t capacity_cols,
                    rlb_dtype dtype) {
        check(rlb_model_set_tensor(h_, kind, layer, data, rows, cols, capacity_cols, dtype));
    }
    void finalize() { check(rlb_model_finalize(h_)); }

    TransformerCaches make_caches() {
        rlb_caches* c = nullptr;
        check(rlb_caches_create(h_, &c));
        return TransformerCaches(c);
    }
    // Transformer::forward(tokens, start_pos, caches) -> vocab x 1 f32 logits of the last token
    std::vector<float> forward(const std::vector<int32_t>& tokens, int start_pos, TransformerCaches& caches) {
        std::vector<float> logits((size_t)vocab_size_);
        check(rlb_forward(h_, caches.handle(), tokens.data(), (int32_t)tokens.size(), start_pos, logits.data()));
        return logits;
    }
    int32_t forward_greedy(const std::vector<int32_t>& tokens, int start_pos, TransformerCaches& caches) {
        int32_t next = 0;
        check(rlb_forward_greedy(h_, caches.handle(), tokens.data(), (int32_t)tokens.size(), start_pos, &next));
        return next;
    }
    rlb_model* handle() const { return h_; }
    int vocab_size() const { return vocab_size_; }

    // Transformer::from_unpickled(emb, dim, n_layers, n_heads, max_seq_len, eps, data_settings, data_source)
    // (src/transformer.rs:242-251): every tensor comes from the data source, Meta or HuggingFace names.
    static std::unique_ptr<Transformer> from_unpickled(int dim, int n_layers, int n_heads, int max_seq_len, double eps,
                                                       const DataSettings& data_settings, const class DataSource& data_source,
                                                       int tp_rank = 0, int tp_size = 1);
  private:
    Transformer() : vocab_size_(0) {}
    rlb_model* h_ = nullptr;
    int vocab_size_;
};

// ModelParams (src/model_params.rs:4-14)
struct ModelParams {
    int dim = 0, n_heads = 0, n_layers = 0;
    double norm_eps = 0;
    long vocab_size = 0;
    static ModelParams from_json(const std::string& path) {
        rlb_model_params p{};
        check(rlb_model_params_from_json(path.c_str(), &p));
        ModelParams m;
        m.dim = p.dim; m.n_heads = p.n_heads; m.n_layers = p.n_layers; m.norm_eps = p.norm_eps; m.vocab_size = p.vocab_size;
        return m;
    }
};

// DataSource (src/data_source.rs:22-30)
class DataSource {
  public:
    static DataSource from_llama_source(const std::string& path) { rlb_data_source* h = nullptr; check(rlb_data_source_open(path.c_str(), &h)); return DataSource(h); }
    static DataSource from_vicuna_source(const std::string& path) { rlb_data_source* h = nullptr; check(rlb_data_source_open_vicuna(path.c_str(), &h)); return DataSource(h); }
    static DataSource from_inferred_source(const std::string& path) { rlb_data_source* h = nullptr; check(rlb_data_source_open_inferred(path.c_str(), &h)); return DataSource(h); }
    ~DataSource() { rlb_data_source_free(h_); }
    DataSource(DataSource&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    DataSource(const DataSource&) = delete;
    DataSource& operator=(const DataSource&) = delete;
    bool need_to_do_antitranspose() const { int32_t v = 0; check(rlb_data_source_need_antitranspose(h_, &v)); return v != 0; }
    rlb_data_source* handle() const { return h_; }
  private:
    explicit DataSource(rlb_data_source* h) : h_(h) {}
    rlb_data_source* h_ = nullptr;
};

inline std::unique_ptr<Transformer> Transformer::from_unpickled(int dim, int n_layers, int n_heads, int max_seq_len, double eps,
                                                                const DataSettings& data_settings, const DataSource& data_source,
                                                                int tp_rank, int tp_size) {
    if (!data_settings.cl) throw Error(RLB_ERR_INVALID, "DataSettings without a CUDA context");
    rlb_model_params p{};
    p.dim = dim; p.n_layers = n_layers; p.n_heads = n_heads; p.max_seq_len = max_seq_len; p.norm_eps = (float)eps;
    p.force_f16 = data_settings.force_f16_ ? 1 : 0; p.tp_rank = tp_rank; p.tp_size = tp_size;
    p.has_percentage_to_gpu = 1; p.percentage_to_gpu = data_settings.percentage_to_gpu_;
    std::unique_ptr<Transformer> t(new Transformer());
    check(rlb_model_from_llama_source(data_settings.cl->handle(), data_source.handle(), &p, &t->h_));
    double v = 0;
    check(rlb_model_get_stat(t->h_, "vocab_size", &v));
    t->vocab_size_ = (int)v;
    return t;
}

// Tokenizer (src/tokenizer.rs)
class Tokenizer {
  public:
    static Tokenizer load(const std::string& path) { rlb_tokenizer* h = nullptr; check(rlb_tokenizer_load(path.c_str(), &h)); return Tokenizer(h); }
    ~Tokenizer() { rlb_tokenizer_free(h_); }
    Tokenizer(Tokenizer&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    Tokenizer(const Tokenizer&) = delete;
    Tokenizer& operator=(const Tokenizer&) = delete;
    std::string id_to_str(int32_t id) const { const char* s = nullptr; check(rlb_tokenizer_id_to_str(h_, id, &s)); return s; }
    // -1 where the reference returns None
    int32_t str_to_id(const std::string& s) const { int32_t id = -1; check(rlb_tokenizer_str_to_id(h_, s.c_str(), &id)); return id; }
    std::vector<int32_t> tokenize_to_ids(const std::string& text) const {
        int32_t n = 0;
        check(rlb_tokenizer_tokenize_to_ids(h_, text.c_str(), nullptr, 0, &n));
        std::vector<int32_t> ids((size_t)n);
        check(rlb_tokenizer_tokenize_to_ids(h_, text.c_str(), ids.data(), n, &n));
        return ids;
    }
    rlb_tokenizer* handle() const { return h_; }
  private:
    explicit Tokenizer(rlb_tokenizer* h) : h_(h) {}
    rlb_tokenizer* h_ = nullptr;
};

// TokenSampler (src/token_sampler.rs): the builder setters return *this
class TokenSampler {
  public:
    TokenSampler() { check(rlb_sampler_create(&h_)); }
    ~TokenSampler() { rlb_sampler_free(h_); }
    TokenSampler(const TokenSampler&) = delete;
    TokenSampler& operator=(const TokenSampler&) = delete;
    float get_temperature() const { float v; check(rlb_sampler_get(h_, &v, nullptr, nullptr, nullptr)); return v; }
    float get_top_p() const { float v; check(rlb_sampler_get(h_, nullptr, &v, nullptr, nullptr)); return v; }
    int32_t get_top_k() const { int32_t v; check(rlb_sampler_get(h_, nullptr, nullptr, &v, nullptr)); return v; }
    float get_repetition_penalty() const { float v; check(rlb_sampler_get(h_, nullptr, nullptr, nullptr, &v)); return v; }
    TokenSampler& temperature(float v) { check(rlb_sampler_set(h_, v, get_top_p(), get_top_k(), get_repetition_penalty())); return *this; }
    TokenSampler& top_p(float v) { check(rlb_sampler_set(h_, get_temperature(), v, get_top_k(), get_repetition_penalty())); return *this; }
    TokenSampler& top_k(int32_t v) { check(rlb_sampler_set(h_, get_temperature(), get_top_p(), v, get_repetition_penalty())); return *this; }
    TokenSampler& repetition_penalty(float v) { check(rlb_sampler_set(h_, get_temperature(), get_top_p(), get_top_k(), v)); return *this; }
    TokenSampler& seed(uint64_t s) { check(rlb_sampler_seed(h_, s)); return *this; }  // no counterpart: the reference uses thread_rng
    // sample(logits, tokenizer, existing_tokens) -> (token, probability); the tokenizer argument is unused there too
    std::pair<int32_t, float> sample(const std::vector<float>& logits, const std::vector<int32_t>& existing_tokens) {
        int32_t tok = 0;
        float p = 0.f;
        check(rlb_sampler_sample(h_, logits.data(), (int32_t)logits.size(), existing_tokens.data(), (int32_t)existing_tokens.size(), &tok, &p));
        return {tok, p};
    }
  private:
    rlb_sampler* h_ = nullptr;
};

}  // namespace rllama

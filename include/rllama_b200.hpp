// Header-only C++ mirror of rllama's model surface over the C ABI of rllama_b200.h:
// Transformer (src/transformer.rs:22-36, :240-383), TransformerCaches (:111-113, :200-214) and
// DataSettings (:38-109), with the reference's method names and argument order. Errors, which
// the reference turns into panics or Err values, become rllama::Error exceptions.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
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
    float percentage_to_gpu_ = 1.0f;  // kept for surface compatibility: there is no CPU path
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
  private:
    rlb_model* h_ = nullptr;
    int vocab_size_;
};

}  // namespace rllama

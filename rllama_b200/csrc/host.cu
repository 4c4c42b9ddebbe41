// Host-side callers of the decode path: rllama's Tokenizer (src/tokenizer.rs) and TokenSampler
// (src/token_sampler.rs), restated in C++ behind the C ABI so that the generation loop
// (src/rllama_main.rs:814-901) can run against this library without the Rust crates.
//
// Tokenizer: the SentencePiece ModelProto is read straight from the protobuf wire format (field 1
// of the message = repeated SentencePiece {1: piece, 2: score, 3: type}); text is cut greedily into
// the longest piece that prefixes the remaining input, as the reference does. Its quirks are kept:
//  * a newline becomes the piece "<0x0A>" when the vocabulary has it and is dropped otherwise;
//  * input that no piece prefixes is skipped one BYTE at a time, and when that byte is the first
//    of a multi-byte character the rest of the text is dropped (str::get(1..) is None there,
//    src/tokenizer.rs:153-155);
//  * pieces live in a map keyed by their text, so a repeated text keeps only its last index.
//
// TokenSampler: temperature, repetition penalty, "max subtraction", softmax, sort, top-k, top-p,
// draw. The reference runs the penalty and the max loops over `0..logits.rows()` after it has
// transposed the logits to 1 x vocab (src/token_sampler.rs:105, :113, :121), so they touch token 0
// only; that is reproduced. The draw uses a seeded generator here (the reference: thread_rng).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <unordered_map>

#include "internal.h"

// ---------------------------------------------------------------------------------------------
// Tokenizer
// ---------------------------------------------------------------------------------------------
struct rlb_tokenizer {
    struct Piece { int type; float score; int idx; };
    std::map<std::string, Piece> pieces;            // BTreeMap<String, Piece> (src/tokenizer.rs:13)
    std::unordered_map<int, const std::string*> by_id;
    int n_proto_pieces = 0;
    size_t max_len = 0;
    bool has_newline_piece = false;
};

namespace {

struct Reader {
    const unsigned char* p;
    const unsigned char* end;
    bool varint(uint64_t* v) {
        uint64_t r = 0;
        for (int shift = 0; shift < 64 && p < end; shift += 7) {
            const unsigned char b = *p++;
            r |= (uint64_t)(b & 0x7f) << shift;
            if (!(b & 0x80)) { *v = r; return true; }
        }
        return false;
    }
    bool skip(int wire) {
        uint64_t n;
        switch (wire) {
            case 0: return varint(&n);
            case 1: if (end - p < 8) return false; p += 8; return true;
            case 2: if (!varint(&n) || (uint64_t)(end - p) < n) return false; p += n; return true;
            case 5: if (end - p < 4) return false; p += 4; return true;
            default: return false;  // groups are not used by this schema
        }
    }
};

// sentence_piece::Type of sentencepiece_model.proto: NORMAL 1, UNKNOWN 2, CONTROL 3, USER_DEFINED 4, UNUSED 5, BYTE 6
bool known_piece_type(uint64_t t) { return t >= 1 && t <= 6; }

}  // namespace

extern "C" int rlb_tokenizer_load(const char* path, rlb_tokenizer** out) {
    if (!path || !out) return rlb_fail(RLB_ERR_INVALID, "tokenizer: null pointer");
    std::ifstream f(path, std::ios::binary);
    if (!f) return rlb_fail(RLB_ERR_INVALID, "tokenizer: cannot open %s", path);
    std::vector<unsigned char> buf((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    auto tk = std::make_unique<rlb_tokenizer>();
    Reader r{buf.data(), buf.data() + buf.size()};
    int idx = 0;
    while (r.p < r.end) {
        uint64_t key;
        if (!r.varint(&key)) return rlb_fail(RLB_ERR_INVALID, "tokenizer: %s is not a SentencePiece model (truncated field key)", path);
        const int field = (int)(key >> 3), wire = (int)(key & 7);
        if (field != 1 || wire != 2) {
            if (!r.skip(wire)) return rlb_fail(RLB_ERR_INVALID, "tokenizer: %s is not a SentencePiece model (bad field %d)", path, field);
            continue;
        }
        uint64_t len;
        if (!r.varint(&len) || (uint64_t)(r.end - r.p) < len) return rlb_fail(RLB_ERR_INVALID, "tokenizer: %s: truncated piece", path);
        Reader m{r.p, r.p + len};
        r.p += len;
        bool has_piece = false;
        std::string text;
        float score = 0.f;
        uint64_t type = 1;
        while (m.p < m.end) {
            uint64_t k2;
            if (!m.varint(&k2)) return rlb_fail(RLB_ERR_INVALID, "tokenizer: %s: truncated piece field", path);
            const int f2 = (int)(k2 >> 3), w2 = (int)(k2 & 7);
            if (f2 == 1 && w2 == 2) {
                uint64_t n;
                if (!m.varint(&n) || (uint64_t)(m.end - m.p) < n) return rlb_fail(RLB_ERR_INVALID, "tokenizer: %s: truncated piece text", path);
                text.assign((const char*)m.p, (size_t)n);
                m.p += n;
                has_piece = true;
            } else if (f2 == 2 && w2 == 5) {
                if (m.end - m.p < 4) return rlb_fail(RLB_ERR_INVALID, "tokenizer: %s: truncated score", path);
                memcpy(&score, m.p, 4);
                m.p += 4;
            } else if (f2 == 3 && w2 == 0) {
                if (!m.varint(&type)) return rlb_fail(RLB_ERR_INVALID, "tokenizer: %s: truncated type", path);
            } else if (!m.skip(w2)) {
                return rlb_fail(RLB_ERR_INVALID, "tokenizer: %s: bad piece field %d", path, f2);
            }
        }
        const int this_idx = idx++;  // enumerate() counts pieces without text too (src/tokenizer.rs:54-59)
        if (!has_piece) continue;
        if (!known_piece_type(type)) return rlb_fail(RLB_ERR_INVALID, "Unknown piece type (%s)", text.c_str());
        tk->pieces[text] = rlb_tokenizer::Piece{(int)type, score, this_idx};
    }
    tk->n_proto_pieces = idx;
    for (const auto& kv : tk->pieces) {
        tk->by_id[kv.second.idx] = &kv.first;
        tk->max_len = std::max(tk->max_len, kv.first.size());
    }
    tk->has_newline_piece = tk->pieces.count("<0x0A>") != 0;
    *out = tk.release();
    return RLB_OK;
}

extern "C" int rlb_tokenizer_free(rlb_tokenizer* tk) {
    delete tk;
    return RLB_OK;
}

extern "C" int rlb_tokenizer_n_pieces(rlb_tokenizer* tk, int32_t* n) {
    if (!tk || !n) return rlb_fail(RLB_ERR_INVALID, "tokenizer: null pointer");
    *n = tk->n_proto_pieces;
    return RLB_OK;
}

extern "C" int rlb_tokenizer_id_to_str(rlb_tokenizer* tk, int32_t id, const char** out) {
    if (!tk || !out) return rlb_fail(RLB_ERR_INVALID, "tokenizer: null pointer");
    auto it = tk->by_id.find(id);
    if (it == tk->by_id.end()) return rlb_fail(RLB_ERR_INVALID, "id out of range");  // the reference panics (src/tokenizer.rs:107)
    *out = it->second->c_str();
    return RLB_OK;
}

extern "C" int rlb_tokenizer_str_to_id(rlb_tokenizer* tk, const char* s, int32_t* id) {
    if (!tk || !s || !id) return rlb_fail(RLB_ERR_INVALID, "tokenizer: null pointer");
    auto it = tk->pieces.find(s);
    *id = it == tk->pieces.end() ? -1 : it->second.idx;
    return RLB_OK;
}

namespace {

// tokenize_to_pieces (src/tokenizer.rs:125-164) on bytes; returns piece indices.
void tokenize_pieces(const rlb_tokenizer* tk, const std::string& text, std::vector<int32_t>* ids) {
    size_t pos = 0;
    const size_t n = text.size();
    while (pos < n) {
        const rlb_tokenizer::Piece* best = nullptr;
        size_t best_len = 0;
        if (text[pos] == '\n') {
            if (tk->has_newline_piece) {
                ids->push_back(tk->pieces.find("<0x0A>")->second.idx);
                pos += 1;
                continue;
            }
            // no such piece: the candidate has length 0 and the byte is skipped below
        } else {
            // the longest piece that prefixes the rest of the text
            for (size_t len = std::min(tk->max_len, n - pos); len >= 1; len--) {
                auto it = tk->pieces.find(text.substr(pos, len));
                if (it != tk->pieces.end()) { best = &it->second; best_len = len; break; }
            }
        }
        if (best_len == 0) {
            // skip one byte; inside a multi-byte character the reference's str::get(1..) yields None
            // and the remaining text is dropped
            if (pos + 1 < n && ((unsigned char)text[pos + 1] & 0xC0) == 0x80) return;
            pos += 1;
        } else {
            ids->push_back(best->idx);
            pos += best_len;
        }
    }
}

}  // namespace

extern "C" int rlb_tokenizer_tokenize_to_ids(rlb_tokenizer* tk, const char* text, int32_t* ids, int32_t cap, int32_t* n) {
    if (!tk || !text || !n) return rlb_fail(RLB_ERR_INVALID, "tokenizer: null pointer");
    // "▁" + text with every space replaced by "▁" (src/tokenizer.rs:167-169)
    std::string s = "\xE2\x96\x81";
    for (const char* p = text; *p; p++) {
        if (*p == ' ') s += "\xE2\x96\x81";
        else s += *p;
    }
    std::vector<int32_t> out;
    out.push_back(1);  // start token
    tokenize_pieces(tk, s, &out);
    *n = (int32_t)out.size();
    if (ids != nullptr) {
        if ((int32_t)out.size() > cap) return rlb_fail(RLB_ERR_LIMIT, "tokenizer: %d ids do not fit in a buffer of %d", (int)out.size(), cap);
        memcpy(ids, out.data(), out.size() * sizeof(int32_t));
    }
    return RLB_OK;
}

// ---------------------------------------------------------------------------------------------
// TokenSampler
// ---------------------------------------------------------------------------------------------
struct rlb_sampler {
    float temperature = 0.2f;  // TokenSampler::new (src/token_sampler.rs:20-28)
    float top_p = 1.0f;
    int32_t top_k = 1;
    float repetition_penalty = 0.8f;
    uint64_t rng = 0x9E3779B97F4A7C15ull;
    std::vector<std::pair<int32_t, float>> cand;  // last candidate list
};

namespace {

uint64_t splitmix(uint64_t* s) {
    uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Everything of TokenSampler::sample up to the draw: fills s->cand with (token, probability) in
// descending order, truncated by top-k and top-p; returns their sum.
float sampler_candidates(rlb_sampler* s, const float* logits, int32_t vocab, const int32_t* existing, int32_t n_existing) {
    std::vector<float> x(logits, logits + vocab);
    if (s->temperature > 0.0f) {
        const float inv = 1.0f / s->temperature;
        for (float& v : x) v *= inv;
    }
    // the loops below run over `logits.rows()` of the transposed 1 x vocab tensor: token 0 only.
    // Net effect: token 0's logit becomes exactly 0 (its own value is the "maximum" that is subtracted)
    // and no other logit changes, whatever the penalty.
    if (s->repetition_penalty != 1.0f) {
        size_t count0 = 0;
        for (int32_t i = 0; i < n_existing; i++) count0 += existing[i] == 0;
        if (count0 > 0) x[0] *= powf(s->repetition_penalty, (float)count0);
    }
    float maxv = -INFINITY;
    if (x[0] > maxv) maxv = x[0];
    x[0] -= maxv;
    // Tensor::softmax (src/tensor.rs:479-494): exp, sequential f32 sum, divide
    float sum = 0.f;
    for (float& v : x) { v = expf(v); sum += v; }
    for (float& v : x) v /= sum;
    s->cand.resize(vocab);
    for (int32_t i = 0; i < vocab; i++) s->cand[i] = {i, x[i]};
    // descending by probability, NaNs last; equal probabilities keep index order (the reference's
    // sort_unstable leaves that order unspecified)
    std::stable_sort(s->cand.begin(), s->cand.end(), [](const std::pair<int32_t, float>& a, const std::pair<int32_t, float>& b) {
        const bool an = std::isnan(a.second), bn = std::isnan(b.second);
        if (an || bn) return !an && bn;
        return a.second > b.second;
    });
    if ((size_t)std::max(0, s->top_k) < s->cand.size()) s->cand.resize((size_t)std::max(0, s->top_k));
    float acc = 0.f;
    for (size_t i = 0; i < s->cand.size(); i++) {
        acc += s->cand[i].second;
        if (acc >= s->top_p) { s->cand.resize(i + 1); break; }
    }
    float total = 0.f;
    for (const auto& c : s->cand) total += c.second;
    return total;
}

}  // namespace

extern "C" int rlb_sampler_create(rlb_sampler** out) {
    if (!out) return rlb_fail(RLB_ERR_INVALID, "sampler: null pointer");
    *out = new rlb_sampler();
    return RLB_OK;
}
extern "C" int rlb_sampler_free(rlb_sampler* s) {
    delete s;
    return RLB_OK;
}
extern "C" int rlb_sampler_set(rlb_sampler* s, float temperature, float top_p, int32_t top_k, float repetition_penalty) {
    if (!s) return rlb_fail(RLB_ERR_INVALID, "sampler: null pointer");
    if (top_k < 0) return rlb_fail(RLB_ERR_INVALID, "sampler: top_k %d is negative", top_k);
    s->temperature = temperature; s->top_p = top_p; s->top_k = top_k; s->repetition_penalty = repetition_penalty;
    return RLB_OK;
}
extern "C" int rlb_sampler_get(rlb_sampler* s, float* temperature, float* top_p, int32_t* top_k, float* repetition_penalty) {
    if (!s) return rlb_fail(RLB_ERR_INVALID, "sampler: null pointer");
    if (temperature) *temperature = s->temperature;
    if (top_p) *top_p = s->top_p;
    if (top_k) *top_k = s->top_k;
    if (repetition_penalty) *repetition_penalty = s->repetition_penalty;
    return RLB_OK;
}
extern "C" int rlb_sampler_seed(rlb_sampler* s, uint64_t seed) {
    if (!s) return rlb_fail(RLB_ERR_INVALID, "sampler: null pointer");
    s->rng = seed;
    return RLB_OK;
}
extern "C" int rlb_sampler_candidates(rlb_sampler* s, const float* logits, int32_t vocab, const int32_t* existing, int32_t n_existing,
                                      int32_t* tokens, float* probs, int32_t cap, int32_t* n) {
    if (!s || !logits || !n || vocab < 1 || (n_existing > 0 && !existing)) return rlb_fail(RLB_ERR_INVALID, "sampler: bad arguments");
    sampler_candidates(s, logits, vocab, existing, n_existing);
    *n = (int32_t)s->cand.size();
    for (int32_t i = 0; i < *n && i < cap; i++) {
        if (tokens) tokens[i] = s->cand[i].first;
        if (probs) probs[i] = s->cand[i].second;
    }
    return RLB_OK;
}
extern "C" int rlb_sampler_sample(rlb_sampler* s, const float* logits, int32_t vocab, const int32_t* existing, int32_t n_existing,
                                  int32_t* token, float* prob) {
    if (!s || !logits || !token || vocab < 1 || (n_existing > 0 && !existing)) return rlb_fail(RLB_ERR_INVALID, "sampler: bad arguments");
    const float total = sampler_candidates(s, logits, vocab, existing, n_existing);
    // uniform in [0, total] (src/token_sampler.rs:159-163)
    const float u = total > 0.0f ? (float)((splitmix(&s->rng) >> 40) * (1.0 / 16777215.0)) * total : 0.0f;
    float acc = 0.f;
    for (const auto& c : s->cand) {
        acc += c.second;
        if (acc >= u) {
            *token = c.first;
            if (prob) *prob = c.second / total;
            return RLB_OK;
        }
    }
    *token = 0;
    if (prob) *prob = 0.0f;
    return RLB_OK;
}

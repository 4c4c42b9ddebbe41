// HTTP inference server of the command-line program: rllama's `server_inference`,
// `handle_request`, `GeneratingSession` and `AttentionCacheRepository`
// (src/rllama_main.rs:296-712) over the C ABI, with a small HTTP/1.1 server on POSIX sockets in
// place of the rocket crate.
//
// POST <api-path> with a JSON body {"prompt": ..., "temperature", "top_k", "top_p",
// "repetition_penalty", "max_seq_len", "max_new_tokens", "no_token_sampling", "stop_at_end_token"}
// answers 200 with a chunked body of JSON lines, one per generated token:
// {"<piece>":{"p":<probability>}} (plus "is_end_token":true on "</s>"), or with every piece's logit
// when no_token_sampling is set. Defaults and checks are the reference's (temperature 1.0, top_k 20,
// top_p 1.0, repetition_penalty 1.0, max_new_tokens 20, stop_at_end_token true; NaN or zero
// parameters answer 400 with the reference's texts; a body that is not the expected JSON answers
// 400 "Invalid JSON."). Every token is produced from a device-side clone of the KV caches kept in a
// repository keyed by the token sequence, evicting the oldest entry beyond the configured size, as
// the reference does; the clone is a device-to-device copy (rlb_caches_true_clone).
#pragma once

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <charconv>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <vector>

#include "../../include/rllama_b200.h"

namespace server {

// ---------------------------------------------------------------------------------------------
// JSON: just enough for the request (an object of scalars) and for the response lines
// ---------------------------------------------------------------------------------------------
struct JsonValue {
    enum Kind { Null, Bool, Number, String, Other } kind = Null;
    bool b = false;
    double num = 0;
    bool is_integer = false;  // written without fraction or exponent
    bool negative = false;
    std::string str;
};

class JsonReader {
public:
    explicit JsonReader(const std::string& s) : s_(s) {}
    // Parses a top-level object into key -> value (nested arrays and objects are skipped as Other).
    bool object(std::map<std::string, JsonValue>* out) {
        ws();
        if (!eat('{')) return false;
        ws();
        if (eat('}')) return end();
        while (true) {
            ws();
            std::string key;
            if (!string(&key)) return false;
            ws();
            if (!eat(':')) return false;
            JsonValue v;
            if (!value(&v, 0)) return false;
            (*out)[key] = v;
            seen_.push_back(key);
            ws();
            if (eat(',')) continue;
            if (eat('}')) return end();
            return false;
        }
    }
    const std::vector<std::string>& keys_in_order() const { return seen_; }

private:
    const std::string& s_;
    size_t p_ = 0;
    std::vector<std::string> seen_;
    void ws() { while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\r' || s_[p_] == '\t')) p_++; }
    bool eat(char c) { if (p_ < s_.size() && s_[p_] == c) { p_++; return true; } return false; }
    bool end() { ws(); return p_ == s_.size(); }
    bool lit(const char* w) { const size_t n = strlen(w); if (s_.compare(p_, n, w) == 0) { p_ += n; return true; } return false; }
    static void utf8(std::string* o, uint32_t cp) {
        if (cp < 0x80) *o += (char)cp;
        else if (cp < 0x800) { *o += (char)(0xC0 | (cp >> 6)); *o += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { *o += (char)(0xE0 | (cp >> 12)); *o += (char)(0x80 | ((cp >> 6) & 0x3F)); *o += (char)(0x80 | (cp & 0x3F)); }
        else { *o += (char)(0xF0 | (cp >> 18)); *o += (char)(0x80 | ((cp >> 12) & 0x3F)); *o += (char)(0x80 | ((cp >> 6) & 0x3F)); *o += (char)(0x80 | (cp & 0x3F)); }
    }
    bool hex4(uint32_t* v) {
        if (p_ + 4 > s_.size()) return false;
        uint32_t r = 0;
        for (int i = 0; i < 4; i++) {
            const char c = s_[p_++];
            r <<= 4;
            if (c >= '0' && c <= '9') r |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') r |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') r |= (uint32_t)(c - 'A' + 10);
            else return false;
        }
        *v = r;
        return true;
    }
    bool string(std::string* out) {
        if (!eat('"')) return false;
        while (p_ < s_.size()) {
            const unsigned char c = (unsigned char)s_[p_++];
            if (c == '"') return true;
            if (c < 0x20) return false;
            if (c != '\\') { *out += (char)c; continue; }
            if (p_ >= s_.size()) return false;
            const char e = s_[p_++];
            switch (e) {
                case '"': *out += '"'; break;
                case '\\': *out += '\\'; break;
                case '/': *out += '/'; break;
                case 'b': *out += '\b'; break;
                case 'f': *out += '\f'; break;
                case 'n': *out += '\n'; break;
                case 'r': *out += '\r'; break;
                case 't': *out += '\t'; break;
                case 'u': {
                    uint32_t cp;
                    if (!hex4(&cp)) return false;
                    if (cp >= 0xD800 && cp < 0xDC00) {  // surrogate pair
                        uint32_t lo;
                        if (!lit("\\u") || !hex4(&lo) || lo < 0xDC00 || lo > 0xDFFF) return false;
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
                        return false;
                    }
                    utf8(out, cp);
                    break;
                }
                default: return false;
            }
        }
        return false;
    }
    bool number(JsonValue* v) {
        const size_t start = p_;
        if (eat('-')) v->negative = true;
        if (p_ >= s_.size()) return false;
        if (s_[p_] == '0') p_++;
        else if (s_[p_] >= '1' && s_[p_] <= '9') while (p_ < s_.size() && isdigit((unsigned char)s_[p_])) p_++;
        else return false;
        v->is_integer = true;
        if (p_ < s_.size() && s_[p_] == '.') {
            v->is_integer = false;
            p_++;
            if (p_ >= s_.size() || !isdigit((unsigned char)s_[p_])) return false;
            while (p_ < s_.size() && isdigit((unsigned char)s_[p_])) p_++;
        }
        if (p_ < s_.size() && (s_[p_] == 'e' || s_[p_] == 'E')) {
            v->is_integer = false;
            p_++;
            if (p_ < s_.size() && (s_[p_] == '+' || s_[p_] == '-')) p_++;
            if (p_ >= s_.size() || !isdigit((unsigned char)s_[p_])) return false;
            while (p_ < s_.size() && isdigit((unsigned char)s_[p_])) p_++;
        }
        v->kind = JsonValue::Number;
        v->num = strtod(s_.substr(start, p_ - start).c_str(), nullptr);
        return true;
    }
    bool value(JsonValue* v, int depth) {
        if (depth > 64) return false;
        ws();
        if (p_ >= s_.size()) return false;
        const char c = s_[p_];
        if (c == '"') { v->kind = JsonValue::String; return string(&v->str); }
        if (c == 't') { v->kind = JsonValue::Bool; v->b = true; return lit("true"); }
        if (c == 'f') { v->kind = JsonValue::Bool; v->b = false; return lit("false"); }
        if (c == 'n') { v->kind = JsonValue::Null; return lit("null"); }
        if (c == '[') {
            p_++;
            v->kind = JsonValue::Other;
            ws();
            if (eat(']')) return true;
            while (true) {
                JsonValue x;
                if (!value(&x, depth + 1)) return false;
                ws();
                if (eat(',')) continue;
                return eat(']');
            }
        }
        if (c == '{') {
            p_++;
            v->kind = JsonValue::Other;
            ws();
            if (eat('}')) return true;
            while (true) {
                ws();
                std::string k;
                JsonValue x;
                if (!string(&k)) return false;
                ws();
                if (!eat(':') || !value(&x, depth + 1)) return false;
                ws();
                if (eat(',')) continue;
                return eat('}');
            }
        }
        return number(v);
    }
};

// serde_json's string escaping: quote, backslash, \b \f \n \r \t, other control characters as \u00XX.
inline std::string json_string(const std::string& s) {
    std::string o = "\"";
    for (unsigned char c : s) {
        switch (c) {
            case '"': o += "\\\""; break;
            case '\\': o += "\\\\"; break;
            case '\b': o += "\\b"; break;
            case '\f': o += "\\f"; break;
            case '\n': o += "\\n"; break;
            case '\r': o += "\\r"; break;
            case '\t': o += "\\t"; break;
            default:
                if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
                else o += (char)c;
        }
    }
    return o + "\"";
}

// serde_json's f32: the shortest digits that read back (ryu), "1.0" for integral values, exponent
// form for very small and very large magnitudes, null for NaN and infinities.
inline std::string json_f32(float v) {
    if (!std::isfinite(v)) return "null";
    char buf[64];
    auto r = std::to_chars(buf, buf + sizeof buf, v);  // shortest round-trip, fixed or scientific whichever is shorter
    std::string s(buf, r.ptr);
    const float a = std::fabs(v);
    if (a != 0.0f && (a < 1e-5f || a >= 1e16f)) {
        auto r2 = std::to_chars(buf, buf + sizeof buf, v, std::chars_format::scientific);
        s.assign(buf, r2.ptr);  // d.ddde-07 here; ryu prints d.ddde-7 and 1e-7
        const size_t e = s.find('e');
        std::string mant = s.substr(0, e), ex = s.substr(e + 1);
        bool neg = false;
        if (!ex.empty() && (ex[0] == '+' || ex[0] == '-')) { neg = ex[0] == '-'; ex.erase(0, 1); }
        while (ex.size() > 1 && ex[0] == '0') ex.erase(0, 1);
        return mant + "e" + (neg ? "-" : "") + ex;
    }
    auto r3 = std::to_chars(buf, buf + sizeof buf, v, std::chars_format::fixed);
    s.assign(buf, r3.ptr);
    if (s.find('.') == std::string::npos) s += ".0";
    return s;
}

// ---------------------------------------------------------------------------------------------
// request
// ---------------------------------------------------------------------------------------------
struct InferenceRequest {
    float temperature = 1.0f, top_p = 1.0f, repetition_penalty = 1.0f;
    uint64_t top_k = 20, max_seq_len = 0, max_new_tokens = 20;
    bool has_max_seq_len = false, no_token_sampling = false, stop_at_end_token = true;
    std::string prompt;
};

// serde_json::from_slice::<InferenceRequest> (src/rllama_main.rs:390-401): optional numbers and
// booleans (null counts as absent), a required string, unknown keys ignored, a repeated key is an error.
inline bool parse_request(const std::string& body, InferenceRequest* req) {
    std::map<std::string, JsonValue> kv;
    JsonReader rd(body);
    if (!rd.object(&kv)) return false;
    static const char* known[] = {"temperature", "top_k", "top_p", "repetition_penalty", "max_seq_len", "max_new_tokens",
                                  "no_token_sampling", "stop_at_end_token", "prompt"};
    for (const char* k : known) {
        int n = 0;
        for (const std::string& s : rd.keys_in_order()) n += s == k;
        if (n > 1) return false;  // "duplicate field"
    }
    auto f32 = [&](const char* k, float* dst) {
        auto it = kv.find(k);
        if (it == kv.end() || it->second.kind == JsonValue::Null) return true;
        if (it->second.kind != JsonValue::Number) return false;
        *dst = (float)it->second.num;
        return true;
    };
    auto usz = [&](const char* k, uint64_t* dst, bool* has) {
        auto it = kv.find(k);
        if (it == kv.end() || it->second.kind == JsonValue::Null) return true;
        const JsonValue& v = it->second;
        if (v.kind != JsonValue::Number || !v.is_integer || v.negative || v.num > 1.8e19) return false;
        *dst = (uint64_t)v.num;
        if (has) *has = true;
        return true;
    };
    auto boolean = [&](const char* k, bool* dst) {
        auto it = kv.find(k);
        if (it == kv.end() || it->second.kind == JsonValue::Null) return true;
        if (it->second.kind != JsonValue::Bool) return false;
        *dst = it->second.b;
        return true;
    };
    if (!f32("temperature", &req->temperature) || !f32("top_p", &req->top_p) || !f32("repetition_penalty", &req->repetition_penalty)) return false;
    if (!usz("top_k", &req->top_k, nullptr) || !usz("max_seq_len", &req->max_seq_len, &req->has_max_seq_len) ||
        !usz("max_new_tokens", &req->max_new_tokens, nullptr))
        return false;
    if (!boolean("no_token_sampling", &req->no_token_sampling) || !boolean("stop_at_end_token", &req->stop_at_end_token)) return false;
    auto it = kv.find("prompt");
    if (it == kv.end() || it->second.kind != JsonValue::String) return false;
    req->prompt = it->second.str;
    return true;
}

// ---------------------------------------------------------------------------------------------
// AttentionCacheRepository (src/rllama_main.rs:570-619): token sequence -> (caches, position, time)
// ---------------------------------------------------------------------------------------------
// Entries hold counted references to the device caches. A KV cache is append-only and an entry's position says
// how many of its rows are valid, so the entries a generating session leaves behind token after token can all
// refer to the ONE physical cache that session keeps writing to: rows below an entry's position never change.
using CachesRef = std::shared_ptr<rlb_caches>;
inline CachesRef make_caches_ref(rlb_caches* c) { return CachesRef(c, [](rlb_caches* p) { rlb_caches_free(p); }); }

class CacheRepository {
public:
    explicit CacheRepository(size_t max_size) : max_(max_size) {}
    // If the sequence is known: the caches of its entry and their position.
    bool get(const std::vector<int32_t>& tokens, CachesRef* caches, size_t* pos) const {
        auto it = map_.find(tokens);
        if (it == map_.end()) return false;
        *caches = it->second.caches;
        *pos = it->second.pos;
        return true;
    }
    void put(const std::vector<int32_t>& tokens, CachesRef caches, size_t pos) {
        map_[tokens] = Entry{std::move(caches), pos, std::chrono::steady_clock::now()};
        limit_size();
    }
    size_t size() const { return map_.size(); }

private:
    struct Entry { CachesRef caches; size_t pos; std::chrono::steady_clock::time_point t; };
    std::map<std::vector<int32_t>, Entry> map_;
    size_t max_;
    void limit_size() {
        while (map_.size() > max_) {  // the oldest entry goes first
            auto oldest = map_.begin();
            for (auto it = map_.begin(); it != map_.end(); ++it)
                if (it->second.t < oldest->second.t) oldest = it;
            map_.erase(oldest);
        }
    }
};

struct ServerState {
    rlb_model* model = nullptr;
    rlb_tokenizer* tokenizer = nullptr;
    int32_t vocab = 0;
    size_t max_seq_len = 0;
    bool exit_after_one_query = false;
    std::mutex repo_mu;
    CacheRepository repo{50};
    // counting semaphore (--inference-server-max-concurrent-inferences)
    std::mutex sem_mu;
    std::condition_variable sem_cv;
    size_t sem_free = 5;
    explicit ServerState(size_t cache_size, size_t concurrent) : repo(cache_size), sem_free(concurrent) {}
};

struct Failure { std::string what; };
inline void ok(int status) { if (status != RLB_OK) throw Failure{rlb_last_error()}; }

// GeneratingSession (src/rllama_main.rs:409-567): one call of `next_line` = one `read` that produces a token.
class GeneratingSession {
public:
    GeneratingSession(ServerState* st, const InferenceRequest& rq, std::vector<int32_t> tokens, size_t req_max_seq_len)
        : st_(st), tokens_(std::move(tokens)), req_max_seq_len_(req_max_seq_len), req_max_new_tokens_(rq.max_new_tokens),
          no_token_sampling_(rq.no_token_sampling), stop_at_end_token_(rq.stop_at_end_token) {
        ok(rlb_sampler_create(&sampler_));
        ok(rlb_sampler_set(sampler_, rq.temperature, rq.top_p, (int32_t)std::min<uint64_t>(rq.top_k, 0x7fffffff), rq.repetition_penalty));
        ok(rlb_sampler_seed(sampler_, (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count()));
        logits_.resize((size_t)st->vocab);
    }
    ~GeneratingSession() { rlb_sampler_free(sampler_); }

    // False when the stream has ended.
    bool next_line(std::string* line) {
        if (tokens_.size() >= req_max_seq_len_ || new_tokens_ >= req_max_new_tokens_) return false;
        CachesRef caches;
        size_t update_pos = 0;
        {
            std::lock_guard<std::mutex> g(st_->repo_mu);
            CachesRef found;
            size_t pos = 0;
            auto fresh = [&]() { rlb_caches* c = nullptr; ok(rlb_caches_create(st_->model, &c)); return make_caches_ref(c); };
            if (st_->repo.get(tokens_, &found, &pos)) {
                if (pos >= prev_pos_) {
                    if (found == own_) {
                        // The entry this session stored after its previous token refers to the caches it is
                        // generating into: they are used in place (the reference clones here,
                        // src/rllama_main.rs:489-503): no allocation, no copy of the whole cache, and the
                        // caches' decode graph is replayed.
                        caches = found;
                    } else {  // somebody else's entry: a true clone, as in the reference
                        rlb_caches* clone = nullptr;
                        ok(rlb_caches_true_clone(found.get(), &clone));
                        caches = make_caches_ref(clone);
                    }
                    update_pos = pos;
                } else {
                    caches = fresh();
                    // The reference continues from prev_pos with these empty caches; positions
                    // before prev_pos would then be attended as zeros, so the sequence is run again
                    // from the start instead.
                    prev_pos_ = 0;
                }
            } else {
                caches = fresh();
                rlb_caches* keep = nullptr;
                ok(rlb_caches_true_clone(caches.get(), &keep));
                st_->repo.put(tokens_, make_caches_ref(keep), prev_pos_);
                update_pos = prev_pos_;
            }
        }
        if (update_pos > prev_pos_) prev_pos_ = update_pos;
        ok(rlb_forward(st_->model, caches.get(), tokens_.data() + prev_pos_, (int32_t)(tokens_.size() - prev_pos_), (int32_t)prev_pos_,
                       logits_.data()));
        prev_pos_ = tokens_.size();
        int32_t tok = 0;
        float prob = 0.f;
        ok(rlb_sampler_sample(sampler_, logits_.data(), st_->vocab, tokens_.data(), (int32_t)tokens_.size(), &tok, &prob));
        tokens_.push_back(tok);
        {
            std::lock_guard<std::mutex> g(st_->repo_mu);
            st_->repo.put(tokens_, caches, prev_pos_);
            own_ = caches;
        }
        new_tokens_++;
        const char* piece = nullptr;
        ok(rlb_tokenizer_id_to_str(st_->tokenizer, tok, &piece));
        bool is_end = false;
        if (std::string(piece) == "</s>" && stop_at_end_token_) {
            new_tokens_ = req_max_new_tokens_;
            is_end = true;
        }
        // a BTreeMap<String, PredResult> as JSON: keys in byte order
        std::map<std::string, std::string> result;
        if (no_token_sampling_) {
            int32_t n = 0;
            ok(rlb_tokenizer_n_pieces(st_->tokenizer, &n));
            for (int32_t i = 0; i < st_->vocab && i < n; i++) {
                const char* p = nullptr;
                if (rlb_tokenizer_id_to_str(st_->tokenizer, i, &p) != RLB_OK) continue;  // (the reference would panic on a hole)
                std::string v = "{\"p\":" + json_f32(logits_[(size_t)i]);
                if (std::string(p) == "</s>") v += ",\"is_end_token\":true";
                result[p] = v + "}";
            }
        } else {
            std::string v = "{\"p\":" + json_f32(prob);
            if (is_end) v += ",\"is_end_token\":true";
            result[piece] = v + "}";
        }
        std::string out = "{";
        bool first = true;
        for (const auto& kv : result) {
            if (!first) out += ",";
            first = false;
            out += json_string(kv.first) + ":" + kv.second;
        }
        *line = out + "}\n";
        return true;
    }

private:
    ServerState* st_;
    rlb_sampler* sampler_ = nullptr;
    std::vector<int32_t> tokens_;
    std::vector<float> logits_;
    size_t req_max_seq_len_, req_max_new_tokens_, new_tokens_ = 0, prev_pos_ = 0;
    CachesRef own_;  // the caches this session generates into (also referenced by the entries it stored)
    bool no_token_sampling_, stop_at_end_token_;
};

// ---------------------------------------------------------------------------------------------
// HTTP
// ---------------------------------------------------------------------------------------------
inline bool send_all(int fd, const std::string& s) {
    size_t off = 0;
    while (off < s.size()) {
        const ssize_t n = ::send(fd, s.data() + off, s.size() - off, MSG_NOSIGNAL);
        if (n <= 0) return false;
        off += (size_t)n;
    }
    return true;
}

inline void respond(int fd, int code, const char* reason, const std::string& body) {
    char head[256];
    snprintf(head, sizeof head, "HTTP/1.1 %d %s\r\nContent-Type: text/plain; charset=utf-8\r\nContent-Length: %zu\r\nServer: rllama-b200\r\nConnection: close\r\n\r\n",
             code, reason, body.size());
    send_all(fd, std::string(head) + body);
}

inline std::string lower(std::string s) { for (char& c : s) c = (char)tolower((unsigned char)c); return s; }

// handle_request (src/rllama_main.rs:632-712) behind a hand-written HTTP/1.1 front end.
inline void handle_connection(ServerState* st, const std::string& api_path, int fd) {
    std::string buf;
    size_t header_end = std::string::npos;
    char tmp[4096];
    while (header_end == std::string::npos && buf.size() < (1u << 16)) {
        const ssize_t n = ::recv(fd, tmp, sizeof tmp, 0);
        if (n <= 0) { ::close(fd); return; }
        buf.append(tmp, (size_t)n);
        header_end = buf.find("\r\n\r\n");
    }
    if (header_end == std::string::npos) { respond(fd, 400, "Bad Request", "Bad request."); ::close(fd); return; }
    const std::string head = buf.substr(0, header_end);
    std::string body = buf.substr(header_end + 4);
    const size_t l1 = head.find("\r\n");
    const std::string request_line = head.substr(0, l1);
    const size_t sp1 = request_line.find(' '), sp2 = request_line.rfind(' ');
    if (sp1 == std::string::npos || sp2 == sp1) { respond(fd, 400, "Bad Request", "Bad request."); ::close(fd); return; }
    const std::string method = request_line.substr(0, sp1);
    std::string path = request_line.substr(sp1 + 1, sp2 - sp1 - 1);
    const size_t q = path.find('?');
    if (q != std::string::npos) path.erase(q);
    size_t content_length = 0;
    bool expect_continue = false;
    size_t pos = l1 == std::string::npos ? head.size() : l1 + 2;
    while (pos < head.size()) {
        size_t e = head.find("\r\n", pos);
        if (e == std::string::npos) e = head.size();
        const std::string line = head.substr(pos, e - pos);
        pos = e + 2;
        const size_t c = line.find(':');
        if (c == std::string::npos) continue;
        const std::string name = lower(line.substr(0, c));
        std::string value = line.substr(c + 1);
        while (!value.empty() && value[0] == ' ') value.erase(0, 1);
        if (name == "content-length") content_length = (size_t)strtoull(value.c_str(), nullptr, 10);
        if (name == "expect" && lower(value) == "100-continue") expect_continue = true;
    }
    auto same_path = [&](const std::string& p) {
        auto strip = [](std::string s) { while (s.size() > 1 && s.back() == '/') s.pop_back(); return s; };
        return strip(p) == strip(api_path);
    };
    if (method != "POST" || !same_path(path)) { respond(fd, 404, "Not Found", "Not found."); ::close(fd); return; }
    if (content_length > (64u << 20)) { respond(fd, 413, "Payload Too Large", "Payload too large."); ::close(fd); return; }
    if (expect_continue && body.size() < content_length) send_all(fd, "HTTP/1.1 100 Continue\r\n\r\n");
    while (body.size() < content_length) {
        const ssize_t n = ::recv(fd, tmp, sizeof tmp, 0);
        if (n <= 0) { ::close(fd); return; }
        body.append(tmp, (size_t)n);
    }
    body.resize(content_length);

    // one of at most `max concurrent inferences` requests at a time (the others wait their turn)
    {
        std::unique_lock<std::mutex> g(st->sem_mu);
        st->sem_cv.wait(g, [&] { return st->sem_free > 0; });
        st->sem_free--;
    }
    struct Release {
        ServerState* st;
        ~Release() { { std::lock_guard<std::mutex> g(st->sem_mu); st->sem_free++; } st->sem_cv.notify_one(); }
    } release{st};

    InferenceRequest rq;
    if (!parse_request(body, &rq)) { respond(fd, 400, "Bad Request", "Invalid JSON."); ::close(fd); return; }
    size_t req_max_seq_len = rq.has_max_seq_len ? (size_t)std::min<uint64_t>(rq.max_seq_len, st->max_seq_len) : st->max_seq_len;
    if (std::isnan(rq.temperature)) { respond(fd, 400, "Bad Request", "Temperature must be a number."); ::close(fd); return; }
    if (rq.top_k == 0) { respond(fd, 400, "Bad Request", "Top-k must be greater than 0."); ::close(fd); return; }
    if (std::isnan(rq.top_p)) { respond(fd, 400, "Bad Request", "Top-p must be a number."); ::close(fd); return; }
    if (std::isnan(rq.repetition_penalty)) { respond(fd, 400, "Bad Request", "Repetition penalty must be a number."); ::close(fd); return; }

    bool finished = false;
    try {
        int32_t n = 0;
        ok(rlb_tokenizer_tokenize_to_ids(st->tokenizer, rq.prompt.c_str(), nullptr, 0, &n));
        std::vector<int32_t> toks((size_t)n);
        ok(rlb_tokenizer_tokenize_to_ids(st->tokenizer, rq.prompt.c_str(), toks.data(), n, &n));
        GeneratingSession session(st, rq, std::move(toks), req_max_seq_len);
        if (!send_all(fd, "HTTP/1.1 200 OK\r\nTransfer-Encoding: chunked\r\nServer: rllama-b200\r\nConnection: close\r\n\r\n")) { ::close(fd); return; }
        std::string line;
        bool alive = true;
        while (alive && session.next_line(&line)) {
            char sz[32];
            snprintf(sz, sizeof sz, "%zx\r\n", line.size());
            alive = send_all(fd, std::string(sz) + line + "\r\n");  // one chunk per token, sent at once
        }
        if (alive) send_all(fd, "0\r\n\r\n");
        finished = true;
    } catch (const Failure& f) {
        fprintf(stderr, "request failed: %s\n", f.what.c_str());
    }
    ::shutdown(fd, SHUT_RDWR);
    ::close(fd);
    if (finished && st->exit_after_one_query) std::exit(0);
}

// Listens and serves until the process ends. Returns only on a socket error.
inline std::string serve(ServerState* st, const std::string& host, int port, const std::string& api_path) {
    const int ls = ::socket(AF_INET, SOCK_STREAM, 0);
    if (ls < 0) return "socket: " + std::string(strerror(errno));
    int one = 1;
    setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host == "localhost" ? "127.0.0.1" : host.c_str(), &addr.sin_addr) != 1) { ::close(ls); return "bad host address " + host; }
    if (::bind(ls, (sockaddr*)&addr, sizeof addr) != 0) { const std::string e = strerror(errno); ::close(ls); return "bind: " + e; }
    if (::listen(ls, 64) != 0) { const std::string e = strerror(errno); ::close(ls); return "listen: " + e; }
    while (true) {
        const int fd = ::accept(ls, nullptr, nullptr);
        if (fd < 0) {
            if (errno == EINTR) continue;
            const std::string e = strerror(errno);
            ::close(ls);
            return "accept: " + e;
        }
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
        std::thread(handle_connection, st, api_path, fd).detach();
    }
}

}  // namespace server

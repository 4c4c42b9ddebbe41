// Checkpoint loading: rllama's LLaMA data source (src/data_source.rs:166-196), its pickle
// reader (src/unpickler.rs:147-241, :317-675), TensorBuilder::load_from_pieces
// (src/tensor.rs:2388-2545), ModelParams (src/model_params.rs) and the construction half of
// Transformer::from_unpickled (src/transformer.rs:242-326), as host code in front of
// rlb_model_set_tensor.
//
// Layout read: <model>/consolidated.NN/data.pkl (pickle protocol 2: a dict name -> tensor record)
// and <model>/consolidated.NN/data/<key> (raw little-endian f16 storage), i.e. an unzipped
// torch checkpoint per model-parallel shard, NN = 00, 01, ... until a shard is missing.
// Shards are concatenated along the axis the reference uses for each tensor: rows for wq wk wv
// w1 w3 output, columns for wo w2 tok_embeddings; gains are taken from the first shard.
// As in the reference only torch.HalfStorage tensors with contiguous rows are accepted.
//
// Second layout (DataSource::VicunaSource, src/huggingface_loader.rs): a HuggingFace directory with
// config.json, pytorch_model.bin.index.json and *.bin files, each a torch.save zip archive read in
// place (stored or deflated entries, zip64 records); tensor names are HuggingFace's and the q/k
// projections carry its rotary row permutation, which is undone on load.
// Deviation: BININT2 is decoded as unsigned (the reference reads it as i16, src/unpickler.rs:484,
// which misreads 32768..65535); NEWTRUE, NONE, TUPLE3, SETITEM and an OrderedDict at top level
// are accepted in addition to the reference's opcode subset.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <dirent.h>
#include <zlib.h>

#include <algorithm>
#include <map>
#include <memory>
#include <set>
#include <sstream>

#include "internal.h"

namespace {

struct PVal;
typedef std::shared_ptr<PVal> PV;
struct PVal {
    enum Kind { MARK, STR, GLOBAL, INT, TUPLE, PERSID, BOOL, REDUCE, DICT, NONE } kind = NONE;
    std::string s, s2;                    // STR; GLOBAL (module, attribute)
    int64_t i = 0;                        // INT, BOOL
    std::vector<PV> items;                // TUPLE; PERSID [value]; REDUCE [callable, args]
    std::vector<std::pair<PV, PV>> dict;  // DICT (insertion order)
};
PV mk(PVal::Kind k) { auto v = std::make_shared<PVal>(); v->kind = k; return v; }

// unpickler::unpickle (src/unpickler.rs:317-675)
int unpickle(const std::vector<unsigned char>& b, PV* out, std::string* why) {
    if (b.size() < 2 || b[0] != 0x80 || b[1] != 2) { *why = "No magic header using Pickle 2 protocol"; return RLB_ERR_INVALID; }
    std::map<uint32_t, PV> memo;
    std::vector<PV> st;
    size_t p = 2;
    auto need = [&](size_t n) { return p + n <= b.size(); };
    auto pop_to_mark = [&](std::vector<PV>* items) {
        while (!st.empty() && st.back()->kind != PVal::MARK) { items->insert(items->begin(), st.back()); st.pop_back(); }
        if (st.empty()) return false;
        st.pop_back();
        return true;
    };
    auto set_item = [&](PV& d, PV k, PV v) {
        if (d->kind == PVal::REDUCE && d->items.size() == 2 && d->items[0]->kind == PVal::GLOBAL && d->items[0]->s == "collections" &&
            d->items[0]->s2 == "OrderedDict") {
            d->kind = PVal::DICT;  // an OrderedDict() call that now receives its items
            d->items.clear();
        }
        if (d->kind != PVal::DICT) return false;
        d->dict.emplace_back(k, v);
        return true;
    };
    while (p < b.size()) {
        const unsigned char op = b[p++];
        switch (op) {
            case '}': st.push_back(mk(PVal::DICT)); break;
            case ')': st.push_back(mk(PVal::TUPLE)); break;
            case '(': st.push_back(mk(PVal::MARK)); break;
            case 'N': st.push_back(mk(PVal::NONE)); break;
            case 0x88: case 0x89: { PV v = mk(PVal::BOOL); v->i = op == 0x88; st.push_back(v); break; }
            case 'q': if (!need(1) || st.empty()) goto trunc; memo[b[p]] = st.back(); p += 1; break;
            case 'r': { if (!need(4) || st.empty()) goto trunc; uint32_t k; memcpy(&k, &b[p], 4); memo[k] = st.back(); p += 4; break; }
            case 'h': { if (!need(1)) goto trunc; auto it = memo.find(b[p]); if (it == memo.end()) { *why = "BINGET of an unset memo slot"; return RLB_ERR_INVALID; } st.push_back(it->second); p += 1; break; }
            case 'j': { if (!need(4)) goto trunc; uint32_t k; memcpy(&k, &b[p], 4); auto it = memo.find(k); if (it == memo.end()) { *why = "LONG_BINGET of an unset memo slot"; return RLB_ERR_INVALID; } st.push_back(it->second); p += 4; break; }
            case 'X': { if (!need(4)) goto trunc; uint32_t n; memcpy(&n, &b[p], 4); p += 4; if (!need(n)) goto trunc; PV v = mk(PVal::STR); v->s.assign((const char*)&b[p], n); p += n; st.push_back(v); break; }
            case 'c': {
                PV v = mk(PVal::GLOBAL);
                size_t e = p; while (e < b.size() && b[e] != '\n') e++; if (e >= b.size()) goto trunc;
                v->s.assign((const char*)&b[p], e - p); p = e + 1;
                e = p; while (e < b.size() && b[e] != '\n') e++; if (e >= b.size()) goto trunc;
                v->s2.assign((const char*)&b[p], e - p); p = e + 1;
                st.push_back(v);
                break;
            }
            case 'J': { if (!need(4)) goto trunc; int32_t k; memcpy(&k, &b[p], 4); p += 4; PV v = mk(PVal::INT); v->i = k; st.push_back(v); break; }
            case 'K': { if (!need(1)) goto trunc; PV v = mk(PVal::INT); v->i = b[p]; p += 1; st.push_back(v); break; }
            case 'M': { if (!need(2)) goto trunc; uint16_t k; memcpy(&k, &b[p], 2); p += 2; PV v = mk(PVal::INT); v->i = k; st.push_back(v); break; }
            case 't': { PV v = mk(PVal::TUPLE); if (!pop_to_mark(&v->items)) { *why = "TUPLE without MARK"; return RLB_ERR_INVALID; } st.push_back(v); break; }
            case 0x85: case 0x86: case 0x87: {
                const size_t n = op - 0x84;
                if (st.size() < n) goto trunc;
                PV v = mk(PVal::TUPLE);
                v->items.assign(st.end() - n, st.end());
                st.resize(st.size() - n);
                st.push_back(v);
                break;
            }
            case 'Q': { if (st.empty()) goto trunc; PV v = mk(PVal::PERSID); v->items.push_back(st.back()); st.pop_back(); st.push_back(v); break; }
            case 'R': { if (st.size() < 2) goto trunc; PV v = mk(PVal::REDUCE); v->items.push_back(st[st.size() - 2]); v->items.push_back(st.back()); st.resize(st.size() - 2); st.push_back(v); break; }
            case 'u': {
                std::vector<PV> items;
                if (!pop_to_mark(&items) || st.empty() || items.size() % 2) { *why = "SETITEMS without MARK or dict"; return RLB_ERR_INVALID; }
                for (size_t i = 0; i + 1 < items.size(); i += 2)
                    if (!set_item(st.back(), items[i], items[i + 1])) { *why = "SETITEMS on a value that is not a dict"; return RLB_ERR_INVALID; }
                break;
            }
            case 's': {
                if (st.size() < 3) goto trunc;
                PV v = st.back(); st.pop_back(); PV k = st.back(); st.pop_back();
                if (!set_item(st.back(), k, v)) { *why = "SETITEM on a value that is not a dict"; return RLB_ERR_INVALID; }
                break;
            }
            case '.':
                if (st.size() != 1) { *why = "pickle ended with more than one value on the stack"; return RLB_ERR_INVALID; }
                *out = st.back();
                return RLB_OK;
            default: {
                char buf[64]; snprintf(buf, sizeof(buf), "unsupported pickle opcode 0x%02x at byte %zu", op, p - 1);
                *why = buf;
                return RLB_ERR_INVALID;
            }
        }
    }
trunc:
    *why = "truncated pickle";
    return RLB_ERR_INVALID;
}

// TensorBuilder (src/tensor.rs:2326-2338) as produced by Value::to_tensor_builder (src/unpickler.rs:147-241)
struct Builder { std::string file; int64_t rows = 0, cols = 0, nitems = 0, offset = 0; };

const PVal* dict_get(const PV& d, const std::string& key) {
    if (!d || d->kind != PVal::DICT) return nullptr;
    for (auto& kv : d->dict)
        if (kv.first->kind == PVal::STR && kv.first->s == key) return kv.second.get();
    return nullptr;
}

bool to_builder(const PVal* v, Builder* out) {
    if (!v || v->kind != PVal::REDUCE || v->items.size() != 2) return false;
    const PVal* call = v->items[0].get();
    const PVal* args = v->items[1].get();
    if (call->kind != PVal::GLOBAL || call->s != "torch._utils" || call->s2 != "_rebuild_tensor_v2") return false;
    if (args->kind != PVal::TUPLE || args->items.size() != 6) return false;
    const PVal* pid = args->items[0].get();
    if (pid->kind != PVal::PERSID || pid->items[0]->kind != PVal::TUPLE) return false;
    const auto& sa = pid->items[0]->items;
    if (sa.size() < 5 || sa[0]->kind != PVal::STR || sa[0]->s != "storage") return false;
    if (sa[1]->kind != PVal::GLOBAL || sa[1]->s != "torch" || sa[1]->s2 != "HalfStorage") return false;  // f16 only (:186-191)
    if (sa[2]->kind != PVal::STR || sa[4]->kind != PVal::INT || args->items[1]->kind != PVal::INT) return false;
    const PVal* shape = args->items[2].get();
    const PVal* stride = args->items[3].get();
    if (shape->kind != PVal::TUPLE || stride->kind != PVal::TUPLE) return false;
    if ((shape->items.size() != 1 && shape->items.size() != 2) || (stride->items.size() != 1 && stride->items.size() != 2)) return false;
    for (auto& x : shape->items) if (x->kind != PVal::INT) return false;
    for (auto& x : stride->items) if (x->kind != PVal::INT) return false;
    out->file = sa[2]->s; out->nitems = sa[4]->i; out->offset = args->items[1]->i;
    if (shape->items.size() == 2) { out->rows = shape->items[0]->i; out->cols = shape->items[1]->i; }
    else { out->rows = 1; out->cols = shape->items[0]->i; }
    if (stride->items.size() == 1) { if (stride->items[0]->i != 1) return false; }
    else if (stride->items[1]->i != 1 || stride->items[0]->i != out->cols) return false;  // contiguous rows only
    return out->rows >= 0 && out->cols >= 0 && out->offset >= 0;
}

}  // namespace

// One torch.save archive of a HuggingFace / Vicuna checkpoint (src/huggingface_loader.rs:20-27).
struct ZipEntry { uint64_t data_offset = 0, comp_size = 0, size = 0; int method = 0; };
struct ZipFile {
    std::string file;
    std::map<std::string, ZipEntry> entries;  // by name without its first directory
    std::set<std::string> tensors;            // tensor names of its data.pkl
};

struct rlb_data_source {
    std::string path;
    std::vector<PV> shards;  // one unpickled dict per consolidated.NN (Vicuna: the merged dict of all archives)
    bool vicuna = false;     // DataSource::VicunaSource (src/data_source.rs:22-30)
    std::vector<ZipFile> zips;
};

namespace {

std::string shard_dir(const rlb_data_source* ds, size_t i) {
    char buf[32];
    snprintf(buf, sizeof(buf), "/consolidated.%02zu", i);
    return ds->path + buf;
}

// Pieces of `name` (all shards, or the first only) -> total shape after concatenation.
int collect(const rlb_data_source* ds, const char* name, int direction, std::vector<Builder>* bs, int64_t* rows, int64_t* cols) {
    bs->clear();
    for (size_t i = 0; i < ds->shards.size(); i++) {
        const PVal* v = dict_get(ds->shards[i], name);
        if (!v) return rlb_fail(RLB_ERR_STATE, "missing field %s", name);  // UnpicklingError::MissingField
        Builder b;
        if (!to_builder(v, &b)) return rlb_fail(RLB_ERR_INVALID, "invalid tensor data for %s (only contiguous torch.HalfStorage tensors load)", name);
        bs->push_back(b);
        if (direction == 2) break;  // from_unpickled_pieces1: identical in every shard, take the first
    }
    if (bs->empty()) return rlb_fail(RLB_ERR_STATE, "data source has no shards");
    *rows = (*bs)[0].rows; *cols = (*bs)[0].cols;
    for (size_t i = 1; i < bs->size(); i++) {
        if (direction == 0) {
            if ((*bs)[i].cols != *cols) return rlb_fail(RLB_ERR_INVALID, "%s: shard %zu has %lld columns, expected %lld", name, i, (long long)(*bs)[i].cols, (long long)*cols);
            *rows += (*bs)[i].rows;
        } else {
            if ((*bs)[i].rows != *rows) return rlb_fail(RLB_ERR_INVALID, "%s: shard %zu has %lld rows, expected %lld", name, i, (long long)(*bs)[i].rows, (long long)*rows);
            *cols += (*bs)[i].cols;
        }
    }
    return RLB_OK;
}

// ---- zip archives (torch.save output; the reference uses the `zip` crate) --------------------
uint32_t rd32(const unsigned char* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
uint16_t rd16(const unsigned char* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
uint64_t rd64(const unsigned char* p) { return (uint64_t)rd32(p) | ((uint64_t)rd32(p + 4) << 32); }

bool read_at(FILE* f, uint64_t off, void* dst, size_t n) {
    return fseeko(f, (off_t)off, SEEK_SET) == 0 && fread(dst, 1, n, f) == n;
}

// huggingface_loader::remove_first_directory (src/huggingface_loader.rs:124-132)
std::string remove_first_directory(const std::string& name) {
    const size_t slash = name.find('/');
    return slash == std::string::npos ? std::string() : name.substr(slash + 1);
}

// Central directory of a zip file (zip64 records included): every entry with the offset of its data.
int zip_list(const std::string& path, std::vector<std::pair<std::string, ZipEntry>>* out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return rlb_fail(RLB_ERR_STATE, "cannot open %s", path.c_str());
    struct Closer { FILE* f; ~Closer() { fclose(f); } } closer{f};
    fseeko(f, 0, SEEK_END);
    const uint64_t fsize = (uint64_t)ftello(f);
    const uint64_t tail = std::min<uint64_t>(fsize, 65536 + 22 + 20);
    std::vector<unsigned char> buf((size_t)tail);
    if (!read_at(f, fsize - tail, buf.data(), (size_t)tail)) return rlb_fail(RLB_ERR_INVALID, "%s: not a zip archive", path.c_str());
    int64_t eocd = -1;
    for (int64_t i = (int64_t)tail - 22; i >= 0; i--)
        if (rd32(&buf[(size_t)i]) == 0x06054b50u) { eocd = i; break; }
    if (eocd < 0) return rlb_fail(RLB_ERR_INVALID, "%s: not a zip archive (no end-of-central-directory record)", path.c_str());
    uint64_t n_entries = rd16(&buf[(size_t)eocd + 10]), cd_size = rd32(&buf[(size_t)eocd + 12]), cd_off = rd32(&buf[(size_t)eocd + 16]);
    if (eocd >= 20 && rd32(&buf[(size_t)eocd - 20]) == 0x07064b50u) {  // zip64 locator -> zip64 end record
        const uint64_t z64 = rd64(&buf[(size_t)eocd - 20 + 8]);
        unsigned char rec[56];
        if (!read_at(f, z64, rec, sizeof rec) || rd32(rec) != 0x06064b50u) return rlb_fail(RLB_ERR_INVALID, "%s: bad zip64 end record", path.c_str());
        n_entries = rd64(rec + 32); cd_size = rd64(rec + 40); cd_off = rd64(rec + 48);
    }
    if (cd_size > fsize || cd_off > fsize - cd_size) return rlb_fail(RLB_ERR_INVALID, "%s: central directory outside the file", path.c_str());
    std::vector<unsigned char> cd((size_t)cd_size);
    if (!read_at(f, cd_off, cd.data(), (size_t)cd_size)) return rlb_fail(RLB_ERR_INVALID, "%s: cannot read the central directory", path.c_str());
    size_t p = 0;
    for (uint64_t e = 0; e < n_entries; e++) {
        if (p + 46 > cd.size() || rd32(&cd[p]) != 0x02014b50u) return rlb_fail(RLB_ERR_INVALID, "%s: bad central directory entry", path.c_str());
        ZipEntry ze;
        ze.method = rd16(&cd[p + 10]);
        ze.comp_size = rd32(&cd[p + 20]);
        ze.size = rd32(&cd[p + 24]);
        const size_t nlen = rd16(&cd[p + 28]), xlen = rd16(&cd[p + 30]), clen = rd16(&cd[p + 32]);
        uint64_t local = rd32(&cd[p + 42]);
        if (p + 46 + nlen + xlen + clen > cd.size()) return rlb_fail(RLB_ERR_INVALID, "%s: truncated central directory", path.c_str());
        const std::string name((const char*)&cd[p + 46], nlen);
        // zip64 extended information: the fields that overflowed, in this order
        const size_t x_end = p + 46 + nlen + xlen;  // end of this entry's extra field (inside cd, checked above)
        for (size_t x = p + 46 + nlen; x + 4 <= x_end;) {
            const uint16_t id = rd16(&cd[x]), len = rd16(&cd[x + 2]);
            const size_t f_end = x + 4 + (size_t)len;
            if (f_end > x_end) return rlb_fail(RLB_ERR_INVALID, "%s: extra field of %s runs past its entry", path.c_str(), name.c_str());
            if (id == 0x0001) {
                size_t q = x + 4;
                if (ze.size == 0xFFFFFFFFu && q + 8 <= f_end) { ze.size = rd64(&cd[q]); q += 8; }
                if (ze.comp_size == 0xFFFFFFFFu && q + 8 <= f_end) { ze.comp_size = rd64(&cd[q]); q += 8; }
                if (local == 0xFFFFFFFFu && q + 8 <= f_end) { local = rd64(&cd[q]); q += 8; }
            }
            x += 4 + (size_t)len;
        }
        unsigned char lh[30];
        if (!read_at(f, local, lh, sizeof lh) || rd32(lh) != 0x04034b50u) return rlb_fail(RLB_ERR_INVALID, "%s: bad local header of %s", path.c_str(), name.c_str());
        ze.data_offset = local + 30 + rd16(lh + 26) + rd16(lh + 28);
        if (ze.method != 0 && ze.method != 8) return rlb_fail(RLB_ERR_INVALID, "%s: %s uses compression method %d (stored and deflate are read)", path.c_str(), name.c_str(), ze.method);
        out->emplace_back(name, ze);
        p += 46 + nlen + xlen + clen;
    }
    return RLB_OK;
}

// The bytes [skip, skip + want) of an entry's uncompressed data.
int zip_read(const std::string& path, const ZipEntry& ze, uint64_t skip, void* dst, uint64_t want) {
    if (skip + want > ze.size) return rlb_fail(RLB_ERR_STATE, "%s: entry of %llu bytes is too short for %llu bytes at offset %llu", path.c_str(),
                                               (unsigned long long)ze.size, (unsigned long long)want, (unsigned long long)skip);
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return rlb_fail(RLB_ERR_STATE, "cannot open %s", path.c_str());
    struct Closer { FILE* f; ~Closer() { fclose(f); } } closer{f};
    if (ze.method == 0) {
        if (!read_at(f, ze.data_offset + skip, dst, (size_t)want)) return rlb_fail(RLB_ERR_STATE, "%s: read error", path.c_str());
        return RLB_OK;
    }
    // deflate: no random access, so the stream is inflated from its start and the prefix dropped
    // (the reference "seeks" the same way, src/data_source.rs:56-74)
    if (fseeko(f, (off_t)ze.data_offset, SEEK_SET) != 0) return rlb_fail(RLB_ERR_STATE, "%s: seek failed", path.c_str());
    z_stream zs;
    memset(&zs, 0, sizeof zs);
    if (inflateInit2(&zs, -MAX_WBITS) != Z_OK) return rlb_fail(RLB_ERR_STATE, "zlib: inflateInit2 failed");
    std::vector<unsigned char> in(1 << 16), scratch(1 << 16);
    uint64_t remaining_in = ze.comp_size, produced = 0;
    unsigned char* outp = (unsigned char*)dst;
    int zr = Z_OK;
    while (produced < skip + want && zr != Z_STREAM_END) {
        if (zs.avail_in == 0) {
            const size_t n = (size_t)std::min<uint64_t>(in.size(), remaining_in);
            if (n == 0 || fread(in.data(), 1, n, f) != n) { inflateEnd(&zs); return rlb_fail(RLB_ERR_STATE, "%s: truncated deflate stream", path.c_str()); }
            remaining_in -= n;
            zs.next_in = in.data();
            zs.avail_in = (uInt)n;
        }
        zs.next_out = scratch.data();
        zs.avail_out = (uInt)scratch.size();
        zr = inflate(&zs, Z_NO_FLUSH);
        if (zr != Z_OK && zr != Z_STREAM_END) { inflateEnd(&zs); return rlb_fail(RLB_ERR_STATE, "%s: corrupt deflate stream", path.c_str()); }
        const uint64_t got = scratch.size() - zs.avail_out;
        // copy the part of [produced, produced + got) that falls into [skip, skip + want)
        const uint64_t lo = std::max<uint64_t>(produced, skip), hi = std::min<uint64_t>(produced + got, skip + want);
        if (hi > lo) memcpy(outp + (lo - skip), scratch.data() + (lo - produced), (size_t)(hi - lo));
        produced += got;
    }
    inflateEnd(&zs);
    if (produced < skip + want) return rlb_fail(RLB_ERR_STATE, "%s: deflate stream ended early", path.c_str());
    return RLB_OK;
}

bool file_exists(const std::string& p) {
    std::ifstream f(p);
    return (bool)f;
}

// serde_json::from_str::<HugginfaceConfig> requires these keys (src/huggingface_loader.rs:29-44)
bool json_has_key(const std::string& text, const char* key) { return text.find(std::string("\"") + key + "\"") != std::string::npos; }

// A number that follows "key": in a flat JSON object (ModelParams is five scalars).
bool json_number(const std::string& text, const char* key, double* out) {
    const std::string pat = std::string("\"") + key + "\"";
    size_t p = text.find(pat);
    if (p == std::string::npos) return false;
    p = text.find(':', p + pat.size());
    if (p == std::string::npos) return false;
    char* end = nullptr;
    const double v = strtod(text.c_str() + p + 1, &end);
    if (end == text.c_str() + p + 1) return false;
    *out = v;
    return true;
}

}  // namespace

extern "C" {

int rlb_data_source_open(const char* model_path, rlb_data_source** out) {
    if (!model_path || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_data_source_open: null pointer");
    *out = nullptr;
    std::unique_ptr<rlb_data_source> ds(new rlb_data_source());
    ds->path = model_path;
    for (size_t part = 0;; part++) {
        std::ifstream f(shard_dir(ds.get(), part) + "/data.pkl", std::ios::binary);
        if (!f) break;  // NotFound ends the shard list (src/data_source.rs:176-186)
        std::vector<unsigned char> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        PV root;
        std::string why;
        if (unpickle(bytes, &root, &why) != RLB_OK) return rlb_fail(RLB_ERR_INVALID, "consolidated.%02zu/data.pkl: %s", part, why.c_str());
        if (root->kind != PVal::DICT) return rlb_fail(RLB_ERR_INVALID, "consolidated.%02zu/data.pkl: top level is not a dict", part);
        ds->shards.push_back(root);
    }
    if (ds->shards.empty()) return rlb_fail(RLB_ERR_STATE, "%s: no consolidated.00/data.pkl", model_path);
    *out = ds.release();
    return RLB_OK;
}

// DataSource::from_vicuna_source (src/data_source.rs:206-215) with HugginfaceModel::unpickle
// (src/huggingface_loader.rs:58-121): config.json and pytorch_model.bin.index.json must parse, every
// *.bin file of the directory is a torch.save zip whose data.pkl dicts are merged into one.
int rlb_data_source_open_vicuna(const char* model_path, rlb_data_source** out) {
    if (!model_path || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_data_source_open_vicuna: null pointer");
    *out = nullptr;
    std::unique_ptr<rlb_data_source> ds(new rlb_data_source());
    ds->path = model_path;
    ds->vicuna = true;
    auto slurp = [](const std::string& p, std::string* text) {
        std::ifstream f(p);
        if (!f) return false;
        std::stringstream ss;
        ss << f.rdbuf();
        *text = ss.str();
        return true;
    };
    std::string config, index;
    if (!slurp(ds->path + "/config.json", &config)) return rlb_fail(RLB_ERR_STATE, "cannot open %s/config.json", model_path);
    for (const char* key : {"vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "max_position_embeddings",
                            "rms_norm_eps", "architectures", "bos_token_id", "eos_token_id", "torch_dtype"})
        if (!json_has_key(config, key)) return rlb_fail(RLB_ERR_INVALID, "Error parsing JSON: %s/config.json: missing field `%s`", model_path, key);
    if (!slurp(ds->path + "/pytorch_model.bin.index.json", &index)) return rlb_fail(RLB_ERR_STATE, "cannot open %s/pytorch_model.bin.index.json", model_path);
    for (const char* key : {"metadata", "total_size", "weight_map"})
        if (!json_has_key(index, key)) return rlb_fail(RLB_ERR_INVALID, "Error parsing JSON: %s/pytorch_model.bin.index.json: missing field `%s`", model_path, key);
    std::vector<std::string> bins;
    if (DIR* d = opendir(model_path)) {
        while (dirent* e = readdir(d)) {
            const std::string n = e->d_name;
            if (n.size() > 4 && n.compare(n.size() - 4, 4, ".bin") == 0) bins.push_back(ds->path + "/" + n);
        }
        closedir(d);
    } else {
        return rlb_fail(RLB_ERR_STATE, "cannot list %s", model_path);
    }
    std::sort(bins.begin(), bins.end());
    PV merged = mk(PVal::DICT);
    for (const std::string& bin : bins) {
        std::vector<std::pair<std::string, ZipEntry>> entries;
        RLB_TRY(zip_list(bin, &entries));
        ZipFile zf;
        zf.file = bin;
        for (auto& kv : entries) {
            zf.entries[remove_first_directory(kv.first)] = kv.second;
            const std::string& n = kv.first;
            if (n.size() >= 8 && n.compare(n.size() - 8, 8, "data.pkl") == 0) {
                std::vector<unsigned char> bytes((size_t)kv.second.size);
                RLB_TRY(zip_read(bin, kv.second, 0, bytes.data(), kv.second.size));
                PV root;
                std::string why;
                if (unpickle(bytes, &root, &why) != RLB_OK) return rlb_fail(RLB_ERR_INVALID, "%s:%s: %s", bin.c_str(), n.c_str(), why.c_str());
                if (root->kind != PVal::DICT) return rlb_fail(RLB_ERR_INVALID, "%s:%s: top level is not a dict", bin.c_str(), n.c_str());
                for (auto& item : root->dict) {
                    if (item.first->kind != PVal::STR) continue;
                    zf.tensors.insert(item.first->s);
                    // Value::merge_dicts (src/unpickler.rs:91-108): later archives replace earlier entries
                    bool replaced = false;
                    for (auto& have : merged->dict)
                        if (have.first->kind == PVal::STR && have.first->s == item.first->s) { have.second = item.second; replaced = true; break; }
                    if (!replaced) merged->dict.push_back(item);
                }
            }
        }
        ds->zips.push_back(std::move(zf));
    }
    ds->shards.push_back(merged);
    *out = ds.release();
    return RLB_OK;
}

// DataSource::from_inferred_source (src/data_source.rs:188-204): params.json marks Meta's layout,
// pytorch_model.bin.index.json the HuggingFace one.
int rlb_data_source_open_inferred(const char* model_path, rlb_data_source** out) {
    if (!model_path || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_data_source_open_inferred: null pointer");
    const std::string p = model_path;
    if (file_exists(p + "/params.json")) return rlb_data_source_open(model_path, out);
    if (file_exists(p + "/pytorch_model.bin.index.json")) return rlb_data_source_open_vicuna(model_path, out);
    *out = nullptr;
    return rlb_fail(RLB_ERR_INVALID, "Unknown source");
}

// DataSource::need_to_do_antitranspose (src/data_source.rs:223-228)
int rlb_data_source_need_antitranspose(rlb_data_source* ds, int32_t* yes) {
    if (!ds || !yes) return rlb_fail(RLB_ERR_INVALID, "rlb_data_source_need_antitranspose: null pointer");
    *yes = ds->vicuna ? 1 : 0;
    return RLB_OK;
}

// Tensor::huggingface_llama_model_antitranspose (src/tensor.rs:841-909): the rows of a head, stored by
// HuggingFace as [2][head_dim / 2] (all even rotary components, then all odd ones), go back to the
// interleaved [head_dim / 2][2] order of Meta's files.
int rlb_huggingface_antitranspose_f16(const uint16_t* src, uint16_t* dst, int64_t rows, int64_t cols, int32_t n_heads) {
    if (!src || !dst) return rlb_fail(RLB_ERR_INVALID, "rlb_huggingface_antitranspose_f16: null pointer");
    if (n_heads <= 0 || rows % n_heads != 0 || (rows / n_heads) % 2 != 0)
        return rlb_fail(RLB_ERR_INVALID, "antitranspose: %lld rows do not split into %d heads of even size", (long long)rows, n_heads);
    const int64_t hd = rows / n_heads, half = hd / 2;
    for (int64_t h = 0; h < n_heads; h++)
        for (int64_t two = 0; two < 2; two++)
            for (int64_t j = 0; j < half; j++)
                memcpy(dst + (h * hd + j * 2 + two) * cols, src + (h * hd + two * half + j) * cols, (size_t)cols * 2);
    return RLB_OK;
}

int rlb_data_source_free(rlb_data_source* ds) {
    delete ds;
    return RLB_OK;
}

int rlb_data_source_shards(rlb_data_source* ds, int32_t* n) {
    if (!ds || !n) return rlb_fail(RLB_ERR_INVALID, "rlb_data_source_shards: null pointer");
    *n = (int32_t)ds->shards.size();
    return RLB_OK;
}

int rlb_data_source_tensor_shape(rlb_data_source* ds, const char* name, int32_t direction, int64_t* rows, int64_t* cols) {
    if (!ds || !name || !rows || !cols) return rlb_fail(RLB_ERR_INVALID, "rlb_data_source_tensor_shape: null pointer");
    if (direction < 0 || direction > 2) return rlb_fail(RLB_ERR_INVALID, "direction must be 0 (rows), 1 (cols) or 2 (first shard)");
    std::vector<Builder> bs;
    return collect(ds, name, direction, &bs, rows, cols);
}

int rlb_data_source_read_f16(rlb_data_source* ds, const char* name, int32_t direction, uint16_t* out, int64_t rows, int64_t cols) {
    if (!ds || !name || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_data_source_read_f16: null pointer");
    if (direction < 0 || direction > 2) return rlb_fail(RLB_ERR_INVALID, "direction must be 0 (rows), 1 (cols) or 2 (first shard)");
    std::vector<Builder> bs;
    int64_t r = 0, c = 0;
    RLB_TRY(collect(ds, name, direction, &bs, &r, &c));
    if (r != rows || c != cols) return rlb_fail(RLB_ERR_INVALID, "%s is %lldx%lld, the buffer is %lldx%lld", name, (long long)r, (long long)c, (long long)rows, (long long)cols);
    int64_t row0 = 0, col0 = 0;
    if (ds->vicuna) {
        // DataSource::open for a Vicuna source (src/data_source.rs:111-160): the archive that holds both the
        // storage file and the tensor's name
        const Builder& b = bs[0];
        const std::string entry = "data/" + b.file;
        for (const ZipFile& zf : ds->zips) {
            auto it = zf.entries.find(entry);
            if (it == zf.entries.end() || !zf.tensors.count(name)) continue;
            return zip_read(zf.file, it->second, (uint64_t)b.offset * 2, out, (uint64_t)rows * cols * 2);
        }
        return rlb_fail(RLB_ERR_STATE, "file not found: %s", entry.c_str());
    }
    for (size_t i = 0; i < bs.size(); i++) {
        const Builder& b = bs[i];
        const std::string path = shard_dir(ds, i) + "/data/" + b.file;
        FILE* f = fopen(path.c_str(), "rb");
        if (!f) return rlb_fail(RLB_ERR_STATE, "cannot open %s", path.c_str());
        if (fseek(f, (long)(b.offset * 2), SEEK_SET) != 0) { fclose(f); return rlb_fail(RLB_ERR_STATE, "%s: seek failed", path.c_str()); }
        for (int64_t row = 0; row < b.rows; row++) {
            uint16_t* dst = out + (row0 + row) * cols + col0;
            if (fread(dst, 2, (size_t)b.cols, f) != (size_t)b.cols) {
                fclose(f);
                return rlb_fail(RLB_ERR_STATE, "read error: path=%s row=%lld expected_len=%lld offset=%lld", path.c_str(), (long long)row,
                                (long long)(b.cols * 2), (long long)b.offset);
            }
        }
        fclose(f);
        if (direction == 0) row0 += b.rows; else col0 += b.cols;
    }
    return RLB_OK;
}

int rlb_model_params_from_json(const char* path, rlb_model_params* out) {
    if (!path || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_model_params_from_json: null pointer");
    std::ifstream f(path);
    if (!f) return rlb_fail(RLB_ERR_STATE, "cannot open %s", path);
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string text = ss.str();
    double dim, heads, layers, eps, vocab = -1;
    // serde aliases of src/model_params.rs:4-14; unknown keys are ignored
    if (!json_number(text, "dim", &dim) && !json_number(text, "hidden_size", &dim)) return rlb_fail(RLB_ERR_INVALID, "%s: missing field dim", path);
    if (!json_number(text, "n_heads", &heads) && !json_number(text, "num_attention_heads", &heads)) return rlb_fail(RLB_ERR_INVALID, "%s: missing field n_heads", path);
    if (!json_number(text, "n_layers", &layers) && !json_number(text, "num_hidden_layers", &layers)) return rlb_fail(RLB_ERR_INVALID, "%s: missing field n_layers", path);
    if (!json_number(text, "norm_eps", &eps) && !json_number(text, "rms_norm_eps", &eps)) return rlb_fail(RLB_ERR_INVALID, "%s: missing field norm_eps", path);
    if (!json_number(text, "vocab_size", &vocab)) return rlb_fail(RLB_ERR_INVALID, "%s: missing field vocab_size", path);
    out->dim = (int32_t)dim; out->n_heads = (int32_t)heads; out->n_layers = (int32_t)layers; out->norm_eps = (float)eps;
    out->vocab_size = (int32_t)vocab;  // Meta's files say -1: the real size comes from the embedding table
    return RLB_OK;
}

// Transformer::from_unpickled (src/transformer.rs:242-326) + Embedding::from_unpickled (src/embedding.rs:13-48).
// params: dim, n_layers, n_heads, norm_eps from params.json; max_seq_len, force_f16, tp_rank, tp_size from the
// caller; ffn_dim and vocab_size are taken from the tensors (w1 rows, embedding rows), as in the reference.
// Every tensor is looked up under Meta's name first and under its HuggingFace name second (the reference's
// from_unpickled_pieces2 / get_str_key2); wq and wk of a HuggingFace source are un-permuted
// (src/transformer.rs:619-622).
int rlb_model_from_llama_source(rlb_ctx* ctx, rlb_data_source* ds, const rlb_model_params* params, rlb_model** out) {
    if (!ctx || !ds || !params || !out) return rlb_fail(RLB_ERR_INVALID, "rlb_model_from_llama_source: null pointer");
    *out = nullptr;
    rlb_model_params p = *params;
    auto pick = [&](const std::string& meta, const std::string& hf) -> std::string {
        if (!ds->shards.empty() && dict_get(ds->shards[0], meta) == nullptr && dict_get(ds->shards[0], hf) != nullptr) return hf;
        return meta;  // (a name missing under both spellings is reported under Meta's)
    };
    int64_t r = 0, c = 0;
    const std::string emb = pick("tok_embeddings.weight", "model.embed_tokens.weight");
    RLB_TRY(rlb_data_source_tensor_shape(ds, emb.c_str(), 1, &r, &c));
    p.vocab_size = (int32_t)r;
    if (c != p.dim) return rlb_fail(RLB_ERR_INVALID, "%s has %lld columns, params say dim %d", emb.c_str(), (long long)c, p.dim);
    RLB_TRY(rlb_data_source_tensor_shape(ds, pick("layers.0.feed_forward.w1.weight", "model.layers.0.mlp.gate_proj.weight").c_str(), 0, &r, &c));
    p.ffn_dim = (int32_t)r;
    rlb_model* m = nullptr;
    RLB_TRY(rlb_model_create(ctx, &p, &m));
    std::vector<uint16_t> buf, tmp;
    auto load = [&](const std::string& name, int direction, rlb_tensor_kind kind, int layer) -> int {
        int64_t rows = 0, cols = 0;
        RLB_TRY(rlb_data_source_tensor_shape(ds, name.c_str(), direction, &rows, &cols));
        buf.resize((size_t)rows * cols);
        RLB_TRY(rlb_data_source_read_f16(ds, name.c_str(), direction, buf.data(), rows, cols));
        if (ds->vicuna && (kind == RLB_WQ || kind == RLB_WK)) {
            tmp.resize(buf.size());
            RLB_TRY(rlb_huggingface_antitranspose_f16(buf.data(), tmp.data(), rows, cols, p.n_heads));
            buf.swap(tmp);
        }
        return rlb_model_set_tensor(m, kind, layer, buf.data(), rows, cols, cols, RLB_F16);
    };
    int s = load(emb, 1, RLB_TOK_EMBEDDINGS, 0);
    for (int l = 0; l < p.n_layers && s == RLB_OK; l++) {
        const std::string pre = "layers." + std::to_string(l) + ".", hpre = "model.layers." + std::to_string(l) + ".";
        struct { const char* suffix; const char* hf; int direction; rlb_tensor_kind kind; } items[] = {
            {"attention.wq.weight", "self_attn.q_proj.weight", 0, RLB_WQ}, {"attention.wk.weight", "self_attn.k_proj.weight", 0, RLB_WK},
            {"attention.wv.weight", "self_attn.v_proj.weight", 0, RLB_WV}, {"attention.wo.weight", "self_attn.o_proj.weight", 1, RLB_WO},
            {"feed_forward.w1.weight", "mlp.gate_proj.weight", 0, RLB_W1}, {"feed_forward.w2.weight", "mlp.down_proj.weight", 1, RLB_W2},
            {"feed_forward.w3.weight", "mlp.up_proj.weight", 0, RLB_W3}, {"attention_norm.weight", "input_layernorm.weight", 2, RLB_ATTENTION_NORM},
            {"ffn_norm.weight", "post_attention_layernorm.weight", 2, RLB_FFN_NORM}};
        for (auto& it : items) {
            s = load(pick(pre + it.suffix, hpre + it.hf), it.direction, it.kind, l);
            if (s != RLB_OK) break;
        }
    }
    if (s == RLB_OK) s = load(pick("norm.weight", "model.norm.weight"), 2, RLB_NORM, 0);
    if (s == RLB_OK) s = load(pick("output.weight", "lm_head.weight"), 0, RLB_OUTPUT, 0);
    if (s == RLB_OK) s = rlb_model_finalize(m);
    if (s != RLB_OK) {
        rlb_model_free(m);
        return s;
    }
    *out = m;
    return RLB_OK;
}

}  // extern "C"

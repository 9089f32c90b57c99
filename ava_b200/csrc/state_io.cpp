// Saving and loading a carried state: `State::save` / `State::load` of the reference (src/state.rs:1114-1329).  The file
// is a safetensors file under the reference's tensor names and shapes:
//   meta.seen U32 [rows], meta.model U32 [2] (fingerprint high, low), meta.blocks U32 [1], meta.cap U32 [2] (max, rule;
//   0 0: no cap), meta.hist U32 [rows, 17], meta.hist_len U32 [rows],
//   lif.{i}.v / .s / .a F32 [rows, d], mem.{i}.f / .s F32 [rows * heads, hs, hs], parts.{i}.stp_u / .stp_x F32 [rows, d], v51.prev [rows, d] / .pvalid [rows] / .last_s [rows] / .mood [rows, k] / .rh [rows, 2],
//   eng.k / eng.v F32 [rows, heads, S, hs] with S the longest row's store and shorter rows padded on the left
//   (src/state.rs:207-328), eng.valid U32 [rows], eng.pad F32 [rows, S] (0 for a slot, -1e9 for padding) when rows differ.
// Written through PATH.tmp and a rename, so the file is whole or absent.  Host code over the C ABI.
//
// Two things differ from the reference and are said in the header: the fingerprint is the engine's own, and the token
// history (meta.hist, which feeds the reference's glance and magnitude codes) is written empty because the engine has
// neither part.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include <cerrno>
#include <sys/stat.h>

#include "../../include/ava_engine.h"

namespace {

constexpr int HIST = 17;           // src/state.rs:35
constexpr float PAD_NEG = -1e9f;   // src/memory.rs:53

struct Out {
    std::string name, dtype;
    std::vector<int64_t> shape;
    std::vector<unsigned char> data;
};

void put_u32(std::vector<Out>* outs, const std::string& name, std::vector<int64_t> shape, const std::vector<uint32_t>& v) {
    Out o{name, "U32", std::move(shape), {}};
    o.data.resize(v.size() * 4);
    std::memcpy(o.data.data(), v.data(), o.data.size());
    outs->push_back(std::move(o));
}

void put_f32(std::vector<Out>* outs, const std::string& name, std::vector<int64_t> shape, const std::vector<float>& v) {
    Out o{name, "F32", std::move(shape), {}};
    o.data.resize(v.size() * 4);
    std::memcpy(o.data.data(), v.data(), o.data.size());
    outs->push_back(std::move(o));
}

bool write_file(const std::string& path, const std::vector<Out>& outs) {
    std::string header = "{";
    uint64_t at = 0;
    for (size_t i = 0; i < outs.size(); ++i) {
        const Out& o = outs[i];
        if (i) header += ",";
        header += "\"" + o.name + "\":{\"dtype\":\"" + o.dtype + "\",\"shape\":[";
        for (size_t k = 0; k < o.shape.size(); ++k) header += (k ? "," : "") + std::to_string(o.shape[k]);
        header += "],\"data_offsets\":[" + std::to_string(at) + "," + std::to_string(at + o.data.size()) + "]}";
        at += o.data.size();
    }
    header += "}";
    while (header.size() % 8) header += ' ';
    const std::string tmp = path + ".tmp";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) return false;
    const uint64_t n = header.size();
    unsigned char lenb[8];
    for (int k = 0; k < 8; ++k) lenb[k] = (unsigned char)(n >> (8 * k));
    bool ok = std::fwrite(lenb, 1, 8, f) == 8 && std::fwrite(header.data(), 1, header.size(), f) == header.size();
    for (const Out& o : outs) ok = ok && (o.data.empty() || std::fwrite(o.data.data(), 1, o.data.size(), f) == o.data.size());
    ok = (std::fclose(f) == 0) && ok;
    if (!ok) {
        std::remove(tmp.c_str());
        return false;
    }
    return std::rename(tmp.c_str(), path.c_str()) == 0;
}

struct CkptCloser {
    void operator()(ava_ckpt* c) const { ava_ckpt_close(c); }
};

}  // namespace

extern "C" {

int ava_state_save(const ava_state* s, const char* path) {
    if (!s || !path) return AVA_ERR_ARG;
    ava_engine* e = ava_state_engine(s);
    const ava_config& c = *ava_engine_config(e);
    const int rows = ava_state_rows(s), d = c.d, L = c.n_blocks;
    std::vector<Out> outs;
    std::vector<uint32_t> seen((size_t)rows);
    for (int r = 0; r < rows; ++r) seen[r] = (uint32_t)ava_state_seen(s, r);
    const uint64_t fp = ava_engine_fingerprint(e);
    put_u32(&outs, "meta.seen", {rows}, seen);
    put_u32(&outs, "meta.model", {2}, {(uint32_t)(fp >> 32), (uint32_t)fp});
    put_u32(&outs, "meta.blocks", {1}, {(uint32_t)L});
    put_u32(&outs, "meta.cap", {2}, {(uint32_t)c.eng_cap, 0u});
    put_u32(&outs, "meta.hist", {rows, HIST}, std::vector<uint32_t>((size_t)rows * HIST, 0u));
    put_u32(&outs, "meta.hist_len", {rows}, std::vector<uint32_t>((size_t)rows, 0u));
    int rc;
    auto rows_of = [&](const std::string& name, int64_t per, std::vector<float>* v) {
        v->assign((size_t)rows * per, 0.0f);
        for (int r = 0; r < rows; ++r)
            if ((rc = ava_state_export(s, r, name.c_str(), v->data() + (size_t)r * per))) return false;
        return true;
    };
    std::vector<float> v;
    for (int i = 0; i < L; ++i) {
        const std::string li = "lif." + std::to_string(i) + ".", mi = "mem." + std::to_string(i) + ".";
        for (const char* k : {"v", "s", "a"}) {
            if (k[0] == 'a' && !c.alif) continue;
            if (!rows_of(li + k, d, &v)) return rc;
            put_f32(&outs, li + k, {rows, d}, v);
        }
        if (c.stp) {
            const std::string pi = "parts." + std::to_string(i) + ".";
            for (const char* k : {"stp_u", "stp_x"}) {
                if (!rows_of(pi + k, d, &v)) return rc;
                put_f32(&outs, pi + k, {rows, d}, v);
            }
        }
        if (!c.fast_mem) continue;
        const int hs = c.head_size, nh = d / hs;
        for (const char* k : {"f", "s"}) {
            if (k[0] == 's' && !(c.mem_momentum > 0.0f)) continue;
            if (!rows_of(mi + k, (int64_t)d * hs, &v)) return rc;
            put_f32(&outs, mi + k, {(int64_t)rows * nh, hs, hs}, v);
        }
    }
    if (c.rhythm) {
        if (!rows_of("v51.rh", 2, &v)) return rc;
        put_f32(&outs, "v51.rh", {rows, 2}, v);
    }
    if (c.dopamine || c.mood > 0) {  // src/v51.rs:1012,1068-1076: [rows, d], [rows], [rows], [rows, k]
        if (!rows_of("v51.prev", d, &v)) return rc;
        put_f32(&outs, "v51.prev", {rows, d}, v);
        if (!rows_of("v51.pvalid", 1, &v)) return rc;
        put_f32(&outs, "v51.pvalid", {rows}, v);
        if (!rows_of("v51.last_s", 1, &v)) return rc;
        put_f32(&outs, "v51.last_s", {rows}, v);
        if (c.mood > 0) {
            if (!rows_of("v51.mood", c.mood, &v)) return rc;
            put_f32(&outs, "v51.mood", {rows, c.mood}, v);
        }
    }
    if (c.eng_block >= 0) {
        const int ehs = c.eng_head_size, enh = d / ehs;
        std::vector<uint32_t> valid((size_t)rows);
        int S = 0;
        bool ragged = false;
        for (int r = 0; r < rows; ++r) {
            valid[r] = (uint32_t)(ava_state_len(s, r, "eng.k") / d);
            S = std::max(S, (int)valid[r]);
            ragged = ragged || valid[r] != valid[0];
        }
        if (S > 0) {  // a state that has read nothing has no store yet (`eng: None`)
            for (const char* k : {"k", "v"}) {
                std::vector<float> all((size_t)rows * d * S, 0.0f), one;
                for (int r = 0; r < rows; ++r) {
                    const int n = (int)valid[r];
                    if (!n) continue;
                    one.resize((size_t)n * d);
                    if ((rc = ava_state_export(s, r, (std::string("eng.") + k).c_str(), one.data()))) return rc;
                    for (int hh = 0; hh < enh; ++hh)  // [heads, n, hs] into the right end of [heads, S, hs]
                        std::memcpy(&all[(((size_t)r * enh + hh) * S + (S - n)) * ehs], &one[(size_t)hh * n * ehs], (size_t)n * ehs * sizeof(float));
                }
                put_f32(&outs, std::string("eng.") + k, {rows, enh, S, ehs}, all);
            }
            put_u32(&outs, "eng.valid", {rows}, valid);
            if (ragged) {
                std::vector<float> pad((size_t)rows * S, 0.0f);
                for (int r = 0; r < rows; ++r)
                    for (int j = 0; j < S - (int)valid[r]; ++j) pad[(size_t)r * S + j] = PAD_NEG;
                put_f32(&outs, "eng.pad", {rows, S}, pad);
            }
        }
    }
    return write_file(path, outs) ? AVA_OK : AVA_ERR_ARG;
}

int ava_state_load(ava_engine* e, const char* path, int32_t max_ctx, ava_state** out) {
    if (!e || !path || !out) return AVA_ERR_ARG;
    *out = nullptr;
    ava_ckpt* raw = nullptr;
    int rc = ava_ckpt_open(path, &raw);
    if (rc) return rc;
    std::unique_ptr<ava_ckpt, CkptCloser> ck(raw);
    const ava_config& c = *ava_engine_config(e);
    auto u32s = [&](const char* name, std::vector<uint32_t>* v) {
        const int i = ava_ckpt_find(ck.get(), name);
        if (i < 0) return false;
        int32_t rank;
        int64_t dims[4];
        const char* dt;
        ava_ckpt_tensor(ck.get(), i, nullptr, &dt, &rank, dims);
        if (std::strcmp(dt, "U32")) return false;
        v->resize((size_t)(dims[0] * dims[1] * dims[2] * dims[3]));
        return ava_ckpt_read_u32(ck.get(), i, v->data(), (int64_t)v->size()) == AVA_OK;
    };
    std::vector<uint32_t> seen, model, blocks, cap, valid;
    if (!u32s("meta.seen", &seen) || !u32s("meta.model", &model) || !u32s("meta.blocks", &blocks) || !u32s("meta.cap", &cap) || model.size() != 2 ||
        blocks.size() != 1 || cap.size() != 2 || seen.empty())
        return AVA_ERR_STATE;  // not a state file
    const uint64_t have = ((uint64_t)model[0] << 32) | model[1];
    if (have != ava_engine_fingerprint(e)) return AVA_ERR_STATE;  // saved by another model
    if ((int)blocks[0] != c.n_blocks || (int)cap[0] != c.eng_cap || cap[1] != 0) return AVA_ERR_STATE;
    const int rows = (int)seen.size(), d = c.d;
    const bool has_eng = c.eng_block >= 0 && ava_ckpt_find(ck.get(), "eng.k") >= 0;
    int S = 0;
    if (has_eng) {
        if (!u32s("eng.valid", &valid) || (int)valid.size() != rows) return AVA_ERR_STATE;
        int64_t dims[4];
        int32_t rank;
        ava_ckpt_tensor(ck.get(), ava_ckpt_find(ck.get(), "eng.k"), nullptr, nullptr, &rank, dims);
        if (rank != 4 || dims[0] != rows || dims[1] * dims[3] != d || dims[3] != c.eng_head_size) return AVA_ERR_STATE;
        S = (int)dims[2];
        for (uint32_t n : valid)
            if ((int)n > S) return AVA_ERR_STATE;
    }
    if (max_ctx < S) max_ctx = S;
    ava_state* st = nullptr;
    if ((rc = ava_state_new(e, rows, max_ctx > 0 ? max_ctx : 1, &st))) return rc;
    struct Guard {
        ava_state* s;
        ~Guard() {
            if (s) ava_state_destroy(s);
        }
    } guard{st};
    std::vector<float> v;
    auto rows_in = [&](const std::string& name, int64_t per) {
        const int i = ava_ckpt_find(ck.get(), name.c_str());
        if (i < 0) return (int)AVA_ERR_STATE;
        v.resize((size_t)rows * per);
        int r2 = ava_ckpt_read_f32(ck.get(), i, v.data(), (int64_t)v.size());
        for (int r = 0; r < rows && !r2; ++r) r2 = ava_state_import(st, r, name.c_str(), v.data() + (size_t)r * per, per);
        return r2;
    };
    for (int i = 0; i < c.n_blocks; ++i) {
        const std::string li = "lif." + std::to_string(i) + ".", mi = "mem." + std::to_string(i) + ".";
        for (const char* k : {"v", "s", "a"}) {
            if (k[0] == 'a' && !c.alif) continue;
            if ((rc = rows_in(li + k, d))) return rc;
        }
        if (c.stp) {
            const std::string pi = "parts." + std::to_string(i) + ".";
            for (const char* k : {"stp_u", "stp_x"})
                if ((rc = rows_in(pi + k, d))) return rc;
        }
        if (!c.fast_mem) continue;
        for (const char* k : {"f", "s"}) {
            if (k[0] == 's' && !(c.mem_momentum > 0.0f)) continue;
            if ((rc = rows_in(mi + k, (int64_t)d * c.head_size))) return rc;
        }
    }
    if (c.rhythm && (rc = rows_in("v51.rh", 2))) return rc;
    if (c.dopamine || c.mood > 0) {
        if ((rc = rows_in("v51.prev", d)) || (rc = rows_in("v51.pvalid", 1)) || (rc = rows_in("v51.last_s", 1))) return rc;
        if (c.mood > 0 && (rc = rows_in("v51.mood", c.mood))) return rc;
    }
    if (has_eng) {
        const int ehs = c.eng_head_size, enh = d / ehs;
        std::vector<float> all((size_t)rows * d * S), one;
        for (const char* k : {"k", "v"}) {
            const std::string name = std::string("eng.") + k;
            if ((rc = ava_ckpt_read_f32(ck.get(), ava_ckpt_find(ck.get(), name.c_str()), all.data(), (int64_t)all.size()))) return AVA_ERR_STATE;
            for (int r = 0; r < rows; ++r) {
                const int n = (int)valid[r];
                if (!n) continue;
                one.resize((size_t)n * d);
                for (int hh = 0; hh < enh; ++hh)
                    std::memcpy(&one[(size_t)hh * n * ehs], &all[(((size_t)r * enh + hh) * S + (S - n)) * ehs], (size_t)n * ehs * sizeof(float));
                if ((rc = ava_state_import(st, r, name.c_str(), one.data(), (int64_t)one.size()))) return rc;
            }
        }
    }
    for (int r = 0; r < rows; ++r) ava_state_set_seen(st, r, seen[r]);
    guard.s = nullptr;
    *out = st;
    return AVA_OK;
}

// ---- one saved state per conversation, in a folder (`ConvStore`, src/state.rs:1334-1384)

int ava_conv_path(const char* dir, const char* id, char* out, int64_t n) {
    if (!dir || !id || !out || n <= 0) return AVA_ERR_ARG;
    // the id itself when it is short and plain (letters, digits, '-', '_'), else its FNV-1a hash
    const size_t len = std::strlen(id);
    bool plain = len > 0 && len <= 64;
    for (size_t k = 0; k < len && plain; ++k) {
        const unsigned char ch = (unsigned char)id[k];
        plain = (ch >= '0' && ch <= '9') || (ch >= 'a' && ch <= 'z') || (ch >= 'A' && ch <= 'Z') || ch == '-' || ch == '_';
    }
    std::string name;
    if (plain) {
        name = id;
    } else {
        uint64_t h = 0xcbf29ce484222325ull;
        for (size_t k = 0; k < len; ++k) h = (h ^ (unsigned char)id[k]) * 0x100000001b3ull;
        char buf[24];
        std::snprintf(buf, sizeof buf, "h%016llx", (unsigned long long)h);
        name = buf;
    }
    std::string path = dir;
    if (!path.empty() && path.back() != '/') path += '/';
    path += "state-" + name + ".safetensors";
    if ((int64_t)path.size() + 1 > n) return AVA_ERR_CAPACITY;
    std::memcpy(out, path.c_str(), path.size() + 1);
    return AVA_OK;
}

int ava_conv_save(const char* dir, const char* id, const ava_state* s) {
    char path[4096];
    int rc = ava_conv_path(dir, id, path, sizeof path);
    if (rc) return rc;
    // the folder is made on first use (one level, as `create_dir_all` of a folder beside the model file)
    std::string cmd_dir = dir;
    if (::mkdir(cmd_dir.c_str(), 0777) != 0 && errno != EEXIST) return AVA_ERR_ARG;
    return ava_state_save(s, path);
}

int ava_conv_load(ava_engine* e, const char* dir, const char* id, int32_t max_ctx, ava_state** out, int32_t* found) {
    if (!out || !found) return AVA_ERR_ARG;
    *out = nullptr;
    *found = AVA_CONV_FRESH;
    char path[4096];
    int rc = ava_conv_path(dir, id, path, sizeof path);
    if (rc) return rc;
    FILE* f = std::fopen(path, "rb");
    if (!f) return AVA_OK;  // no saved state for this conversation: start fresh
    std::fclose(f);
    rc = ava_state_load(e, path, max_ctx, out);
    *found = rc == AVA_OK ? AVA_CONV_RESUMED : AVA_CONV_STALE;  // stale: saved by another model, or unreadable
    return AVA_OK;
}

}  // extern "C"

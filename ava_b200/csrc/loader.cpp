// Checkpoint loader: the caller side of the engine that the reference keeps in src/ckpt.rs (a model's shape from the
// tensor names of its .safetensors file, ckpt.rs:21-47; the block options from the arch.txt beside it, ckpt.rs:102-113,
// src/arch.rs:273-420,596-607) and in Model::set_int8 (src/model.rs:949-991: every matrix quantised once with
// ava_parts::quant::quantize_int8).  Host code only: it reads the file, fills an ava_config and feeds the engine
// through ava_engine_set_f32 / ava_engine_set_q8_from_f32.
//
// safetensors layout: u64 little-endian header length N, N bytes of JSON {"name": {"dtype": "F32", "shape": [..],
// "data_offsets": [begin, end]}, ..., "__metadata__": {..}}, then the data buffer the offsets point into.
#include <cctype>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/ava_engine.h"

namespace {

thread_local std::string g_err;

int fail(int code, const std::string& why) {
    g_err = why;
    return code;
}

struct Entry {
    std::string name, dtype;
    std::vector<int64_t> shape;
    uint64_t begin = 0, end = 0;
    int64_t count() const {
        int64_t n = 1;
        for (int64_t s : shape) n *= s;
        return n;
    }
};

// ---- the little JSON the header needs: objects, arrays, strings, integers (anything else is skipped by kind)
struct Json {
    const char* p;
    const char* end;
    bool ok = true;
    void ws() {
        while (p < end && std::isspace((unsigned char)*p)) ++p;
    }
    bool eat(char c) {
        ws();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
    std::string str() {
        std::string s;
        ws();
        if (p >= end || *p != '"') {
            ok = false;
            return s;
        }
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                    case 'n': s += '\n'; break;
                    case 't': s += '\t'; break;
                    case 'u':  // \uXXXX: tensor names are ASCII; keep the low byte
                        if (p + 4 < end) {
                            s += (char)std::strtol(std::string(p + 1, p + 5).c_str(), nullptr, 16);
                            p += 4;
                        }
                        break;
                    default: s += *p;
                }
                ++p;
            } else {
                s += *p++;
            }
        }
        if (p >= end) ok = false;
        else ++p;
        return s;
    }
    int64_t integer() {
        ws();
        char* q = nullptr;
        const long long v = std::strtoll(p, &q, 10);
        if (q == p) ok = false;
        p = q;
        return v;
    }
    void skip() {  // any value
        ws();
        if (p >= end) {
            ok = false;
            return;
        }
        if (*p == '"') {
            str();
        } else if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            ++p;
            if (eat(close)) return;
            do {
                if (open == '{') {
                    str();
                    if (!eat(':')) ok = false;
                }
                skip();
            } while (ok && eat(','));
            if (!eat(close)) ok = false;
        } else {
            while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;
        }
    }
};

bool parse_header(const char* text, size_t n, std::vector<Entry>* out) {
    Json j{text, text + n};
    if (!j.eat('{')) return false;
    if (j.eat('}')) return true;
    do {
        const std::string name = j.str();
        if (!j.ok || !j.eat(':')) return false;
        if (name == "__metadata__") {
            j.skip();
            continue;
        }
        Entry e;
        e.name = name;
        if (!j.eat('{')) return false;
        do {
            const std::string key = j.str();
            if (!j.ok || !j.eat(':')) return false;
            if (key == "dtype") {
                e.dtype = j.str();
            } else if (key == "shape" || key == "data_offsets") {
                std::vector<int64_t> v;
                if (!j.eat('[')) return false;
                if (!j.eat(']')) {
                    do v.push_back(j.integer());
                    while (j.ok && j.eat(','));
                    if (!j.eat(']')) return false;
                }
                if (key == "shape") {
                    e.shape = v;
                } else {
                    if (v.size() != 2 || v[0] < 0 || v[1] < v[0]) return false;
                    e.begin = (uint64_t)v[0];
                    e.end = (uint64_t)v[1];
                }
            } else {
                j.skip();
            }
        } while (j.ok && j.eat(','));
        if (!j.ok || !j.eat('}')) return false;
        out->push_back(std::move(e));
    } while (j.ok && j.eat(','));
    return j.ok && j.eat('}');
}

int dtype_size(const std::string& d) {
    if (d == "F32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16") return 2;
    return 0;
}

float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 31u, man = h & 1023u;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: value = man * 2^-24
            const float v = std::ldexp((float)man, -24);
            std::memcpy(&bits, &v, 4);
            bits |= sign;
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

}  // namespace

struct ava_ckpt {
    std::vector<Entry> entries;
    std::map<std::string, int> index;
    std::vector<unsigned char> data;           // the data buffer
    mutable std::vector<std::vector<float>> f32;  // tensors widened to f32 on first use (F32 tensors are read in place)
};

namespace {

const float* tensor_f32(const ava_ckpt* c, int i) {
    const Entry& e = c->entries[i];
    const unsigned char* src = c->data.data() + e.begin;
    if (e.dtype == "F32" && reinterpret_cast<uintptr_t>(src) % 4 == 0) return reinterpret_cast<const float*>(src);
    if (c->f32.size() != c->entries.size()) c->f32.resize(c->entries.size());
    std::vector<float>& v = c->f32[i];
    if (v.empty()) {
        const int64_t n = e.count();
        v.resize((size_t)n);
        if (e.dtype == "F32") {
            std::memcpy(v.data(), src, (size_t)n * 4);
        } else {
            for (int64_t k = 0; k < n; ++k) {
                uint16_t h;
                std::memcpy(&h, src + 2 * k, 2);
                if (e.dtype == "BF16") {
                    const uint32_t b = (uint32_t)h << 16;
                    std::memcpy(&v[(size_t)k], &b, 4);
                } else {
                    v[(size_t)k] = half_to_float(h);
                }
            }
        }
    }
    return v.data();
}

// "b12.mlp.w1" -> (12, "mlp.w1"); false for names outside the blocks
bool block_name(const std::string& name, int* block, std::string* rest) {
    if (name.size() < 4 || name[0] != 'b' || !std::isdigit((unsigned char)name[1])) return false;
    const size_t dot = name.find('.');
    if (dot == std::string::npos) return false;
    for (size_t k = 1; k < dot; ++k)
        if (!std::isdigit((unsigned char)name[k])) return false;
    *block = std::atoi(name.substr(1, dot - 1).c_str());
    *rest = name.substr(dot + 1);
    return true;
}

bool is_matrix(const std::string& rest) {
    static const char* m[] = {"mem.win", "mem.wout", "hebb.wq", "hebb.wk", "hebb.wv", "hebb.we", "hebb.wg", "hebb.wo",
                              "eng.wq",  "eng.wk",   "eng.wv",  "eng.wo",  "mlp.w1",  "mlp.w2"};
    for (const char* s : m)
        if (rest == s) return true;
    return false;
}

}  // namespace

extern "C" {

const char* ava_loader_error(void) { return g_err.c_str(); }

int ava_ckpt_open(const char* path, ava_ckpt** out) {
    if (!path || !out) return fail(AVA_ERR_ARG, "null argument");
    *out = nullptr;
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(AVA_ERR_MISSING, std::string("cannot open ") + path);
    std::unique_ptr<FILE, int (*)(FILE*)> closer(f, std::fclose);
    unsigned char lenb[8];
    if (std::fread(lenb, 1, 8, f) != 8) return fail(AVA_ERR_ARG, std::string(path) + ": shorter than a safetensors header");
    uint64_t hlen = 0;
    for (int k = 7; k >= 0; --k) hlen = (hlen << 8) | lenb[k];
    if (std::fseek(f, 0, SEEK_END) != 0) return fail(AVA_ERR_ARG, "seek failed");
    const long long size = std::ftell(f);
    if (size < 8 || hlen > (uint64_t)size - 8 || hlen > (1ull << 28)) return fail(AVA_ERR_ARG, std::string(path) + ": header length out of range");
    std::fseek(f, 8, SEEK_SET);
    std::string header((size_t)hlen, '\0');
    if (std::fread(&header[0], 1, (size_t)hlen, f) != hlen) return fail(AVA_ERR_ARG, std::string(path) + ": truncated header");
    std::unique_ptr<ava_ckpt> c(new ava_ckpt());
    if (!parse_header(header.data(), header.size(), &c->entries)) return fail(AVA_ERR_ARG, std::string(path) + ": header is not the expected JSON");
    const uint64_t dlen = (uint64_t)size - 8 - hlen;
    for (size_t i = 0; i < c->entries.size(); ++i) {
        const Entry& e = c->entries[i];
        const int es = dtype_size(e.dtype);
        if (!es) return fail(AVA_NOT_APPLICABLE, e.name + ": dtype " + e.dtype + " (F32, F16, BF16 and U32 are read)");
        if (e.shape.size() > 4) return fail(AVA_NOT_APPLICABLE, e.name + ": more than 4 dimensions");
        for (int64_t s : e.shape)
            if (s < 0) return fail(AVA_ERR_ARG, e.name + ": negative dimension");
        // the element count with every step checked: a shape whose product wraps must not pass as a small tensor
        uint64_t count = 1;
        bool wraps = false;
        for (int64_t s : e.shape) {
            if (s != 0 && count > (dlen / (uint64_t)es + 1) / (uint64_t)s + 1) wraps = true;
            if (!wraps) count *= (uint64_t)s;
        }
        if (wraps || e.begin > e.end || e.end > dlen || e.end - e.begin != count * (uint64_t)es)
            return fail(AVA_ERR_ARG, e.name + ": data offsets do not match its shape");
        if (!c->index.emplace(e.name, (int)i).second) return fail(AVA_ERR_ARG, e.name + ": named twice");
    }
    c->data.resize((size_t)dlen);
    if (dlen && std::fread(c->data.data(), 1, (size_t)dlen, f) != dlen) return fail(AVA_ERR_ARG, std::string(path) + ": truncated data");
    *out = c.release();
    return AVA_OK;
}

void ava_ckpt_close(ava_ckpt* c) { delete c; }

int32_t ava_ckpt_count(const ava_ckpt* c) { return c ? (int32_t)c->entries.size() : 0; }

int32_t ava_ckpt_find(const ava_ckpt* c, const char* name) {
    if (!c || !name) return -1;
    auto it = c->index.find(name);
    return it == c->index.end() ? -1 : it->second;
}

int ava_ckpt_tensor(const ava_ckpt* c, int32_t i, const char** name, const char** dtype, int32_t* rank, int64_t* dims) {
    if (!c || i < 0 || i >= (int32_t)c->entries.size()) return fail(AVA_ERR_ARG, "tensor index out of range");
    const Entry& e = c->entries[i];
    if (name) *name = e.name.c_str();
    if (dtype) *dtype = e.dtype.c_str();
    if (rank) *rank = (int32_t)e.shape.size();
    if (dims)
        for (size_t k = 0; k < 4; ++k) dims[k] = k < e.shape.size() ? e.shape[k] : 1;
    return AVA_OK;
}

int ava_ckpt_read_u32(const ava_ckpt* c, int32_t i, uint32_t* out, int64_t n) {
    if (!c || !out || i < 0 || i >= (int32_t)c->entries.size()) return fail(AVA_ERR_ARG, "tensor index out of range");
    const Entry& e = c->entries[i];
    if (e.dtype != "U32") return fail(AVA_ERR_ARG, e.name + ": not a U32 tensor");
    if (n != e.count()) return fail(AVA_ERR_ARG, e.name + ": element count differs");
    std::memcpy(out, c->data.data() + e.begin, (size_t)n * 4);
    return AVA_OK;
}

int ava_ckpt_read_f32(const ava_ckpt* c, int32_t i, float* out, int64_t n) {
    if (!c || !out || i < 0 || i >= (int32_t)c->entries.size()) return fail(AVA_ERR_ARG, "tensor index out of range");
    if (c->entries[i].dtype == "U32") return fail(AVA_ERR_ARG, c->entries[i].name + ": an integer tensor (ava_ckpt_read_u32)");
    if (n != c->entries[i].count()) return fail(AVA_ERR_ARG, c->entries[i].name + ": element count differs");
    std::memcpy(out, tensor_f32(c, i), (size_t)n * 4);
    return AVA_OK;
}

int ava_arch_flags(const char* flags, ava_config* cfg) {
    if (!cfg) return fail(AVA_ERR_ARG, "null config");
    std::istringstream in(flags ? flags : "");
    std::vector<std::string> a;
    for (std::string t; in >> t;) a.push_back(t);
    bool channel_gates = false;
    int kwta_div = 0;
    for (size_t i = 0; i < a.size(); ++i) {
        const std::string& k = a[i];
        auto value = [&](std::string* v) {
            if (i + 1 >= a.size()) return false;
            *v = a[++i];
            return true;
        };
        std::string v;
        // switches the step reads
        if (k == "--value-residual") cfg->value_residual = 1;
        else if (k == "--lif-scale") cfg->lif_scale = 1;
        else if (k == "--alif") cfg->alif = 1;
        else if (k == "--stp") cfg->stp = 1;
        else if (k == "--dendrite") cfg->dendrite = 1;
        else if (k == "--thalamus") cfg->thalamus = 1;
        else if (k == "--dopamine") cfg->dopamine = 1;
        else if (k == "--letters") cfg->letters = 1;
        else if (k == "--rhythm") cfg->rhythm = 1;
        else if (k == "--cerebellum-head") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--cerebellum-head needs a value");
            const int g = std::atoi(v.c_str());
            if (g < 0 || g % 32) return fail(AVA_ERR_ARG, "--cerebellum-head " + v + ": a multiple of 32 (src/v51b.rs:110-112)");
            cfg->cb_units = g;
        }
        else if (k == "--mood") cfg->mood = 4;  // MOOD_UNITS (src/v51.rs:53)
        else if (k == "--mood-units") {
            if (!value(&v) || std::atoi(v.c_str()) < 1 || std::atoi(v.c_str()) > 16) return fail(AVA_ERR_ARG, "--mood-units needs an integer from 1 to 16");
            cfg->mood = std::atoi(v.c_str());
        }
        else if (k == "--neuromod") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--neuromod needs a value");
            const int n = std::atoi(v.c_str());
            if (n != 0 && (n < 2 || n > 4)) return fail(AVA_NOT_APPLICABLE, "--neuromod " + v + ": the engine covers 2 to 4 signals");
            cfg->neuromod = n;
        }
        // switches that shape training or initial values only (src/arch.rs:159-169, src/model.rs:269-275)
        else if (k == "--resid-fix" || k == "--lif-reset-grad") {}
        else if (k == "--timescales" || k == "--lif-init") {
            if (!value(&v)) return fail(AVA_ERR_ARG, k + " needs a value");
        } else if (k == "--head-size") {
            if (!value(&v) || std::atoi(v.c_str()) <= 0) return fail(AVA_ERR_ARG, "--head-size needs a positive integer");
            cfg->head_size = std::atoi(v.c_str());
        } else if (k == "--gates") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--gates needs a value");
            if (v != "channel") return fail(AVA_NOT_APPLICABLE, "--gates " + v + ": the engine covers per-channel gates (--gates channel)");
            channel_gates = true;
        } else if (k == "--kwta") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--kwta needs a value");
            const size_t slash = v.find('/');
            const double f = slash == std::string::npos ? std::atof(v.c_str()) : std::atof(v.substr(0, slash).c_str()) / std::atof(v.substr(slash + 1).c_str());
            if (!(f > 0.0 && f <= 1.0)) return fail(AVA_ERR_ARG, "--kwta " + v + ": a fraction in (0, 1]");
            const double div = std::round(1.0 / f);
            if (std::fabs(1.0 / div - f) > 1e-9) return fail(AVA_ERR_ARG, "--kwta " + v + ": must be 1/n");
            kwta_div = (int)div;
        } else if (k == "--mlp-act") {
            if (!value(&v) || (v != "relu" && v != "relu2")) return fail(AVA_ERR_ARG, "--mlp-act: relu or relu2");
            cfg->relu2 = v == "relu2";
        } else if (k == "--mem-momentum") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--mem-momentum needs a value");
            cfg->mem_momentum = (float)std::atof(v.c_str());
            if (!(cfg->mem_momentum >= 0.0f && cfg->mem_momentum < 1.0f)) return fail(AVA_ERR_ARG, "--mem-momentum: must be in [0, 1)");
        } else if (k == "--residual") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--residual needs a value");
            if (v == "attn") return fail(AVA_NOT_APPLICABLE, "--residual attn: not covered by the engine");
            if (v != "plain" && v != "dense") return fail(AVA_ERR_ARG, "--residual: plain, dense or attn");
            cfg->dense = v == "dense";
        } else if (k == "--surrogate-slope") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--surrogate-slope needs a value");
            cfg->slope = (float)std::atof(v.c_str());
        } else if (k == "--spikes") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--spikes needs a value");
            if (v == "binary") cfg->spikes = 0;
            else if (v == "ternary") cfg->spikes = 1;
            else if (v == "int2") cfg->spikes = 2;
            else return fail(AVA_ERR_ARG, "--spikes: binary, ternary or int2");
        } else if (k == "--homeostasis") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--homeostasis needs a value");
            cfg->theta = std::atof(v.c_str()) != 0.0;  // per-neuron thresholds are then part of the model
        } else if (k == "--gate") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--gate needs a value");
            if (v == "sigmoid") return fail(AVA_NOT_APPLICABLE, "--gate sigmoid: the engine covers the silu output gate");
            if (v != "silu") return fail(AVA_ERR_ARG, "--gate: silu or sigmoid");
        } else if (k == "--gate-rank") {
            if (!value(&v)) return fail(AVA_ERR_ARG, "--gate-rank needs a value");  // the sigmoid gate's rank; unused with silu
        } else if (k.rfind("--", 0) == 0) {
            // every other block option adds a part to the step that the engine does not have (src/arch.rs:286-312,
            // src/memory.rs:160-191, src/v51.rs:104-118, src/v51b.rs:70-75, src/v50.rs)
            return fail(AVA_NOT_APPLICABLE, k + ": a block option the engine does not cover");
        } else {
            return fail(AVA_ERR_ARG, k + " is not a block flag");
        }
    }
    if (kwta_div > 0) {
        if (cfg->hidden % kwta_div) return fail(AVA_ERR_ARG, "--kwta: must divide the hidden width");
        cfg->kwta_k = cfg->hidden / kwta_div;
    }
    if (cfg->fast_mem && !channel_gates) return fail(AVA_NOT_APPLICABLE, "per-head gates (the default --gates head): the engine covers --gates channel");
    if (cfg->fast_mem && (cfg->head_size <= 0 || cfg->d % cfg->head_size)) return fail(AVA_ERR_ARG, "--head-size must divide d");
    return AVA_OK;
}

int ava_config_from_ckpt(const ava_ckpt* c, const char* kind, const char* arch_flags, ava_config* out) {
    if (!c || !kind || !out) return fail(AVA_ERR_ARG, "null argument");
    const int tok = ava_ckpt_find(c, "tok_emb");
    if (tok < 0 || c->entries[tok].shape.size() != 2) return fail(AVA_ERR_MISSING, "the file has no tok_emb [vocab, d]");
    ava_config cfg{};
    cfg.vocab = (int32_t)c->entries[tok].shape[0];
    cfg.d = (int32_t)c->entries[tok].shape[1];
    cfg.eng_block = -1;
    bool theta = false, wg = false;
    for (const Entry& e : c->entries) {
        int b;
        std::string rest;
        if (!block_name(e.name, &b, &rest)) {
            // tensors outside the blocks: the embedding and final norm, and the covered parts' own (nucleus, relay,
            // cerebellum read-out, mood, letters, rhythm)
            static const char* const whole[] = {"tok_emb", "final.norm", "nm.norm", "nm.wn", "nm.bn", "th.read", "th.gate", "th.bias", "cbh.wo"};
            static const char* const prefix[] = {"v51.mood.", "v51.letters.", "v51.rhythm."};
            bool known = false;
            for (const char* n : whole) known |= e.name == n;
            for (const char* p : prefix) known |= e.name.rfind(p, 0) == 0;
            if (!known)
                return fail(AVA_NOT_APPLICABLE, e.name + ": a tensor of a part the engine does not cover (glance, magnitude code, order head)");
            continue;
        }
        cfg.n_blocks = std::max(cfg.n_blocks, b + 1);
        if (rest == "eng.wq") cfg.eng_block = b;
        if (rest == "mem.theta") theta = true;
        if (rest == "hebb.wg") wg = true;
        if (rest == "mlp.w1" && e.shape.size() == 2) cfg.hidden = (int32_t)e.shape[1];
    }
    if (cfg.n_blocks == 0) return fail(AVA_ERR_MISSING, "the file has no blocks (b0.*)");
    if (cfg.hidden == 0) cfg.hidden = 4 * cfg.d;            // MLP_MULT (src/model.rs:251-258)
    cfg.kwta_k = cfg.hidden / 8;                            // KWTA_DIV (src/model.rs:41); --kwta 1/n changes it
    cfg.eng_head_size = 32;                                 // HEAD_SIZE (src/model.rs:43)
    cfg.gate_rank = 32;                                     // GATE_RANK (src/arch.rs:80)
    cfg.slope = 4.0f;
    cfg.theta = theta;
    const std::string k = kind;
    if (k == "S" || k == "s") {
        // spiking memory + sparse MLP: binary spikes, fixed threshold, relu, plain residual (src/model/fstep.rs:536-548,673-688)
        cfg.fast_mem = 0;
        cfg.head_size = cfg.d;
        if (arch_flags && *arch_flags) return fail(AVA_NOT_APPLICABLE, "block options are for model D (src/arch.rs:638-640)");
    } else if (k == "D" || k == "d") {
        cfg.fast_mem = 1;
        cfg.head_size = 32;
        cfg.out_gate = wg;
        if (!arch_flags || !*arch_flags)
            return fail(AVA_NOT_APPLICABLE, "model D without block options: its per-head gated step is not covered; the engine covers the block-options step (--gates channel ...)");
        const int rc = ava_arch_flags(arch_flags, &cfg);
        if (rc) return rc;
    } else {
        return fail(AVA_NOT_APPLICABLE, "model kind " + k + ": the engine covers S and D with block options");
    }
    *out = cfg;
    return AVA_OK;
}

int ava_engine_load_ckpt(ava_engine* e, const ava_ckpt* c) {
    if (!e || !c) return fail(AVA_ERR_ARG, "null argument");
    for (size_t i = 0; i < c->entries.size(); ++i) {
        const Entry& t = c->entries[i];
        int b;
        std::string rest;
        if (t.dtype == "U32") return fail(AVA_ERR_ARG, t.name + ": an integer tensor in a model file");
        const float* w = tensor_f32(c, (int)i);
        int rc;
        if (block_name(t.name, &b, &rest) && is_matrix(rest)) {
            if (t.shape.size() != 2) return fail(AVA_ERR_ARG, t.name + ": a matrix [din, dout] was expected");
            rc = ava_engine_set_q8_from_f32(e, t.name.c_str(), w, (int32_t)t.shape[0], (int32_t)t.shape[1]);
        } else {
            rc = ava_engine_set_f32(e, t.name.c_str(), w, t.count());
        }
        if (rc) return fail(rc, t.name + ": " + ava_last_error(e));
    }
    return AVA_OK;
}

}  // extern "C"

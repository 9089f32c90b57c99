// One traced token: `Model::step_trace` of the reference (design-tests/nn/gpu/src/model/fstep/arch.rs:420-476, the
// chat app's event feed).  Every value is a copy of what the step computed on the device, or a size computed here, on
// the host, from those copies; nothing feeds back, so logits and state are the untraced step's.  Host code over the
// C ABI: the step runs with its intermediates kept (ava_debug_keep) and the record is assembled from them.
//
// Per block: "spikes" [d] as they reach W_out, "winners" [hidden] (0/1: at or above the k-th largest unit), "hidden"
// [hidden] as it reaches W2, and with the fast-weight memory per head "mem_write" = |F' - alpha F| (alpha per row of F),
// "mem_read" = |y| before its norm, "mem_keep" = mean alpha, "mem_gate" = mean write strength; at the engram's block
// "engram_attn" [heads, keys] (this token's key last) and "engram_read" [d] as added.  Block -1: "input_rms" [1].
// The glance's place code and the magnitude code of the reference's record belong to parts the engine does not have.
#include <algorithm>
#include <cmath>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/ava_engine.h"
#include "ava_math.h"

struct ava_trace {
    std::map<std::pair<std::string, int>, std::vector<float>> v;
};

namespace {

// sum of squares in index order from 0, then the root (the reference's `iter().map(v * v).sum().sqrt()`)
float norm_seq(const float* x, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; ++i) s = ava::add(s, ava::mul(x[i], x[i]));
    return ava::root(s);
}

float mean_seq(const float* x, size_t n) {
    float s = 0.0f;
    for (size_t i = 0; i < n; ++i) s = ava::add(s, x[i]);
    return ava::div(s, (float)n);
}

}  // namespace

extern "C" {

int ava_step_trace(ava_engine* e, ava_state* s, uint32_t tok, float* logits, ava_trace** out) {
    if (!e || !s || !logits || !out) return AVA_ERR_ARG;
    if (ava_state_rows(s) != 1) return AVA_ERR_ARG;  // one token of one sequence, as the reference's
    const ava_config* cp = ava_engine_config(e);
    if (!cp) return AVA_ERR_ARG;
    const ava_config c = *cp;
    int rc;
    const int d = c.d, H = c.hidden, L = c.n_blocks, hs = c.head_size, nh = d / hs;
    if (c.eng_block >= 0 && c.eng_cap > 0) return AVA_NOT_APPLICABLE;  // the attention is taken from the store after the step: a capped store may have dropped a key
    // the fast weights before the step (the write's size is measured against them)
    std::vector<std::vector<float>> f0(L);
    if (c.fast_mem)
        for (int i = 0; i < L; ++i) {
            f0[i].resize((size_t)d * hs);
            if ((rc = ava_state_export(s, 0, ("mem." + std::to_string(i) + ".f").c_str(), f0[i].data()))) return rc;
        }
    if ((rc = ava_debug_keep(e, 1))) return rc;
    rc = ava_step(e, s, &tok, logits);
    std::unique_ptr<ava_trace> tr(new ava_trace());
    auto keep_off = [&](int code) {
        ava_debug_keep(e, 0);
        return code;
    };
    if (rc) return keep_off(rc);
    auto get = [&](const char* name, int block, size_t n, std::vector<float>* v) {
        v->resize(n);
        return ava_debug_get(e, name, block, v->data());
    };
    std::vector<float> a, b;
    if ((rc = get("x_in", -1, d, &a))) return keep_off(rc);
    {
        float s2 = 0.0f;  // sqrt(sum(v * v) / d)
        for (int i = 0; i < d; ++i) s2 = ava::add(s2, ava::mul(a[i], a[i]));
        tr->v[{"input_rms", -1}] = {ava::root(ava::div(s2, (float)std::max(d, 1)))};
    }
    for (int i = 0; i < L; ++i) {
        if ((rc = get(c.stp ? "stp_out" : "spikes", i, d, &a))) return keep_off(rc);
        tr->v[{"spikes", i}] = a;
        if ((rc = get("u", i, H, &a))) return keep_off(rc);
        {
            std::vector<float> w(H, 1.0f);
            if (c.kwta_k < H) {
                std::vector<float> srt(a);
                std::nth_element(srt.begin(), srt.begin() + (c.kwta_k - 1), srt.end(), [](float x, float y) { return x > y; });
                const float kth = srt[c.kwta_k - 1];
                for (int j = 0; j < H; ++j) w[j] = ava::sub(a[j], kth) >= 0.0f ? 1.0f : 0.0f;
            }
            tr->v[{"winners", i}] = w;
        }
        if ((rc = get(c.dendrite && c.fast_mem ? "a_dend" : "a", i, H, &a))) return keep_off(rc);
        tr->v[{"hidden", i}] = a;
        if (c.fast_mem) {
            std::vector<float> ex, be, yraw, f1((size_t)d * hs);
            if ((rc = get("ex", i, d, &ex)) || (rc = get("be", i, d, &be)) || (rc = get("y_raw", i, d, &yraw))) return keep_off(rc);
            if ((rc = ava_state_export(s, 0, ("mem." + std::to_string(i) + ".f").c_str(), f1.data()))) return keep_off(rc);
            std::vector<float> wr(nh), rd(nh), kp(nh), gt(nh);
            for (int h = 0; h < nh; ++h) {
                float s2 = 0.0f;
                for (int r = 0; r < hs; ++r) {
                    const float xa = ex[h * hs + r];
                    const size_t base = (size_t)h * hs * hs + (size_t)r * hs;
                    for (int q = 0; q < hs; ++q) {
                        const float dl = ava::sub(f1[base + q], ava::mul(f0[i][base + q], xa));
                        s2 = ava::add(s2, ava::mul(dl, dl));
                    }
                }
                wr[h] = ava::root(s2);
                rd[h] = norm_seq(&yraw[h * hs], hs);
                kp[h] = mean_seq(&ex[h * hs], hs);
                gt[h] = mean_seq(&be[h * hs], hs);
            }
            tr->v[{"mem_write", i}] = wr;
            tr->v[{"mem_read", i}] = rd;
            tr->v[{"mem_keep", i}] = kp;
            tr->v[{"mem_gate", i}] = gt;
        }
        if (i == c.eng_block) {
            const int ehs = c.eng_head_size, enh = d / ehs;
            const int64_t len = ava_state_len(s, 0, "eng.k");
            if (len < 0) return keep_off(AVA_ERR_STATE);
            const int n = (int)(len / d);
            std::vector<float> kk((size_t)len), qkv;
            if ((rc = ava_state_export(s, 0, "eng.k", kk.data())) || (rc = get("eng_qkv", i, 3 * (size_t)d, &qkv))) return keep_off(rc);
            // per head: score_j = K[j][0] q0, then one fused multiply-add per further channel, times scale plus 0; softmax
            // with the maximum found by "replace while smaller", the exponentials summed from 0 in order
            // (src/model/fstep/arch.rs:453-472, src/model/fstep.rs:303-330)
            const float scale = (float)(1.0 / std::sqrt((double)ehs));
            std::vector<float> w((size_t)enh * n);
            for (int h = 0; h < enh; ++h) {
                float* o = &w[(size_t)h * n];
                const float* q = &qkv[(size_t)h * ehs];
                for (int j = 0; j < n; ++j) {
                    const float* kr = &kk[((size_t)h * n + j) * ehs];
                    float sc = ava::mul(kr[0], q[0]);
                    for (int ch = 1; ch < ehs; ++ch) sc = ava::fma(kr[ch], q[ch], sc);
                    o[j] = ava::add(ava::mul(sc, scale), 0.0f);
                }
                float mx = o[0];
                for (int j = 0; j < n; ++j)
                    if (mx < o[j]) mx = o[j];
                float den = 0.0f;
                for (int j = 0; j < n; ++j) {
                    o[j] = ava::expf_(ava::sub(o[j], mx));
                    den = ava::add(den, o[j]);
                }
                for (int j = 0; j < n; ++j) o[j] = ava::div(o[j], den);
            }
            tr->v[{"engram_attn", i}] = w;
            if ((rc = get("eng_r", i, d, &a))) return keep_off(rc);
            tr->v[{"engram_read", i}] = a;
        }
    }
    ava_debug_keep(e, 0);
    *out = tr.release();
    return AVA_OK;
}

int64_t ava_trace_get(const ava_trace* t, const char* name, int32_t block, float* out, int64_t cap) {
    if (!t || !name) return -1;
    auto it = t->v.find({name, block});
    if (it == t->v.end()) return -1;
    const int64_t n = (int64_t)it->second.size();
    if (out) std::copy(it->second.begin(), it->second.begin() + std::min(n, cap), out);
    return n;
}

void ava_trace_free(ava_trace* t) { delete t; }

}  // extern "C"

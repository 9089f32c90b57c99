// The callers' side of the step: the token sampler and the batched generation loop, as host code over the C ABI.
//
// `ava_pick` follows `diary::pick` (src/diary.rs:686-718: the most likely token at temperature <= 0, else
// softmax(logits / temperature), the top-k kept, one SplitMix64 draw over their mass; constants of the generator:
// nn/data/src/rng.rs:7-31).  `ava_generate` follows `state::generate` (src/state.rs:1388-1458): prompts read in batched
// passes, rows of one length together; then all rows step together, one token per pass; a row leaves the batch at EOS
// or when the caller's stop rule says so.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <numeric>
#include <string>
#include <vector>

#include "../../include/ava_engine.h"
#include "kernels.cuh"

namespace {

uint64_t splitmix_next(uint64_t* state) {
    *state += 0x9E3779B97F4A7C15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

uint32_t argmax_lowest(const float* x, int n) {
    int best = 0;
    for (int i = 1; i < n; ++i)
        if (x[i] > x[best]) best = i;
    return (uint32_t)best;
}

struct StateOwner {
    ava_state* s = nullptr;
    StateOwner() = default;
    explicit StateOwner(ava_state* p) : s(p) {}
    StateOwner(StateOwner&& o) noexcept : s(o.s) { o.s = nullptr; }
    StateOwner& operator=(StateOwner&& o) noexcept {
        if (this != &o) {
            if (s) ava_state_destroy(s);
            s = o.s;
            o.s = nullptr;
        }
        return *this;
    }
    StateOwner(const StateOwner&) = delete;
    StateOwner& operator=(const StateOwner&) = delete;
    ~StateOwner() {
        if (s) ava_state_destroy(s);
    }
};

}  // namespace

extern "C" {

uint64_t ava_splitmix64_next(uint64_t* state) { return state ? splitmix_next(state) : 0; }

int ava_pick(const float* logits, int32_t vocab, float temperature, int32_t top_k, uint64_t* rng_state, uint32_t* token, float* logp,
             float* sample_logp) {
    if (!logits || vocab <= 0 || !token) return AVA_ERR_ARG;
    // ln p(token) under the model itself (temperature 1, every token allowed), in f64 as `pick_traced` takes it
    auto model_logp = [&](uint32_t j) {
        double mx = -INFINITY;
        for (int i = 0; i < vocab; ++i) mx = std::max(mx, (double)logits[i]);
        double sum = 0.0;
        for (int i = 0; i < vocab; ++i) sum += std::exp((double)logits[i] - mx);
        return (float)((double)logits[j] - (mx + std::log(sum)));
    };
    if (temperature <= 0.0f) {
        *token = argmax_lowest(logits, vocab);
        if (logp) *logp = model_logp(*token);
        if (sample_logp) *sample_logp = 0.0f;
        return AVA_OK;
    }
    if (!rng_state) return AVA_ERR_ARG;
    // softmax(logits * (1 / temperature)) in f32: largest value out, exp, sum in index order, divide
    const float inv_t = (float)(1.0 / (double)temperature);
    std::vector<float> p((size_t)vocab);
    float mx = -INFINITY;
    for (int i = 0; i < vocab; ++i) {
        p[i] = logits[i] * inv_t + 0.0f;
        mx = std::max(mx, p[i]);
    }
    float sum = 0.0f;
    for (int i = 0; i < vocab; ++i) {
        p[i] = ava_host_expf(p[i] - mx);
        sum += p[i];
    }
    for (int i = 0; i < vocab; ++i) p[i] = p[i] / sum;
    // the top_k most likely, ties in index order (a stable descending sort cut at top_k)
    const int k = std::max(1, std::min((int)top_k, (int)vocab));
    std::vector<int> order((size_t)vocab);
    std::iota(order.begin(), order.end(), 0);
    std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](int a, int b) { return p[a] > p[b] || (p[a] == p[b] && a < b); });
    double total = 0.0;
    for (int j = 0; j < k; ++j) total += (double)p[order[j]];
    double r = (double)(splitmix_next(rng_state) >> 11) / (double)(1ull << 53) * total;
    int out = order[k - 1];
    for (int j = 0; j < k; ++j) {
        r -= (double)p[order[j]];
        if (r <= 0.0) {
            out = order[j];
            break;
        }
    }
    *token = (uint32_t)out;
    if (logp) *logp = model_logp(*token);
    if (sample_logp) *sample_logp = (float)std::log((double)p[out] / total);
    return AVA_OK;
}

namespace {
struct Sampler {
    float temperature;
    int32_t top_k;
    uint64_t* rng;
};
}  // namespace

static int generate_impl(ava_engine* e, const uint32_t* prompts, const int32_t* prompt_len, int32_t n_prompts, int32_t max_new, int32_t batch_rows,
                         int32_t max_ctx, uint32_t eos, ava_pick_fn pick, const Sampler* smp, ava_stop_fn stop, void* user, uint32_t* out,
                         int32_t* out_len) {
    if (!e || !prompts || !prompt_len || n_prompts <= 0 || max_new < 0 || !out || !out_len) return AVA_ERR_ARG;
    std::vector<size_t> start((size_t)n_prompts);
    size_t at = 0;
    int longest = 0;
    for (int r = 0; r < n_prompts; ++r) {
        if (prompt_len[r] <= 0) return AVA_ERR_ARG;  // `generate: an empty prompt`
        start[r] = at;
        at += (size_t)prompt_len[r];
        longest = std::max(longest, (int)prompt_len[r]);
        out_len[r] = 0;
    }
    if (max_ctx <= 0) max_ctx = longest + max_new + 1;
    if (max_ctx < longest + max_new) return AVA_ERR_CAPACITY;
    const ava_config* cfg = ava_engine_config(e);
    const int V = cfg->vocab;
    // decided once per call: the draws are taken on the device when its sampler covers (vocabulary, top_k); when it
    // does not, every step returns its logits and `ava_pick` draws on the host from the same generator (`diary::pick`
    // works for any top_k, src/diary.rs:686-718)
    const bool dev_sampler = smp && smp->temperature > 0.0f && ava::sample_covered(V, smp->top_k);
    const bool host_sampler = smp && smp->temperature > 0.0f && !dev_sampler;
    std::vector<int> order((size_t)n_prompts);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return prompt_len[a] < prompt_len[b]; });
    const int br = std::max(1, (int)batch_rows);
    std::vector<float> logits;
    std::vector<uint32_t> next_tok;
    for (size_t i = 0; i < order.size();) {
        // a group: up to br rows; each run of equal-length prompts is read in one pass
        const std::vector<int> group(order.begin() + i, order.begin() + std::min(order.size(), i + (size_t)br));
        i += group.size();
        std::vector<StateOwner> parts;
        std::vector<float> last((size_t)group.size() * ((pick || smp) ? V : 0));
        bool first_pick = smp != nullptr;  // the sampler's first token of a group comes from the prompt's logits on the host
        std::vector<uint32_t> greedy(group.size());
        for (size_t j = 0; j < group.size();) {
            const int len = prompt_len[group[j]];
            size_t run = 0;
            while (j + run < group.size() && prompt_len[group[j + run]] == len) ++run;
            std::vector<uint32_t> ids(run * (size_t)len);
            for (size_t k = 0; k < run; ++k) std::memcpy(&ids[k * len], prompts + start[group[j + k]], (size_t)len * sizeof(uint32_t));
            ava_state* st = nullptr;
            int rc = ava_state_new(e, (int32_t)run, max_ctx, &st);
            if (rc) return rc;
            parts.emplace_back(st);
            logits.resize(run * (size_t)V);
            if ((rc = ava_forward_with_state(e, st, ids.data(), len, 1, logits.data()))) return rc;
            for (size_t k = 0; k < run; ++k) {
                if (pick || smp) std::memcpy(&last[(j + k) * V], &logits[k * V], (size_t)V * sizeof(float));
                else greedy[j + k] = argmax_lowest(&logits[k * V], V);
            }
            j += run;
        }
        StateOwner st;
        if (parts.size() == 1) {
            st = std::move(parts[0]);
        } else {
            std::vector<const ava_state*> ptrs;
            for (const StateOwner& p : parts) ptrs.push_back(p.s);
            ava_state* joined = nullptr;
            const int rc = ava_state_cat(ptrs.data(), (int32_t)ptrs.size(), &joined);
            if (rc) return rc;
            st = StateOwner(joined);
        }
        parts.clear();
        std::vector<int> live(group);  // prompt index of each state row
        if (first_pick && dev_sampler && max_new > 0) {
            // the first tokens, from the prompts' logits: drawn on the device too when the sampler covers the case (the
            // uniform numbers in the rows' order, as the loop below would draw them)
            uint64_t saved = *smp->rng;
            std::vector<double> u(live.size());
            for (double& v : u) v = (double)(splitmix_next(smp->rng) >> 11) / (double)(1ull << 53);
            if (ava_op_sample(ava_engine_device(e), last.data(), (int32_t)live.size(), V, smp->temperature, smp->top_k, u.data(), greedy.data()) == AVA_OK)
                first_pick = false;
            else
                *smp->rng = saved;  // not covered: the host sampler takes them, from the same generator state
        }
        for (int step = 0; step < max_new; ++step) {
            std::vector<int32_t> keep;
            std::vector<uint32_t> next;
            for (size_t k = 0; k < live.size(); ++k) {
                const int r = live[k];
                uint32_t tok;
                if (pick) {
                    tok = pick(user, r, &last[k * V], V);
                } else if (first_pick) {
                    const int prc = ava_pick(&last[k * V], V, smp->temperature, smp->top_k, smp->rng, &tok, nullptr, nullptr);
                    if (prc) return prc;
                } else {
                    tok = greedy[k];
                }
                if (tok == eos) continue;
                out[(size_t)r * max_new + out_len[r]++] = tok;
                if (stop && stop(user, r, out + (size_t)r * max_new, out_len[r])) continue;
                keep.push_back((int32_t)k);
                next.push_back(tok);
            }
            if (!host_sampler) first_pick = false;  // a sampler the device does not cover keeps drawing on the host
            if (keep.empty() || step + 1 == max_new) break;
            if (keep.size() != live.size()) {
                ava_state* sel = nullptr;
                const int rc = ava_state_select(st.s, keep.data(), (int32_t)keep.size(), &sel);
                if (rc) return rc;
                st = StateOwner(sel);
                std::vector<int> nl;
                for (int32_t k : keep) nl.push_back(live[k]);
                live.swap(nl);
            }
            int rc;
            if (pick || host_sampler) {
                last.resize(next.size() * (size_t)V);
                rc = ava_step(e, st.s, next.data(), last.data());
            } else if (smp && smp->temperature > 0.0f) {
                // the next pass picks for the live rows in order: their draws are taken now, in that order
                std::vector<double> u(next.size());
                for (double& v : u) v = (double)(splitmix_next(smp->rng) >> 11) / (double)(1ull << 53);
                greedy.resize(next.size());
                rc = ava_step_sample(e, st.s, next.data(), smp->temperature, smp->top_k, u.data(), greedy.data());
            } else {
                greedy.resize(next.size());
                rc = ava_step_greedy(e, st.s, next.data(), greedy.data());  // the arg-max is taken on the device
            }
            if (rc) return rc;
        }
    }
    return AVA_OK;
}

int ava_generate(ava_engine* e, const uint32_t* prompts, const int32_t* prompt_len, int32_t n_prompts, int32_t max_new, int32_t batch_rows,
                 int32_t max_ctx, uint32_t eos, ava_pick_fn pick, ava_stop_fn stop, void* user, uint32_t* out, int32_t* out_len) {
    return generate_impl(e, prompts, prompt_len, n_prompts, max_new, batch_rows, max_ctx, eos, pick, nullptr, stop, user, out, out_len);
}

int ava_generate_sampled(ava_engine* e, const uint32_t* prompts, const int32_t* prompt_len, int32_t n_prompts, int32_t max_new, int32_t batch_rows,
                         int32_t max_ctx, uint32_t eos, float temperature, int32_t top_k, uint64_t* rng_state, ava_stop_fn stop, void* user,
                         uint32_t* out, int32_t* out_len) {
    if (!rng_state) return AVA_ERR_ARG;
    const Sampler smp{temperature, top_k, rng_state};
    return generate_impl(e, prompts, prompt_len, n_prompts, max_new, batch_rows, max_ctx, eos, nullptr, &smp, stop, user, out, out_len);
}

}  // extern "C"

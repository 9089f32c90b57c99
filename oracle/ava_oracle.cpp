// CPU oracle for the per-token block step of the Ava spiking language model.
// TEST INFRASTRUCTURE ONLY: see ava_oracle.h for what it is, what it follows and who may load it.
//
// Build with -ffp-contract=off: every multiply-add that the reference fuses is written std::fmaf here, and every
// one it does not fuse must stay two roundings.

#include "ava_oracle.h"

#include <algorithm>
#include <cmath>
#include <limits>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#define ORC_HAVE_AVX2 1
#else
#define ORC_HAVE_AVX2 0
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ------------------------------------------------------------------------------------------------ math hooks
float libm_exp(float x) { return std::exp(x); }
float libm_log(float x) { return std::log(x); }
// Rust's f32::powf(-0.5) is the platform powf
float libm_rsqrt(float x) { return std::pow(x, -0.5f); }

float libm_sin(float x) { return std::sin(x); }
float libm_cos(float x) { return std::cos(x); }
orc_fn1 g_exp = libm_exp, g_log = libm_log, g_rsqrt = libm_rsqrt, g_sin = libm_sin, g_cos = libm_cos;
int g_threads = 1;
int g_simd = 1;
double g_event_max = 0.5;  // int8.rs:459
thread_local int g_last_event_rows = 0;

constexpr int TILE = 64;       // int8.rs:41
constexpr float NORM_EPS = 1e-5f;  // model.rs:36

// ------------------------------------------------------------------------------------------------ A0 quantiser
// quant.rs:18-31: scale[c] = max_r |w[r][c]| / 127 (1 when the column is all zero); q = round(w / scale)
// clamped to +-127, round = half away from zero (Rust f32::round).
void quantize_int8(const float* w, int rows, int cols, int8_t* q, float* scale) {
    for (int c = 0; c < cols; ++c) scale[c] = 0.f;
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) scale[c] = std::max(scale[c], std::fabs(w[(size_t)r * cols + c]));
    for (int c = 0; c < cols; ++c) scale[c] = scale[c] > 0.f ? scale[c] / 127.0f : 1.0f;
    for (size_t i = 0; i < (size_t)rows * cols; ++i) {
        float v = std::round(w[i] / scale[i % cols]);  // roundf: half away from zero
        v = std::min(std::max(v, -127.0f), 127.0f);
        q[i] = (int8_t)v;
    }
}

// ------------------------------------------------------------------------------------------------ A1 int8 products
// One weight matrix W [din, dout] in int8 with one f32 scale per output column, packed in column tiles of 64
// (int8.rs:46-72): q[(tile * din + j) * 64 + cc], columns past dout are 0 with scale 1.
struct QW {
    int din = 0, dout = 0, tiles = 0;
    std::vector<int8_t> q;
    std::vector<float> scale;

    void from_q(const int8_t* qr, const float* sc, int din_, int dout_) {
        din = din_;
        dout = dout_;
        tiles = (dout + TILE - 1) / TILE;
        q.assign((size_t)tiles * din * TILE, 0);
        scale.assign((size_t)tiles * TILE, 1.0f);
        std::copy(sc, sc + dout, scale.begin());
        for (int j = 0; j < din; ++j)
            for (int c = 0; c < dout; ++c) q[((size_t)(c / TILE) * din + j) * TILE + c % TILE] = qr[(size_t)j * dout + c];
    }
    bool ok() const { return din > 0; }
};

// -0 counts as zero, NaN as non-zero (int8.rs:261-269)
inline bool nonzero(float v) { return v != 0.0f; }

// int8.rs:315-331: acc from +0, fma(x[j], (f32) q[j][c], acc) over every j or the listed non-zero j, increasing;
// then acc * scale.
void tile_scalar(const float* x, int din, const int* idx, int nidx, const int8_t* qt, const float* sc, float* out, int n_out) {
    float acc[TILE];
    for (int c = 0; c < TILE; ++c) acc[c] = 0.f;
    auto add = [&](int j) {
        const float xj = x[j];
        const int8_t* row = qt + (size_t)j * TILE;
        for (int c = 0; c < TILE; ++c) acc[c] = std::fmaf(xj, (float)row[c], acc[c]);
    };
    if (idx)
        for (int i = 0; i < nidx; ++i) add(idx[i]);
    else
        for (int j = 0; j < din; ++j) add(j);
    for (int c = 0; c < n_out; ++c) out[c] = acc[c] * sc[c];
}

#if ORC_HAVE_AVX2
// The reference's AVX2 kernel (int8.rs:389-435) keeps 8 accumulators of 8 lanes over one 64-column tile row; each
// lane is the same fma chain as the scalar code, so the same bits.
inline __m256 w8(const int8_t* p) { return _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i*)p))); }

void tile_avx2(const float* x, int din, const int* idx, int nidx, const int8_t* qt, const float* sc, float* out, int n_out) {
    __m256 a[8];
    for (auto& v : a) v = _mm256_setzero_ps();
    auto add = [&](int j) {
        const __m256 xb = _mm256_set1_ps(x[j]);
        const int8_t* p = qt + (size_t)j * TILE;
        for (int v = 0; v < 8; ++v) a[v] = _mm256_fmadd_ps(xb, w8(p + 8 * v), a[v]);
    };
    if (idx)
        for (int i = 0; i < nidx; ++i) add(idx[i]);
    else
        for (int j = 0; j < din; ++j) add(j);
    alignas(32) float buf[TILE];
    for (int v = 0; v < 8; ++v) _mm256_store_ps(buf + 8 * v, _mm256_mul_ps(a[v], _mm256_loadu_ps(sc + 8 * v)));
    std::memcpy(out, buf, sizeof(float) * n_out);
}
#endif

void tile_any(const float* x, int din, const int* idx, int nidx, const int8_t* qt, const float* sc, float* out, int n_out) {
#if ORC_HAVE_AVX2
    if (g_simd) return tile_avx2(x, din, idx, nidx, qt, sc, out, n_out);
#endif
    tile_scalar(x, din, idx, nidx, qt, sc, out, n_out);
}

// int8.rs:166-211 without the row-blocked kernel (which changes the speed only): per row its non-zero count, an event
// list when the count is at most event_max * din, then one (tile, row) unit after another.
void q8_matmul(const QW& w, const float* x, int m, float* y) {
    const int din = w.din;
    std::vector<int> off(m + 1, 0);
    std::vector<char> ev(m, 0);
    std::vector<int> cnt(m, 0);
    const double lim = g_event_max * (double)din;
    for (int r = 0; r < m; ++r) {
        int c = 0;
        for (int j = 0; j < din; ++j) c += nonzero(x[(size_t)r * din + j]);
        cnt[r] = c;
        ev[r] = (double)c <= lim;
        off[r + 1] = off[r] + (ev[r] ? c : 0);
    }
    std::vector<int> idx(off[m]);
    int nev = 0;
    for (int r = 0; r < m; ++r) {
        if (!ev[r]) continue;
        ++nev;
        int n = off[r];
        for (int j = 0; j < din; ++j)
            if (nonzero(x[(size_t)r * din + j])) idx[n++] = j;
    }
    g_last_event_rows = nev;
    const int units = m * w.tiles;
    // unit u: tile u / m, row u % m (int8.rs:184-195)
    auto run = [&](int u) {
        const int t = u / m, r = u % m;
        const int c0 = t * TILE;
        const int n_out = std::min(TILE, w.dout - c0);
        tile_any(x + (size_t)r * din, din, ev[r] ? idx.data() + off[r] : nullptr, off[r + 1] - off[r], w.q.data() + (size_t)t * din * TILE,
                 w.scale.data() + c0, y + (size_t)r * w.dout + c0, n_out);
    };
    size_t work = 0;
    for (int r = 0; r < m; ++r) work += ev[r] ? cnt[r] : din;
    work *= (size_t)w.tiles * TILE;
    const int want = (int)std::min<size_t>({(size_t)g_threads, work / (1u << 16), (size_t)units});  // PAR_MIN, int8.rs:44
    if (want <= 1) {
        for (int u = 0; u < units; ++u) run(u);
    } else {
#pragma omp parallel for num_threads(want) schedule(static)
        for (int u = 0; u < units; ++u) run(u);
    }
}

// ------------------------------------------------------------------------------------------------ A2 small ops
// fstep.rs:212-220: squares summed one after another from 0, the mean's affine (sum * (1/n) + 0), affine(1, eps),
// powf(-0.5).
float inv_rms(const float* x, int n) {
    float s = 0.f;
    for (int i = 0; i < n; ++i) s += x[i] * x[i];
    const float ms = s * (float)(1.0 / (double)n) + 0.0f;
    return g_rsqrt(ms * 1.0f + NORM_EPS);
}

void rmsnorm(const float* x, const float* gain, int n, float* y) {
    const float inv = inv_rms(x, n);
    for (int i = 0; i < n; ++i) y[i] = (x[i] * inv) * gain[i];
}

// fstep.rs:271-282
void l2_heads(float* x, int n, int hs) {
    for (int h = 0; h + hs <= n; h += hs) {
        float s = 0.f;
        for (int i = 0; i < hs; ++i) s += x[h + i] * x[h + i];
        const float inv = g_rsqrt(s * 1.0f + (float)1e-6);
        for (int i = 0; i < hs; ++i) x[h + i] = x[h + i] * inv;
    }
}

// fstep.rs:285-292
void head_norm(float* y, int n, int hs) {
    for (int h = 0; h + hs <= n; h += hs) {
        const float inv = inv_rms(y + h, hs);
        for (int i = 0; i < hs; ++i) y[h + i] = y[h + i] * inv;
    }
}

// tanh as Rust's f32::tanh (the platform's libm), or, when another exp has been plugged in (orc_set_math), the
// composite from that exp that the engine's kernels use: the two sides then agree bit for bit.
float tanh_f(float x) {
    if (g_exp == libm_exp) return std::tanh(x);
    const float ax = std::fabs(x);
    if (!(ax == ax)) return std::numeric_limits<float>::quiet_NaN();
    if (ax < 2.44140625e-4f) return x;
    if (ax > 9.5f) return x > 0.0f ? 1.0f : -1.0f;
    const float t = g_exp(ax * -2.0f);
    const float r = (1.0f - t) / (1.0f + t);
    return x < 0.0f ? -r : r;
}

// fstep.rs:260-262: (exp(-x) * 1 + 1)^-1
float sigmoid(float x) { return 1.0f / (g_exp(-x) * 1.0f + 1.0f); }

// fstep.rs:265-268: -(relu(-x) + ln(exp(-|x|) * 1 + 1))
float log_sigmoid(float x) {
    const float soft = g_log(g_exp(-std::fabs(x)) * 1.0f + 1.0f);
    return -(std::max(-x, 0.0f) + soft);
}

// fstep.rs:222-257: the one-row f32 product in gemm's order: out = w0 * x0, then fma(w_j, x_j, out); 2 inputs:
// (w1 * x1) + (w0 * x0); 1 input: the product.
void gemv(const float* x, int k, const float* w, int n, float* out) {
    if (k == 0) {
        for (int c = 0; c < n; ++c) out[c] = 0.f;
    } else if (k == 1) {
        for (int c = 0; c < n; ++c) out[c] = w[c] * x[0];
    } else if (k == 2) {
        for (int c = 0; c < n; ++c) out[c] = w[n + c] * x[1] + w[c] * x[0];
    } else {
        for (int c = 0; c < n; ++c) out[c] = w[c] * x[0];
        for (int j = 1; j < k; ++j) {
            const float xj = x[j];
            const float* wr = w + (size_t)j * n;
            for (int c = 0; c < n; ++c) out[c] = std::fmaf(wr[c], xj, out[c]);
        }
    }
}

void add_into(float* x, const float* o, int n) {
    for (int i = 0; i < n; ++i) x[i] = x[i] + o[i];
}

bool all_finite(const float* x, int n) {
    for (int i = 0; i < n; ++i)
        if (!std::isfinite(x[i])) return false;
    return true;
}

// ------------------------------------------------------------------------------------------------ A3 LIF
// fstep/arch.rs:173-228.  theta NULL: 1.0 for every channel; rho/gain NULL: no adaptive threshold.
void lif(const float* cur, const float* beta, const float* theta, const float* rho, const float* gain, int spikes, float slope,
         const float* v0, const float* s0, const float* a0, int d, float* s, float* v, float* a) {
    auto th = [&](int c) { return theta ? theta[c] : 1.0f; };
    const bool alif = rho && gain;
    if (spikes == 0 && !alif) {
        // state::lif_infer form: v = beta v + I - th s; s = H(v - th)
        for (int c = 0; c < d; ++c) {
            const float vv = beta[c] * v0[c] + cur[c] - th(c) * s0[c];
            v[c] = vv;
            s[c] = (vv - th(c) >= 0.0f) ? 1.0f : 0.0f;
        }
        return;
    }
    auto soft_step = [&](float u) { return u / (std::fabs(u) * slope + 1.0f); };
    auto heav = [](float u) { return u >= 0.0f ? 1.0f : 0.0f; };
    const int levels = spikes == 2 ? 2 : 1;
    for (int c = 0; c < d; ++c) {
        float th_prev, th_t;
        if (alif) {
            const float a_prev = a0 ? a0[c] : 0.0f;
            th_prev = th(c) + a_prev * gain[c];
            const float an = a_prev * rho[c] + std::fabs(s0[c]) * (rho[c] * -1.0f + 1.0f);
            a[c] = an;
            th_t = th(c) + an * gain[c];
        } else {
            th_prev = th_t = th(c);
        }
        const float vv = v0[c] * beta[c] + cur[c] - s0[c] * th_prev;
        v[c] = vv;
        if (spikes == 0) {
            const float u = vv - th_t;
            const float sg = soft_step(u);
            s[c] = sg + (heav(u) - sg);
        } else {
            float soft = 0.f, hard = 0.f;
            for (int k = 1; k <= levels; ++k) {
                const float kth = th_t * (float)k + 0.0f;
                const float up = vv - kth, down = -vv - kth;
                const float s1 = soft_step(up) - soft_step(down);
                const float h1 = heav(up) - heav(down);
                if (k == 1) {
                    soft = s1;
                    hard = h1;
                } else {
                    soft = soft + s1;
                    hard = hard + h1;
                }
            }
            s[c] = soft + (hard - soft);
        }
    }
}

// ------------------------------------------------------------------------------------------------ A5 fast-weight head
// fstep/arch.rs:256-337 (head_rows): F, S [hs, hs] (row = key dim, col = value dim).
//     rr = (e F + r0) + p2 S
//     y  = ((q alpha) F + (q.w) v) - (q.ah) rr + (q M) S
//     F' = ((F * alpha_row + w v^T) - ah rr^T) + S * M
//     S' = ((S * M + 0) + w v^T) - ah rr^T
void head_rows(int hs, const float* e, const float* v, const float* w, const float* ah, const float* qg, const float* ex, float qw, float qa,
               float ke, float tinv, bool mom, float m, const float* qs, const float* p2, const float* f0, const float* s0, float* y, float* f1,
               float* s1) {
    std::vector<float> rr(hs), t1(hs), tq;
    for (int a = 0; a < hs; ++a) {
        const float* frow = f0 + (size_t)a * hs;
        const float pa = e[a], ga = qg[a];
        if (a == 0) {
            for (int b = 0; b < hs; ++b) {
                rr[b] = frow[b] * pa;
                t1[b] = frow[b] * ga;
            }
        } else {
            for (int b = 0; b < hs; ++b) {
                rr[b] = std::fmaf(frow[b], pa, rr[b]);
                t1[b] = std::fmaf(frow[b], ga, t1[b]);
            }
        }
    }
    for (int b = 0; b < hs; ++b) rr[b] = rr[b] + tinv * (ke * v[b]);
    if (mom) {
        std::vector<float> z(hs);
        tq.assign(hs, 0.f);
        for (int a = 0; a < hs; ++a) {
            const float* srow = s0 + (size_t)a * hs;
            const float pa = p2[a], q_a = qs[a];
            if (a == 0) {
                for (int b = 0; b < hs; ++b) {
                    z[b] = srow[b] * pa;
                    tq[b] = srow[b] * q_a;
                }
            } else {
                for (int b = 0; b < hs; ++b) {
                    z[b] = std::fmaf(srow[b], pa, z[b]);
                    tq[b] = std::fmaf(srow[b], q_a, tq[b]);
                }
            }
        }
        for (int b = 0; b < hs; ++b) rr[b] = rr[b] + z[b];
    }
    for (int b = 0; b < hs; ++b) y[b] = (t1[b] + qw * v[b]) - qa * rr[b];
    if (mom)
        for (int b = 0; b < hs; ++b) y[b] = y[b] + tq[b];
    if (mom) {
        for (int a = 0; a < hs; ++a) {
            const float wa = w[a], aa = ah[a], xa = ex[a];
            const float* frow = f0 + (size_t)a * hs;
            const float* srow = s0 + (size_t)a * hs;
            for (int b = 0; b < hs; ++b) {
                const float wv = wa * v[b], ar = aa * rr[b];
                f1[(size_t)a * hs + b] = ((frow[b] * xa + wv) - ar) + srow[b] * m;
                s1[(size_t)a * hs + b] = ((srow[b] * m + 0.0f) + wv) - ar;
            }
        }
    } else {
        for (int a = 0; a < hs; ++a) {
            const float wa = w[a], aa = ah[a], xa = ex[a];
            const float* frow = f0 + (size_t)a * hs;
            for (int b = 0; b < hs; ++b) f1[(size_t)a * hs + b] = (frow[b] * xa + wa * v[b]) - aa * rr[b];
        }
    }
}

// ------------------------------------------------------------------------------------------------ A6 plain delta rule
// fstep.rs:397-436 (fw_rows, Rule::Delta) with p = k^T F by gemv (fstep.rs:592-595).
void delta_plain(int hs, const float* f0, const float* k, const float* v, const float* q, float al, float b, float* f1, float* y) {
    std::vector<float> p(hs);
    gemv(k, hs, f0, hs, p.data());
    for (int a = 0; a < hs; ++a) {
        const float ka = k[a], qa = q[a];
        for (int c = 0; c < hs; ++c) {
            const float corr = (ka * p[c]) * b;
            const float r = ((f0[(size_t)a * hs + c] - corr) * al) + ((ka * v[c]) * b);
            f1[(size_t)a * hs + c] = r;
            y[c] = a == 0 ? r * qa : std::fmaf(r, qa, y[c]);
        }
    }
}

// ------------------------------------------------------------------------------------------------ A7 kWTA
// fstep.rs:295-299: the k-th largest value (selection; ties give the same value).
float kth_largest(const float* u, int n, int k) {
    std::vector<float> b(u, u + n);
    std::nth_element(b.begin(), b.begin() + (k - 1), b.end(), [](float a, float c) { return a > c; });
    return b[k - 1];
}

// fstep/arch.rs:982-989
void kwta(const float* u, int n, int k, bool relu2, float* a) {
    if (k >= n) {
        for (int i = 0; i < n; ++i) a[i] = std::max(u[i] * 1.0f, 0.0f);
    } else {
        const float kth = kth_largest(u, n, k);
        for (int i = 0; i < n; ++i) a[i] = std::max(u[i] * ((u[i] - kth >= 0.0f) ? 1.0f : 0.0f), 0.0f);
    }
    if (relu2)
        for (int i = 0; i < n; ++i) a[i] = a[i] * a[i];
}

// --cerebellum-head's fixed wiring (src/v51b.rs:241-266): Marsaglia's xorshift64 (13, 7, 17) from seed | 1; per unit
// `fan_in` distinct inputs (a draw modulo the input count, redrawn while already picked), then per input one more
// draw whose lowest bit gives the sign of 1 / sqrt(fan_in).
void cb_wiring(int inputs, int g, int fan_in, uint64_t seed, std::vector<uint32_t>* idx, std::vector<float>* w) {
    uint64_t s = seed | 1;
    auto next = [&]() {
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        return s;
    };
    const float amp = 1.0f / std::sqrt((float)fan_in);
    idx->clear();
    w->clear();
    std::vector<uint32_t> picked;
    for (int u = 0; u < g; ++u) {
        picked.clear();
        while ((int)picked.size() < std::min(fan_in, inputs)) {
            const uint32_t r = (uint32_t)(next() % (uint64_t)inputs);
            if (std::find(picked.begin(), picked.end(), r) == picked.end()) picked.push_back(r);
        }
        for (uint32_t r : picked) {
            idx->push_back(r);
            w->push_back((next() & 1) == 0 ? amp : -amp);
        }
    }
}

// ------------------------------------------------------------------------------------------------ A8 engram read
// fstep.rs:303-356: per key the score chain K[j][0] q0, then fma(K[j][a], q[a], .), times scale plus 0; softmax with
// the max found by "replace while mx < s", exp(s - mx), the sum from 0, each divided; then the one-row product p . V.
void attend(const float* q, const float* kc, const float* vc, int n, int hs, float scale, float* out) {
    std::vector<float> sc(n);
    for (int j = 0; j < n; ++j) {
        const float* kr = kc + (size_t)j * hs;
        float s = kr[0] * q[0];
        for (int a = 1; a < hs; ++a) s = std::fmaf(kr[a], q[a], s);
        sc[j] = s * scale + 0.0f;
    }
    float mx = sc[0];
    for (int j = 0; j < n; ++j)
        if (mx < sc[j]) mx = sc[j];
    float den = 0.f;
    for (int j = 0; j < n; ++j) {
        sc[j] = g_exp(sc[j] - mx);
        den += sc[j];
    }
    for (int j = 0; j < n; ++j) sc[j] = sc[j] / den;
    gemv(sc.data(), n, vc, hs, out);
}

float bf16_round(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {  // NaN stays NaN
        u |= 0x00400000u;
        u &= 0xffff0000u;
    } else {
        u += 0x7fffu + ((u >> 16) & 1u);
        u &= 0xffff0000u;
    }
    float r;
    std::memcpy(&r, &u, 4);
    return r;
}

// ------------------------------------------------------------------------------------------------ trace
struct Trace {
    bool on = false;
    std::map<std::pair<std::string, int>, std::vector<float>> t;
    void put(const char* name, int block, const float* p, size_t n) {
        if (on) t[{name, block}] = std::vector<float>(p, p + n);
    }
    void put(const char* name, int block, const std::vector<float>& v) { put(name, block, v.data(), v.size()); }
};
Trace g_trace;

}  // namespace

// ================================================================================================ model level
struct Block {
    // the spiking memory
    std::vector<float> mem_norm, beta_param, theta, arho, again;
    QW win, wout;
    // short-term plasticity of the spikes' synapse (--stp): parameters and their sigmoids
    std::vector<float> stp_u, stp_f, stp_d, stp_mix, stp_U, stp_F, stp_D;
    std::vector<float> rh_w, rh_r;          // --rhythm: the write strength's and the read's gates [4, heads]
    std::vector<float> da_w, da_c, mood_g;  // --dopamine: gate [d] twice; --mood: gain [k, d] (blocks after the first)
    // the dendrites of the MLP's units (--dendrite): A [d, 32], B [32, hidden]
    std::vector<float> dend_a, dend_b;
    // the fast-weight memory
    std::vector<float> hebb_norm, wa, wb, ba, bb, wa1, wa2, wb1, wb2, off, vres;
    QW wq, wk, wv, we, wg, wo;
    // the engram
    std::vector<float> eng_norm;
    QW ewq, ewk, ewv, ewo;
    // the MLP
    std::vector<float> mlp_norm;
    QW w1, w2;
    std::vector<float> dense;
    // derived once: sigmoid(beta_param), sigmoid(arho)
    std::vector<float> beta, rho;
    bool derived = false;
};

struct orc_model {
    orc_config cfg;
    std::vector<float> tok_emb, final_norm;
    std::vector<float> nm_norm, nm_wn, nm_bn;  // --neuromod: the nucleus (gain [d], read-out [d, k], bias [k])
    std::vector<float> rhy_lw, rhy_wr, rhy_br;  // --rhythm: log frequencies [2], reset read-out [d, 2] and bias [2]
    std::vector<float> mood_lam, mood_win, mood_bin;  // --mood: decay, input weight and bias [k]
    // --letters (src/v51.rs:449-482): per token 16 byte ids, their places counted from the end, a mask and 1 / sqrt(used);
    // byte [256, 64], pos [16, 64], end [16, 64] embeddings and the read-out [64, d]
    std::vector<uint32_t> let_ids, let_eidx;
    std::vector<float> let_mask, let_inv, let_byte, let_pos, let_end, let_wo;
    std::vector<float> cb_w;     // --cerebellum-head: the read-out [G, d]
    std::vector<uint32_t> cb_idx;  // its fixed wiring: 4 inputs of [xf, rmsnorm(emb)] per unit, weights +-1/2
    std::vector<float> cb_sgn;
    std::vector<float> th_read, th_gate, th_bias;  // --thalamus: reads [L, d, 16], gates [L, 16, 2], biases [L, 2]
    QW head;
    std::vector<Block> blocks;
    int nh() const { return cfg.d / cfg.head_size; }
    int enh() const { return cfg.d / cfg.eng_head_size; }
};

struct RowState {
    std::vector<std::vector<float>> v, s, a;    // per block [d]
    std::vector<std::vector<float>> f, ms;      // per block [nh, hs, hs]
    std::vector<std::vector<float>> su, sx;     // per block [d]: the synapse's (u, x) with --stp
    std::vector<float> rh;                      // --rhythm: the time since each clock's last reset [2]
    std::vector<float> prev, mood;              // --dopamine / --mood: block 0's last normed output [d], the mood [k]
    std::vector<float> pvalid, last_s;          // [1] each: whether there is a prev, the last surprise
    std::vector<float> ek, evv;                 // engram [enh, n, ehs]
    int eng_n = 0;
    int64_t seen = 0;
};

struct orc_state {
    const orc_model* m;
    std::vector<RowState> rows;
};

namespace {

std::vector<float>* f32_slot(orc_model* m, const std::string& name, int64_t* want) {
    const orc_config& c = m->cfg;
    const int d = c.d, nh = m->nh(), r = c.gate_rank;
    if (name == "tok_emb") { *want = (int64_t)c.vocab * d; return &m->tok_emb; }
    if (name == "nm.norm") { *want = d; return &m->nm_norm; }
    if (name == "nm.wn") { *want = (int64_t)d * c.neuromod; return &m->nm_wn; }
    if (name == "nm.bn") { *want = c.neuromod; return &m->nm_bn; }
    if (name == "v51.rhythm.lw") { *want = 2; return &m->rhy_lw; }
    if (name == "v51.rhythm.wr") { *want = (int64_t)d * 2; return &m->rhy_wr; }
    if (name == "v51.rhythm.br") { *want = 2; return &m->rhy_br; }
    if (name == "v51.mood.lam") { *want = c.mood; return &m->mood_lam; }
    if (name == "v51.mood.win") { *want = c.mood; return &m->mood_win; }
    if (name == "v51.mood.bin") { *want = c.mood; return &m->mood_bin; }
    if (name == "v51.letters.byte") { *want = 256 * 64; return &m->let_byte; }
    if (name == "v51.letters.pos") { *want = 16 * 64; return &m->let_pos; }
    if (name == "v51.letters.end") { *want = 16 * 64; return &m->let_end; }
    if (name == "v51.letters.wo") { *want = (int64_t)64 * d; return &m->let_wo; }
    if (name == "cbh.wo") { *want = (int64_t)c.cb_units * d; return &m->cb_w; }
    if (name == "th.read") { *want = (int64_t)c.n_blocks * d * 16; return &m->th_read; }
    if (name == "th.gate") { *want = (int64_t)c.n_blocks * 16 * 2; return &m->th_gate; }
    if (name == "th.bias") { *want = (int64_t)c.n_blocks * 2; return &m->th_bias; }
    if (name == "final.norm") { *want = d; return &m->final_norm; }
    if (name.size() < 3 || name[0] != 'b') return nullptr;
    const size_t dot = name.find('.');
    if (dot == std::string::npos) return nullptr;
    const int i = std::atoi(name.substr(1, dot - 1).c_str());
    if (i < 0 || i >= c.n_blocks) return nullptr;
    Block& b = m->blocks[i];
    b.derived = false;
    const std::string rest = name.substr(dot + 1);
    struct E { const char* n; std::vector<float>* p; int64_t len; };
    const E table[] = {
        {"mem.norm", &b.mem_norm, d}, {"mem.beta", &b.beta_param, d}, {"mem.theta", &b.theta, d}, {"mem.arho", &b.arho, d},
        {"mem.again", &b.again, d}, {"parts.stp.u_param", &b.stp_u, d}, {"parts.stp.f_param", &b.stp_f, d}, {"parts.stp.d_param", &b.stp_d, d},
        {"parts.stp.mix", &b.stp_mix, d}, {"v51.dend_a", &b.dend_a, (int64_t)d * 32}, {"v51.dend_b", &b.dend_b, (int64_t)32 * c.hidden},
        {"hebb.norm", &b.hebb_norm, d}, {"hebb.wa", &b.wa, (int64_t)d * nh}, {"hebb.wb", &b.wb, (int64_t)d * nh},
        {"hebb.ba", &b.ba, nh}, {"hebb.bb", &b.bb, nh}, {"hebb.wa1", &b.wa1, (int64_t)d * r}, {"hebb.wa2", &b.wa2, (int64_t)r * d},
        {"hebb.wb1", &b.wb1, (int64_t)d * r}, {"hebb.wb2", &b.wb2, (int64_t)r * d}, {"hebb.off", &b.off, d}, {"hebb.vres", &b.vres, 2},
        {"eng.norm", &b.eng_norm, d}, {"mlp.norm", &b.mlp_norm, d}, {"dense", &b.dense, i + 2},
        {"v51.rh_w", &b.rh_w, (int64_t)4 * nh}, {"v51.rh_r", &b.rh_r, (int64_t)4 * nh}, {"v51.da_w", &b.da_w, d}, {"v51.da_c", &b.da_c, d}, {"v51.mood_g", &b.mood_g, (int64_t)c.mood * d},
    };
    for (const E& e : table)
        if (rest == e.n) { *want = e.len; return e.p; }
    return nullptr;
}

QW* q8_slot(orc_model* m, const std::string& name, int* din, int* dout) {
    const orc_config& c = m->cfg;
    const int d = c.d;
    if (name == "head") { *din = d; *dout = c.vocab; return &m->head; }
    if (name.size() < 3 || name[0] != 'b') return nullptr;
    const size_t dot = name.find('.');
    if (dot == std::string::npos) return nullptr;
    const int i = std::atoi(name.substr(1, dot - 1).c_str());
    if (i < 0 || i >= c.n_blocks) return nullptr;
    Block& b = m->blocks[i];
    const std::string rest = name.substr(dot + 1);
    struct E { const char* n; QW* p; int din, dout; };
    const E table[] = {
        {"mem.win", &b.win, d, d}, {"mem.wout", &b.wout, d, d}, {"hebb.wq", &b.wq, d, d}, {"hebb.wk", &b.wk, d, d}, {"hebb.wv", &b.wv, d, d},
        {"hebb.we", &b.we, d, d}, {"hebb.wg", &b.wg, d, d}, {"hebb.wo", &b.wo, d, d}, {"eng.wq", &b.ewq, d, d}, {"eng.wk", &b.ewk, d, d},
        {"eng.wv", &b.ewv, d, d}, {"eng.wo", &b.ewo, d, d}, {"mlp.w1", &b.w1, d, c.hidden}, {"mlp.w2", &b.w2, c.hidden, d},
    };
    for (const E& e : table)
        if (rest == e.n) { *din = e.din; *dout = e.dout; return e.p; }
    return nullptr;
}

void derive(const orc_model* mc) {
    orc_model* m = const_cast<orc_model*>(mc);
    for (Block& b : m->blocks) {
        if (b.derived) continue;
        b.beta.resize(b.beta_param.size());
        for (size_t c = 0; c < b.beta.size(); ++c) b.beta[c] = sigmoid(b.beta_param[c]);  // fstep/arch.rs:640
        b.rho.resize(b.arho.size());
        for (size_t c = 0; c < b.rho.size(); ++c) b.rho[c] = sigmoid(b.arho[c]);  // fstep/arch.rs:660
        b.stp_U.resize(b.stp_u.size());
        b.stp_F.resize(b.stp_f.size());
        b.stp_D.resize(b.stp_d.size());
        for (size_t c = 0; c < b.stp_u.size(); ++c) {  // fstep/arch_f3.rs:82
            b.stp_U[c] = sigmoid(b.stp_u[c]);
            b.stp_F[c] = sigmoid(b.stp_f[c]);
            b.stp_D[c] = sigmoid(b.stp_d[c]);
        }
        b.derived = true;
    }
}

// S: the spikes s [d] through the synapse from its carried (u, x) (fstep/arch_f3.rs:72-106; the part itself:
// nn/parts/src/stp.rs:42-85): what reaches W_out, the new (u, x), and the efficacy e / U of each channel.
void stp_step(const float* s, const float* U, const float* F, const float* D, const float* mix, const float* u0, const float* x0, int d,
              float* out, float* u1, float* x1, float* eff_out) {
    for (int c = 0; c < d; ++c) {
        const float uu = U[c], df = F[c], dd = D[c], sv = s[c];
        // ava_parts::stp::events: k = (s >= 0)(s <= 1) - (s < 0)(s >= -1), s k + (clamp(|s|, 0, 1) - s k)
        auto f = [](bool b) { return b ? 1.0f : 0.0f; };
        const float k = f(sv >= 0.0f) * f(sv <= 1.0f) - f(sv < 0.0f) * f(sv >= -1.0f);
        const float sk = sv * k;
        float a = std::fabs(sv);
        a = a < 0.0f ? 0.0f : a;
        a = a > 1.0f ? 1.0f : a;
        const float ev = sk + (a - sk);
        const float u = u0[c], x = x0[c];
        const float u_plus = u + ((u * -1.0f + 1.0f) * uu) * ev;
        const float e = u_plus * x;
        const float eff = e / uu;
        const float x_used = x - e * ev;
        u1[c] = u_plus * df;
        x1[c] = ((x_used * -1.0f + 1.0f) * dd) * -1.0f + 1.0f;
        out[c] = sv + ((sv * eff) - sv) * mix[c];
        if (eff_out) eff_out[c] = eff;
    }
}

// fstep/arch.rs:525-1073 for R rows at once (one token each; the rows are independent, state.rs:13-15).  The int8
// products take the R rows as one batch, as the reference's batched path does (each row's outputs are the bits of the
// row alone, int8.rs:7-8); everything else runs row by row.  Returns 0, or 1 when the reference's fused step would
// refuse a token (non-finite gates or keys): such a row is left uncommitted.
// fstep/arch_f3.rs:207-283 on one row: xf [d] plus the read-out of the sparse code of [xf, rmsnorm(emb, 1)]
void cb_correct(const orc_model* m, const float* emb, float* xf) {
    const int d = m->cfg.d, g = m->cfg.cb_units, k = g / 32;
    std::vector<float> u(xf, xf + d), ones(d, 1.0f), en(d), h(g), a(g);
    rmsnorm(emb, ones.data(), d, en.data());
    u.insert(u.end(), en.begin(), en.end());
    for (int j = 0; j < g; ++j) {
        float s = 0.f;
        for (int q = 0; q < 4; ++q) s += u[m->cb_idx[(size_t)j * 4 + q]] * m->cb_sgn[(size_t)j * 4 + q];
        h[j] = s;
    }
    kwta(h.data(), g, k, false, a.data());
    float s2 = 0.f;
    for (int j = 0; j < g; ++j) s2 += a[j] * a[j];
    const float len = std::sqrt(s2) * 1.0f + (float)1e-6;
    std::vector<std::pair<int, float>> act;
    for (int j = 0; j < g; ++j) {
        const float c = a[j] / len;
        if (c != 0.0f) act.emplace_back(j, c);
    }
    if (act.empty()) act.emplace_back(0, 0.0f);
    std::vector<float> corr(d, 0.f);
    for (const auto& e : act)
        for (int c = 0; c < d; ++c) corr[c] += m->cb_w[(size_t)e.first * d + c] * e.second;
    for (int c = 0; c < d; ++c) xf[c] = xf[c] + corr[c];
}

int step_rows(const orc_model* m, RowState** rows, int R, const uint32_t* tok, float* logits, size_t logit_stride, bool trace) {
    const orc_config& cfg = m->cfg;
    const int d = cfg.d, hs = cfg.head_size, nh = m->nh(), H = cfg.hidden, L = cfg.n_blocks;
    for (int r = 0; r < R; ++r)
        if (tok[r] >= (uint32_t)cfg.vocab) return -2;
    const bool mom = cfg.mem_momentum > 0.0f;
    const float mf = cfg.mem_momentum;
    auto T = [&](const char* n, int blk, const float* p, size_t len) { if (trace) g_trace.put(n, blk, p, len); };
    const int nt = std::max(1, std::min(g_threads, R));
    (void)nt;

    std::vector<float> x((size_t)R * d), h((size_t)R * d), tmp((size_t)R * d);
    for (int r = 0; r < R; ++r) std::copy(m->tok_emb.begin() + (size_t)tok[r] * d, m->tok_emb.begin() + (size_t)(tok[r] + 1) * d, x.begin() + (size_t)r * d);
    T("x_in", -1, x.data(), d);
    if (cfg.letters) {
        // R (fstep/arch_f2.rs:34-60): l = (0 + m_0 tanh((E[b_0] + Q[e_0]) + P[0]) + ...) inv, then l Wo in the one-row order
        const int DL = 64, LM = 16;
        for (int r = 0; r < R; ++r) {
            const size_t t = tok[r];
            std::vector<float> l(DL, 0.f), o(d);
            for (int j = 0; j < LM; ++j) {
                const uint32_t bb = m->let_ids[t * LM + j], kk = m->let_eidx[t * LM + j];
                for (int c = 0; c < DL; ++c) {
                    const float s = tanh_f((m->let_byte[(size_t)bb * DL + c] + m->let_end[(size_t)kk * DL + c]) + m->let_pos[(size_t)j * DL + c]);
                    l[c] += s * m->let_mask[t * LM + j];
                }
            }
            for (int c = 0; c < DL; ++c) l[c] *= m->let_inv[t];
            gemv(l.data(), DL, m->let_wo.data(), d, o.data());
            add_into(&x[(size_t)r * d], o.data(), d);
        }
        T("x_let", -1, x.data(), d);
    }
    // Y (fstep/arch_f4.rs:47-92): before the blocks, from the input after the letters: the clocks' times and phase features
    std::vector<float> rh_f, rh_a;  // [R][4] cos, sin of each phase; [R][2] the new times
    if (cfg.rhythm) {
        rh_f.resize((size_t)R * 4);
        rh_a.resize((size_t)R * 2);
        for (int r = 0; r < R; ++r) {
            std::vector<float> hn(x.begin() + (size_t)r * d, x.begin() + (size_t)(r + 1) * d);
            head_norm(hn.data(), d, d);
            float pre[2];
            gemv(hn.data(), d, m->rhy_wr.data(), 2, pre);
            for (int o = 0; o < 2; ++o) {
                pre[o] = pre[o] + m->rhy_br[o];
                const float l = log_sigmoid(-pre[o]);  // ln(1 - r)
                const float big = l * 1.0f, before = big - l, diff = big - before;
                const float w = g_exp(diff > 0.0f ? 0.0f : diff) * 1.0f;
                const float a = w + g_exp(big) * rows[r]->rh[o];
                rh_a[(size_t)r * 2 + o] = a;
                const float ph = a * g_exp(m->rhy_lw[o]);
                rh_f[(size_t)r * 4 + 2 * o] = g_cos(ph);
                rh_f[(size_t)r * 4 + 2 * o + 1] = g_sin(ph);
            }
        }
        T("rh_f", -1, rh_f.data(), 4);
    }
    std::vector<std::vector<float>> streams;
    if (cfg.dense) streams.push_back(x);
    std::vector<float> v_first;
    bool have_v_first = false;

    std::vector<RowState> nw(R);  // the new states, committed at the end
    for (RowState& n : nw) {
        n.v.resize(L); n.s.resize(L); n.a.resize(L); n.f.resize(L); n.ms.resize(L); n.su.resize(L); n.sx.resize(L);
    }
    std::vector<char> bad(R, 0);
    bool eng_written = false;

    std::vector<float> ctx;  // P: the block's memory read [R, d]
    // --neuromod (fstep/arch.rs:616,1029,1108-1119; src/v50.rs:20-29): three signals per row after block 0, for the later blocks
    const int NM_NE = 0, NM_ACH = 1, NM_DA = 2, nk = cfg.neuromod;
    std::vector<float> sig;  // [R][nk], empty in block 0
    // --dopamine / --mood (fstep/arch_f3.rs:106-186): after block 0 the surprise at this token, CE(head(prev), tok) * valid
    // with prev block 0's normed output of the token before; z = s / ln V; the mood's one-step scan
    const bool surprise = cfg.dopamine || cfg.mood > 0;
    bool have_surprise = false;
    std::vector<float> sur_prev, sur_s, sur_z, mood_now;
    // --thalamus (fstep/arch_f2.rs:62-153; src/v51b.rs:312-325): the relay's running sum of reads rmsnorm(x) R_j [R][16],
    // each block's two gates 2 sigmoid(tanh(acc / sqrt(reads)) G_i + c_i): [0] the residual's, [1] the memory read's
    const int TK = 16;
    std::vector<float> th_acc, th_g, x_in;
    int th_reads = 0;
    const std::vector<float> th_ones(cfg.thalamus ? d : 0, 1.0f);
    auto relay_read = [&](int j) {
        if (th_acc.empty()) th_acc.assign((size_t)R * TK, 0.f);
        for (int r = 0; r < R; ++r) {
            std::vector<float> xn(d), z(TK);
            rmsnorm(&x[(size_t)r * d], th_ones.data(), d, xn.data());
            gemv(xn.data(), d, &m->th_read[(size_t)j * d * TK], TK, z.data());
            for (int k = 0; k < TK; ++k) th_acc[(size_t)r * TK + k] = j == 0 ? z[k] : th_acc[(size_t)r * TK + k] + z[k];
        }
        ++th_reads;
    };
    if (cfg.thalamus) relay_read(0);
    for (int i = 0; i < L; ++i) {
        const Block& b = m->blocks[i];
        if (cfg.thalamus) {
            x_in = x;
            th_g.assign((size_t)R * 2, 1.0f);
            const float mulf = (float)(1.0 / std::sqrt((double)th_reads));
            for (int r = 0; r < R; ++r) {
                float f[TK], z[2];
                for (int k = 0; k < TK; ++k) f[k] = tanh_f(th_acc[(size_t)r * TK + k] * mulf + 0.0f);
                gemv(f, TK, &m->th_gate[(size_t)i * TK * 2], 2, z);
                for (int c = 0; c < 2; ++c) th_g[(size_t)r * 2 + c] = sigmoid(z[c] + m->th_bias[(size_t)i * 2 + c]) * 2.0f + 0.0f;
            }
            T("th_g", i, th_g.data(), 2);
        }
        // ---- the spiking memory (fstep/arch.rs:636-677)
#pragma omp parallel for num_threads(nt) schedule(static)
        for (int r = 0; r < R; ++r) rmsnorm(&x[(size_t)r * d], b.mem_norm.data(), d, &h[(size_t)r * d]);
        T("h_lif", i, h.data(), d);
        std::vector<float> cur((size_t)R * d), sp((size_t)R * d);
        q8_matmul(b.win, h.data(), R, cur.data());
#pragma omp parallel for num_threads(nt) schedule(static)
        for (int r = 0; r < R; ++r) {
            float* c_ = &cur[(size_t)r * d];
            if (cfg.lif_scale)
                for (int c = 0; c < d; ++c) c_[c] = c_[c] * (b.beta[c] * -1.0f + 1.0f);
            if (!sig.empty())  // NE: the input current times its signal, after --lif-scale
                for (int c = 0; c < d; ++c) c_[c] = c_[c] * sig[(size_t)r * nk + NM_NE];
            if (have_surprise && cfg.mood > 0 && i > 0) {  // M: the current times tanh(mood G)·1 + 1, after NE (fstep/arch_f3.rs:176-186)
                std::vector<float> z(d);
                gemv(&mood_now[(size_t)r * cfg.mood], cfg.mood, b.mood_g.data(), d, z.data());
                for (int c = 0; c < d; ++c) c_[c] = c_[c] * (tanh_f(z[c]) * 1.0f + 1.0f);
            }
            RowState& st = *rows[r];
            nw[r].v[i].resize(d);
            nw[r].a[i].resize(cfg.alif ? d : 0);
            lif(c_, b.beta.data(), cfg.theta ? b.theta.data() : nullptr, cfg.alif ? b.rho.data() : nullptr, cfg.alif ? b.again.data() : nullptr,
                cfg.spikes, cfg.slope, st.v[i].data(), st.s[i].data(), cfg.alif ? st.a[i].data() : nullptr, d, &sp[(size_t)r * d],
                nw[r].v[i].data(), cfg.alif ? nw[r].a[i].data() : nullptr);
            nw[r].s[i].assign(&sp[(size_t)r * d], &sp[(size_t)r * d] + d);
        }
        T("cur", i, cur.data(), d);
        T("spikes", i, sp.data(), d);
        if (cfg.stp) {
            // the LIF keeps its spikes; what reaches W_out went through the synapse
            for (int r = 0; r < R; ++r) {
                nw[r].su[i].resize(d);
                nw[r].sx[i].resize(d);
                stp_step(&sp[(size_t)r * d], b.stp_U.data(), b.stp_F.data(), b.stp_D.data(), b.stp_mix.data(), rows[r]->su[i].data(),
                         rows[r]->sx[i].data(), d, &sp[(size_t)r * d], nw[r].su[i].data(), nw[r].sx[i].data(), nullptr);
            }
            T("stp_out", i, sp.data(), d);
        }
        q8_matmul(b.wout, sp.data(), R, tmp.data());
        add_into(x.data(), tmp.data(), R * d);
        T("x_lif", i, x.data(), d);

        // ---- the fast-weight memory (fstep/arch.rs:679-907); a kind-S block has none (fstep.rs:536-548, then :673)
        if (cfg.fast_mem) {
#pragma omp parallel for num_threads(nt) schedule(static)
        for (int r = 0; r < R; ++r) rmsnorm(&x[(size_t)r * d], b.hebb_norm.data(), d, &h[(size_t)r * d]);
        T("h_mem", i, h.data(), d);
        std::vector<float> q((size_t)R * d), kraw((size_t)R * d), v((size_t)R * d), weo((size_t)R * d), gq(cfg.out_gate ? (size_t)R * d : 0);
        q8_matmul(b.wq, h.data(), R, q.data());
        q8_matmul(b.wk, h.data(), R, kraw.data());
        q8_matmul(b.wv, h.data(), R, v.data());
        q8_matmul(b.we, h.data(), R, weo.data());
        if (cfg.out_gate) q8_matmul(b.wg, h.data(), R, gq.data());
        if (trace) {
            std::vector<float> all;
            for (auto* p : {&q, &kraw, &v, &weo, &gq})
                if (!p->empty()) all.insert(all.end(), p->begin(), p->begin() + d);
            T("qkveg", i, all.data(), all.size());
        }
        if (cfg.value_residual && !have_v_first) {
            v_first = v;  // block 0's values, before any mixing (fstep/arch.rs:695)
            have_v_first = true;
        }
        const bool mix_v = cfg.value_residual && i > 0 && !b.vres.empty();
        std::vector<float> y((size_t)R * d);
        struct Tr { std::vector<float> k, ek, w, ah, qg, ex, yraw, qw, qa, be; } tr;
#pragma omp parallel for num_threads(nt) schedule(static)
        for (int r = 0; r < R; ++r) {
            float* qr = &q[(size_t)r * d];
            float* vr = &v[(size_t)r * d];
            const float* hr = &h[(size_t)r * d];
            const float* kr = &kraw[(size_t)r * d];
            l2_heads(qr, d, hs);
            std::vector<float> k(kr, kr + d);
            l2_heads(k.data(), d, hs);
            if (mix_v) {
                const float p0 = b.vres[0] * 1.0f + 1.0f;
                const float* vf = &v_first[(size_t)r * d];
                for (int c = 0; c < d; ++c) vr[c] = vr[c] * p0 + vf[c] * b.vres[1];
            }
            const int rk = cfg.gate_rank;
            std::vector<float> za(nh), zb(nh), z1(rk), lra(d), lrb(d);
            gemv(hr, d, b.wa.data(), nh, za.data());
            gemv(hr, d, b.wb.data(), nh, zb.data());
            add_into(za.data(), b.ba.data(), nh);
            add_into(zb.data(), b.bb.data(), nh);
            gemv(hr, d, b.wa1.data(), rk, z1.data());
            gemv(z1.data(), rk, b.wa2.data(), d, lra.data());
            gemv(hr, d, b.wb1.data(), rk, z1.data());
            gemv(z1.data(), rk, b.wb2.data(), d, lrb.data());

            // Y: this block's gains per head from the token's phase features, 1 + tanh(f G) (fstep/arch_f4.rs:94-107)
            std::vector<float> rgw, rgr;
            if (cfg.rhythm) {
                rgw.resize(nh); rgr.resize(nh);
                gemv(&rh_f[(size_t)r * 4], 4, b.rh_w.data(), nh, rgw.data());
                gemv(&rh_f[(size_t)r * 4], 4, b.rh_r.data(), nh, rgr.data());
                for (int e = 0; e < nh; ++e) {
                    rgw[e] = tanh_f(rgw[e]) * 1.0f + 1.0f;
                    rgr[e] = tanh_f(rgr[e]) * 1.0f + 1.0f;
                }
            }
            RowState& st = *rows[r];
            std::vector<float> fnew((size_t)nh * hs * hs), snew(mom ? (size_t)nh * hs * hs : 0);
            std::vector<float> ek(d), ex(d), w(d), ah(d), qg(d), yraw(d), qwv(nh), qav(nh);
            float* yr = &y[(size_t)r * d];
            bool bad_row = false;
            for (int e = 0; e < nh && !bad_row; ++e) {
                const int o = e * hs;
                std::vector<float> la(hs), be(hs), qs, p2, e0(hs);
                if (trace && r == 0 && e == 0) tr.be.assign(d, 0.f);
                for (int c = 0; c < hs; ++c) {
                    la[c] = log_sigmoid((za[e] + b.off[o + c]) + lra[o + c]);
                    be[c] = sigmoid(zb[e] + lrb[o + c]) * 2.0f + 0.0f;
                    if (cfg.rhythm) be[c] = be[c] * rgw[e];  // Y: before ACh's clamp
                    if (!sig.empty()) {  // ACh: the write strength times its signal, kept in [0, 2] (maximum, then minimum)
                        float v = be[c] * sig[(size_t)r * nk + NM_ACH];
                        v = v < 0.0f ? 0.0f : v;
                        be[c] = v > 2.0f ? 2.0f : v;
                    }
                }
                if (trace && r == 0) std::copy(be.begin(), be.end(), tr.be.begin() + o);
                for (int c = 0; c < hs; ++c) ek[o + c] = kr[o + c] + weo[(size_t)r * d + o + c];
                l2_heads(ek.data() + o, hs, hs);
                for (int c = 0; c < hs; ++c) {
                    ex[o + c] = g_exp(la[c]);
                    w[o + c] = k[o + c] * be[c];
                    ah[o + c] = ek[o + c] * (be[c] * ex[o + c]);
                    qg[o + c] = qr[o + c] * ex[o + c];
                }
                if (!all_finite(la.data(), hs) || !all_finite(ek.data() + o, hs) || !all_finite(w.data() + o, hs) ||
                    !all_finite(ah.data() + o, hs) || !all_finite(qr + o, hs) || !all_finite(vr + o, hs)) {
                    bad_row = true;
                    break;
                }
                if (mom) {
                    qs.resize(hs);
                    p2.resize(hs);
                    const float gsx = 0.0f * mf + 0.0f;
                    for (int c = 0; c < hs; ++c) {
                        qs[c] = qr[o + c] * (1.0f * mf + 0.0f);
                        p2[c] = ek[o + c] * gsx;
                    }
                }
                auto sum0 = [&](const float* a, const float* c2) {
                    float s = 0.f;
                    for (int c = 0; c < hs; ++c) s += a[c] * c2[c];
                    return s;
                };
                for (int c = 0; c < hs; ++c) e0[c] = ek[o + c] * 0.0f;
                const float qw = sum0(qr + o, w.data() + o), qa = sum0(qr + o, ah.data() + o);
                const float ke = sum0(e0.data(), w.data() + o), ae = sum0(e0.data(), ah.data() + o);
                const float tinv = -(ae * 0.0f) + 1.0f;
                if (tinv != 1.0f) {
                    bad_row = true;
                    break;
                }
                qwv[e] = qw;
                qav[e] = qa;
                head_rows(hs, ek.data() + o, vr + o, w.data() + o, ah.data() + o, qg.data() + o, ex.data() + o, qw, qa, ke, tinv, mom, mf,
                          mom ? qs.data() : nullptr, mom ? p2.data() : nullptr, st.f[i].data() + (size_t)e * hs * hs,
                          mom ? st.ms[i].data() + (size_t)e * hs * hs : nullptr, yr + o, fnew.data() + (size_t)e * hs * hs,
                          mom ? snew.data() + (size_t)e * hs * hs : nullptr);
                std::copy(yr + o, yr + o + hs, yraw.begin() + o);
                head_norm(yr + o, hs, hs);
                if (cfg.rhythm)  // Y: the read's gain, after the head norm and before the output gate
                    for (int c = 0; c < hs; ++c) yr[o + c] = yr[o + c] * rgr[e];
                if (cfg.out_gate)
                    for (int c = 0; c < hs; ++c) {
                        const float g = gq[(size_t)r * d + o + c];
                        yr[o + c] = yr[o + c] * (g / (1.0f + g_exp(-g)));
                    }
            }
            if (bad_row) {
                bad[r] = 1;
                std::fill(yr, yr + d, 0.f);
            }
            nw[r].f[i] = std::move(fnew);
            nw[r].ms[i] = std::move(snew);
            if (trace && r == 0) {
                tr.k = k; tr.ek = ek; tr.w = w; tr.ah = ah; tr.qg = qg; tr.ex = ex; tr.yraw = yraw; tr.qw = qwv; tr.qa = qav;
            }
        }
        if (trace) {
            T("q", i, q.data(), d); T("k", i, tr.k.data(), d); T("v", i, v.data(), d); T("ek", i, tr.ek.data(), d); T("w", i, tr.w.data(), d);
            T("ah", i, tr.ah.data(), d); T("qg", i, tr.qg.data(), d); T("ex", i, tr.ex.data(), d); T("qw", i, tr.qw.data(), nh);
            T("qa", i, tr.qa.data(), nh); T("y_raw", i, tr.yraw.data(), d); T("y", i, y.data(), d); T("be", i, tr.be.data(), d);
        }
        q8_matmul(b.wo, y.data(), R, tmp.data());
        if (cfg.dendrite) ctx.assign(tmp.begin(), tmp.begin() + (size_t)R * d);  // P: the memory's read, the dendrites' context
        if (cfg.thalamus)  // TH: the memory gate (after the dendrites' copy)
            for (int r = 0; r < R; ++r)
                for (int c = 0; c < d; ++c) tmp[(size_t)r * d + c] = tmp[(size_t)r * d + c] * th_g[(size_t)r * 2 + 1];
        add_into(x.data(), tmp.data(), R * d);
        T("x_mem", i, x.data(), d);
        }

        // ---- the engram (fstep/arch.rs:909-974)
        if (i == cfg.eng_block) {
            const int ehs = cfg.eng_head_size, enh = m->enh();
#pragma omp parallel for num_threads(nt) schedule(static)
            for (int r = 0; r < R; ++r) rmsnorm(&x[(size_t)r * d], b.eng_norm.data(), d, &h[(size_t)r * d]);
            T("h_eng", i, h.data(), d);
            std::vector<float> eq((size_t)R * d), ekk((size_t)R * d), evv((size_t)R * d), o((size_t)R * d);
            q8_matmul(b.ewq, h.data(), R, eq.data());
            q8_matmul(b.ewk, h.data(), R, ekk.data());
            q8_matmul(b.ewv, h.data(), R, evv.data());
            if (trace) {
                std::vector<float> all;
                for (auto* p : {&eq, &ekk, &evv}) all.insert(all.end(), p->begin(), p->begin() + d);
                T("eng_qkv", i, all.data(), all.size());
            }
            const float scale = (float)(1.0 / std::sqrt((double)ehs));
#pragma omp parallel for num_threads(nt) schedule(static)
            for (int r = 0; r < R; ++r) {
                float* kk = &ekk[(size_t)r * d];
                float* vv = &evv[(size_t)r * d];
                if (cfg.eng_store_bf16)
                    for (int c = 0; c < d; ++c) {
                        kk[c] = bf16_round(kk[c]);
                        vv[c] = bf16_round(vv[c]);
                    }
                const RowState& st = *rows[r];
                const int n0 = st.eng_n, n = n0 + 1;
                // [enh, n, ehs] with this token's row appended per head (fstep.rs:449-459)
                std::vector<float> kc((size_t)enh * n * ehs), vc((size_t)enh * n * ehs);
                for (int hh = 0; hh < enh; ++hh) {
                    std::copy(st.ek.begin() + (size_t)hh * n0 * ehs, st.ek.begin() + (size_t)(hh + 1) * n0 * ehs, kc.begin() + (size_t)hh * n * ehs);
                    std::copy(st.evv.begin() + (size_t)hh * n0 * ehs, st.evv.begin() + (size_t)(hh + 1) * n0 * ehs, vc.begin() + (size_t)hh * n * ehs);
                    std::copy(kk + hh * ehs, kk + (hh + 1) * ehs, kc.begin() + ((size_t)hh * n + n0) * ehs);
                    std::copy(vv + hh * ehs, vv + (hh + 1) * ehs, vc.begin() + ((size_t)hh * n + n0) * ehs);
                }
                for (int hh = 0; hh < enh; ++hh)
                    attend(&eq[(size_t)r * d + hh * ehs], kc.data() + (size_t)hh * n * ehs, vc.data() + (size_t)hh * n * ehs, n, ehs, scale,
                           &o[(size_t)r * d + hh * ehs]);
                // the oldest-first cap (state.rs:526-538)
                int keep = n;
                if (cfg.eng_cap > 0 && n > cfg.eng_cap) keep = cfg.eng_cap;
                nw[r].ek.resize((size_t)enh * keep * ehs);
                nw[r].evv.resize((size_t)enh * keep * ehs);
                for (int hh = 0; hh < enh; ++hh) {
                    std::copy(kc.begin() + ((size_t)hh * n + (n - keep)) * ehs, kc.begin() + (size_t)(hh + 1) * n * ehs,
                              nw[r].ek.begin() + (size_t)hh * keep * ehs);
                    std::copy(vc.begin() + ((size_t)hh * n + (n - keep)) * ehs, vc.begin() + (size_t)(hh + 1) * n * ehs,
                              nw[r].evv.begin() + (size_t)hh * keep * ehs);
                }
                nw[r].eng_n = keep;
            }
            eng_written = true;
            T("eng_o", i, o.data(), d);
            q8_matmul(b.ewo, o.data(), R, tmp.data());
            T("eng_r", i, tmp.data(), d);
            add_into(x.data(), tmp.data(), R * d);
            T("x_eng", i, x.data(), d);
        }

        // ---- the sparse MLP (fstep/arch.rs:976-999)
#pragma omp parallel for num_threads(nt) schedule(static)
        for (int r = 0; r < R; ++r) rmsnorm(&x[(size_t)r * d], b.mlp_norm.data(), d, &h[(size_t)r * d]);
        T("h_mlp", i, h.data(), d);
        std::vector<float> u((size_t)R * H), a((size_t)R * H);
        q8_matmul(b.w1, h.data(), R, u.data());
        T("u", i, u.data(), H);
#pragma omp parallel for num_threads(nt) schedule(static)
        for (int r = 0; r < R; ++r) kwta(&u[(size_t)r * H], H, cfg.kwta_k, cfg.relu2 != 0, &a[(size_t)r * H]);
        T("a", i, a.data(), H);
        if (cfg.dendrite && cfg.fast_mem) {
            // P (fstep/arch_f4.rs:120-141): the units times 1 + tanh(head_norm(ctx) A B), the two products in gemm's one-row order
            const int rk = 32;
#pragma omp parallel for num_threads(nt) schedule(static)
            for (int r = 0; r < R; ++r) {
                std::vector<float> hn(ctx.begin() + (size_t)r * d, ctx.begin() + (size_t)(r + 1) * d), z1(rk), z(H);
                head_norm(hn.data(), d, d);
                gemv(hn.data(), d, b.dend_a.data(), rk, z1.data());
                gemv(z1.data(), rk, b.dend_b.data(), H, z.data());
                float* ar = &a[(size_t)r * H];
                for (int j = 0; j < H; ++j) ar[j] = ar[j] * (tanh_f(z[j]) * 1.0f + 1.0f);
            }
            T("a_dend", i, a.data(), H);
        }
        q8_matmul(b.w2, a.data(), R, tmp.data());
        if (have_surprise && cfg.dopamine && i > 0)  // DA: the output times tanh(z w + c)·1 + 1, z the surprise / ln V (fstep/arch_f4.rs:131-143)
            for (int r = 0; r < R; ++r)
                for (int c = 0; c < d; ++c)
                    tmp[(size_t)r * d + c] = tmp[(size_t)r * d + c] * (tanh_f(sur_z[r] * b.da_w[c] + b.da_c[c]) * 1.0f + 1.0f);
        if (!sig.empty())  // DA: the MLP's output times its signal
            for (int r = 0; r < R; ++r)
                for (int c = 0; c < d; ++c) tmp[(size_t)r * d + c] = tmp[(size_t)r * d + c] * sig[(size_t)r * nk + NM_DA];
        add_into(x.data(), tmp.data(), R * d);
        if (cfg.thalamus)  // TH: the residual rule x + (x - x_in)(g_res 1 + -1) on the block's whole change
            for (int r = 0; r < R; ++r) {
                const float gm1 = th_g[(size_t)r * 2] * 1.0f + -1.0f;
                for (int c = 0; c < d; ++c) {
                    const size_t at = (size_t)r * d + c;
                    x[at] = x[at] + (x[at] - x_in[at]) * gm1;
                }
            }

        // ---- the dense residual mix (fstep/arch.rs:1014-1024)
        if (cfg.dense) {
            streams.push_back(x);
            std::vector<float> mix = x;
            for (size_t j = 0; j < streams.size(); ++j)
                for (size_t c = 0; c < (size_t)R * d; ++c) mix[c] = mix[c] + streams[j][c] * b.dense[j];
            x = mix;
        }
        T("x_out", i, x.data(), d);
        if (cfg.thalamus && i + 1 < L) relay_read(i + 1);  // the relay reads this block's output for the later gates
        if (i == 0 && surprise) {
            sur_prev.resize((size_t)R * d); sur_s.assign(R, 0.f); sur_z.assign(R, 0.f); mood_now.assign((size_t)R * cfg.mood, 0.f);
            std::vector<float> row(cfg.vocab);
            for (int r = 0; r < R; ++r) {
                rmsnorm(&x[(size_t)r * d], m->final_norm.data(), d, &sur_prev[(size_t)r * d]);
                const RowState& st = *rows[r];
                q8_matmul(m->head, st.prev.data(), 1, row.data());
                float mx = -std::numeric_limits<float>::infinity();
                for (float v : row) mx = std::max(mx, v);
                float se = 0.f;
                for (float v : row) se += g_exp(v - mx);
                const float lse = mx + g_log(se);
                sur_s[r] = (lse - row[tok[r]]) * st.pvalid[0];
                sur_z[r] = sur_s[r] * (float)(1.0 / std::log((double)cfg.vocab)) + 0.0f;
                for (int j = 0; j < cfg.mood; ++j) {
                    const float u = sur_z[r] * m->mood_win[j] + m->mood_bin[j];
                    const float ll = log_sigmoid(m->mood_lam[j]), oml = sigmoid(-m->mood_lam[j]);
                    const float p = g_exp(0.0f * ll) * 1.0f;
                    mood_now[(size_t)r * cfg.mood + j] = p * (u * oml) + st.mood[j] * g_exp(1.0f * ll);
                }
            }
            have_surprise = true;
            T("sur_z", 0, sur_z.data(), 1);
            if (cfg.mood > 0) T("mood", 0, mood_now.data(), cfg.mood);
        }
        if (i == 0 && nk > 0) {
            // the nucleus reads block 0's output: 2 sigmoid(rmsnorm(x, g) W + b)
            sig.assign((size_t)R * nk, 0.f);
            for (int r = 0; r < R; ++r) {
                std::vector<float> hn(d), z(nk);
                rmsnorm(&x[(size_t)r * d], m->nm_norm.data(), d, hn.data());
                gemv(hn.data(), d, m->nm_wn.data(), nk, z.data());
                for (int k = 0; k < nk; ++k) sig[(size_t)r * nk + k] = sigmoid(z[k] + m->nm_bn[k]) * 2.0f + 0.0f;
            }
            T("nm_sig", 0, sig.data(), nk);
        }
    }
#pragma omp parallel for num_threads(nt) schedule(static)
    for (int r = 0; r < R; ++r) rmsnorm(&x[(size_t)r * d], m->final_norm.data(), d, &h[(size_t)r * d]);
    T("x_final", -1, h.data(), d);
    if (cfg.cb_units > 0) {  // CB: the cerebellum's correction of the final normed state, from it and the token's embedding
        for (int r = 0; r < R; ++r) cb_correct(m, &m->tok_emb[(size_t)tok[r] * d], &h[(size_t)r * d]);
        T("x_cb", -1, h.data(), d);
    }
    if (logit_stride == (size_t)cfg.vocab) {
        q8_matmul(m->head, h.data(), R, logits);
    } else {
        std::vector<float> lg((size_t)R * cfg.vocab);
        q8_matmul(m->head, h.data(), R, lg.data());
        for (int r = 0; r < R; ++r) std::copy(lg.begin() + (size_t)r * cfg.vocab, lg.begin() + (size_t)(r + 1) * cfg.vocab, logits + r * logit_stride);
    }

    // everything computed: the states move on (fstep/arch.rs:1059-1069); a refused row keeps its state
    int rc = 0;
    for (int r = 0; r < R; ++r) {
        if (bad[r]) {
            rc = 1;
            continue;
        }
        RowState& st = *rows[r];
        st.v = std::move(nw[r].v); st.s = std::move(nw[r].s); st.a = std::move(nw[r].a);
        st.f = std::move(nw[r].f); st.ms = std::move(nw[r].ms);
        if (cfg.stp) {
            st.su = std::move(nw[r].su);
            st.sx = std::move(nw[r].sx);
        }
        if (cfg.rhythm) st.rh.assign(rh_a.begin() + (size_t)r * 2, rh_a.begin() + (size_t)(r + 1) * 2);
        if (surprise) {  // fstep/arch_f3.rs:324-336
            st.prev.assign(sur_prev.begin() + (size_t)r * d, sur_prev.begin() + (size_t)(r + 1) * d);
            st.pvalid[0] = 1.0f;
            st.last_s[0] = sur_s[r];
            if (cfg.mood > 0) st.mood.assign(mood_now.begin() + (size_t)r * cfg.mood, mood_now.begin() + (size_t)(r + 1) * cfg.mood);
        }
        if (eng_written) {
            st.ek = std::move(nw[r].ek);
            st.evv = std::move(nw[r].evv);
            st.eng_n = nw[r].eng_n;
        }
        st.seen += 1;
    }
    return rc;
}

bool parse_state_name(const orc_state* s, int row, const std::string& name, const std::vector<float>** out) {
    const RowState& r = s->rows[row];
    if (name == "eng.k") { *out = &r.ek; return true; }
    if (name == "eng.v") { *out = &r.evv; return true; }
    if (name == "v51.prev") { *out = &r.prev; return true; }
    if (name == "v51.mood") { *out = &r.mood; return true; }
    if (name == "v51.rh") { *out = &r.rh; return true; }
    if (name == "v51.pvalid") { *out = &r.pvalid; return true; }
    if (name == "v51.last_s") { *out = &r.last_s; return true; }
    const size_t d1 = name.find('.'), d2 = name.rfind('.');
    if (d1 == std::string::npos || d2 == d1) return false;
    const std::string kind = name.substr(0, d1), what = name.substr(d2 + 1);
    const int i = std::atoi(name.substr(d1 + 1, d2 - d1 - 1).c_str());
    if (i < 0 || i >= s->m->cfg.n_blocks) return false;
    if (kind == "lif") {
        if (what == "v") { *out = &r.v[i]; return true; }
        if (what == "s") { *out = &r.s[i]; return true; }
        if (what == "a") { *out = &r.a[i]; return true; }
    } else if (kind == "parts" && s->m->cfg.stp) {
        if (what == "stp_u") { *out = &r.su[i]; return true; }
        if (what == "stp_x") { *out = &r.sx[i]; return true; }
    } else if (kind == "mem" && s->m->cfg.fast_mem) {
        if (what == "f") { *out = &r.f[i]; return true; }
        if (what == "s") { *out = &r.ms[i]; return true; }
    }
    return false;
}

}  // namespace

// ================================================================================================ C API
extern "C" {

void orc_set_math(orc_fn1 e, orc_fn1 l, orc_fn1 r) {
    if (e) g_exp = e;
    if (l) g_log = l;
    if (r) g_rsqrt = r;
}
void orc_reset_math(void) { g_exp = libm_exp; g_log = libm_log; g_rsqrt = libm_rsqrt; g_sin = libm_sin; g_cos = libm_cos; }
void orc_set_trig(orc_fn1 s, orc_fn1 c) {
    if (s) g_sin = s;
    if (c) g_cos = c;
}
void orc_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
void orc_set_simd(int on) { g_simd = on; }
void orc_set_event_max(double v) { g_event_max = v; }

void orc_quantize_int8(const float* w, int rows, int cols, int8_t* q, float* scale) { quantize_int8(w, rows, cols, q, scale); }

void orc_q8_matmul(const float* x, int m, const int8_t* q, const float* scale, int din, int dout, float* y) {
    QW w;
    w.from_q(q, scale, din, dout);
    q8_matmul(w, x, m, y);
}
int orc_last_event_rows(void) { return g_last_event_rows; }
void orc_rmsnorm(const float* x, const float* gain, int n, float* y) { rmsnorm(x, gain, n, y); }
void orc_l2_heads(float* x, int n, int hs) { l2_heads(x, n, hs); }
void orc_head_norm(float* y, int n, int hs) { head_norm(y, n, hs); }
float orc_sigmoid(float x) { return sigmoid(x); }
float orc_log_sigmoid(float x) { return log_sigmoid(x); }
void orc_gemv(const float* x, int k, const float* w, int n, float* out) { gemv(x, k, w, n, out); }
void orc_lif(const float* cur, const float* beta, const float* theta, const float* rho, const float* gain, int spikes, float slope,
             const float* v0, const float* s0, const float* a0, int d, float* s1, float* v1, float* a1) {
    lif(cur, beta, theta, rho, gain, spikes, slope, v0, s0, a0, d, s1, v1, a1);
}
void orc_stp(const float* s, const float* u_param, const float* f_param, const float* d_param, const float* mix, const float* u0, const float* x0,
             int d, float* out, float* u1, float* x1, float* eff) {
    std::vector<float> U(d), F(d), D(d);
    for (int c = 0; c < d; ++c) {
        U[c] = sigmoid(u_param[c]);
        F[c] = sigmoid(f_param[c]);
        D[c] = sigmoid(d_param[c]);
    }
    stp_step(s, U.data(), F.data(), D.data(), mix, u0, x0, d, out, u1, x1, eff);
}
int orc_model_set_token_bytes(orc_model* m, const uint8_t* bytes, const int64_t* offsets) {
    // src/v51.rs:455-469
    const int V = m->cfg.vocab, LM = 16;
    m->let_ids.assign((size_t)V * LM, 0);
    m->let_eidx.assign((size_t)V * LM, 0);
    m->let_mask.assign((size_t)V * LM, 0.f);
    m->let_inv.assign(V, 0.f);
    for (int t = 0; t < V; ++t) {
        const int64_t len = offsets[t + 1] - offsets[t];
        if (len < 0) return -1;
        const int used = (int)std::min<int64_t>(len, LM);
        for (int j = 0; j < used; ++j) {
            m->let_ids[(size_t)t * LM + j] = bytes[offsets[t] + j];
            m->let_eidx[(size_t)t * LM + j] = (uint32_t)std::min<int64_t>(len - 1 - j, LM - 1);
            m->let_mask[(size_t)t * LM + j] = 1.0f;
        }
        if (used > 0) m->let_inv[t] = 1.0f / std::sqrt((float)used);
    }
    return 0;
}
void orc_cb_wiring(int inputs, int g, uint32_t* idx, float* w) {
    std::vector<uint32_t> i;
    std::vector<float> s;
    cb_wiring(inputs, g, 4, 0x51B0CE7Eull, &i, &s);
    std::copy(i.begin(), i.end(), idx);
    std::copy(s.begin(), s.end(), w);
}
float orc_kth_largest(const float* u, int n, int k) { return kth_largest(u, n, k); }
void orc_kwta(const float* u, int n, int k, int relu2, float* a) { kwta(u, n, k, relu2 != 0, a); }
void orc_attend(const float* q, const float* kc, const float* vc, int n, int hs, float scale, float* out) { attend(q, kc, vc, n, hs, scale, out); }
void orc_head_rows(int hs, const float* e, const float* v, const float* w, const float* ah, const float* qg, const float* ex, float qw, float qa,
                   float ke, float tinv, float mom, const float* qs, const float* p2, const float* f0, const float* s0, float* y, float* f1,
                   float* s1) {
    head_rows(hs, e, v, w, ah, qg, ex, qw, qa, ke, tinv, mom > 0.0f, mom, qs, p2, f0, s0, y, f1, s1);
}
void orc_delta_plain(int hs, const float* f0, const float* k, const float* v, const float* q, float al, float b, float* f1, float* y) {
    delta_plain(hs, f0, k, v, q, al, b, f1, y);
}
float orc_bf16_round(float x) { return bf16_round(x); }

orc_model* orc_model_new(const orc_config* cfg) {
    if (!cfg || cfg->d <= 0 || cfg->head_size <= 0 || cfg->d % cfg->head_size != 0) return nullptr;
    if (cfg->eng_block >= 0 && (cfg->eng_head_size <= 0 || cfg->d % cfg->eng_head_size != 0)) return nullptr;
    orc_model* m = new orc_model();
    m->cfg = *cfg;
    m->blocks.resize(cfg->n_blocks);
    if (cfg->cb_units > 0) cb_wiring(2 * cfg->d, cfg->cb_units, 4, 0x51B0CE7Eull, &m->cb_idx, &m->cb_sgn);  // src/v51b.rs:47-49,292
    return m;
}
void orc_model_free(orc_model* m) { delete m; }

int orc_model_set_f32(orc_model* m, const char* name, const float* data, int64_t n) {
    int64_t want = 0;
    std::vector<float>* slot = f32_slot(m, name, &want);
    if (!slot || want != n) return -1;
    slot->assign(data, data + n);
    return 0;
}
int orc_model_set_q8(orc_model* m, const char* name, const int8_t* q, const float* scale, int din, int dout) {
    int wi = 0, wo = 0;
    QW* slot = q8_slot(m, name, &wi, &wo);
    if (!slot || wi != din || wo != dout) return -1;
    slot->from_q(q, scale, din, dout);
    return 0;
}
int orc_model_set_q8_from_f32(orc_model* m, const char* name, const float* w, int din, int dout) {
    std::vector<int8_t> q((size_t)din * dout);
    std::vector<float> sc(dout);
    quantize_int8(w, din, dout, q.data(), sc.data());
    return orc_model_set_q8(m, name, q.data(), sc.data(), din, dout);
}
int orc_model_check(orc_model* m, char* missing, int cap) {
    const orc_config& c = m->cfg;
    auto fail = [&](const std::string& n) {
        if (missing && cap > 0) std::snprintf(missing, cap, "%s", n.c_str());
        return -1;
    };
    if (m->tok_emb.empty()) return fail("tok_emb");
    if (m->final_norm.empty()) return fail("final.norm");
    if (c.neuromod > 0 && (m->nm_norm.empty() || m->nm_wn.empty() || m->nm_bn.empty())) return fail("nm.norm / nm.wn / nm.bn");
    if (c.rhythm && (m->rhy_lw.empty() || m->rhy_wr.empty() || m->rhy_br.empty())) return fail("v51.rhythm.lw / wr / br");
    if (c.mood > 0 && (m->mood_lam.empty() || m->mood_win.empty() || m->mood_bin.empty())) return fail("v51.mood.lam / win / bin");
    if (c.cb_units > 0 && m->cb_w.empty()) return fail("cbh.wo");
    if (c.letters && (m->let_byte.empty() || m->let_pos.empty() || m->let_end.empty() || m->let_wo.empty())) return fail("v51.letters.byte / pos / end / wo");
    if (c.letters && m->let_ids.empty()) return fail("the tokens' spellings (orc_model_set_token_bytes)");
    if (c.thalamus && (m->th_read.empty() || m->th_gate.empty() || m->th_bias.empty())) return fail("th.read / th.gate / th.bias");
    if (!m->head.ok()) return fail("head");
    for (int i = 0; i < c.n_blocks; ++i) {
        const Block& b = m->blocks[i];
        const std::string p = "b" + std::to_string(i) + ".";
        struct F { const char* n; const std::vector<float>* v; bool need; };
        const F fs[] = {{"mem.norm", &b.mem_norm, true}, {"mem.beta", &b.beta_param, true}, {"mem.theta", &b.theta, c.theta != 0},
                        {"mem.arho", &b.arho, c.alif != 0}, {"mem.again", &b.again, c.alif != 0}, {"hebb.norm", &b.hebb_norm, c.fast_mem != 0},
                        {"hebb.wa", &b.wa, c.fast_mem != 0}, {"hebb.wb", &b.wb, c.fast_mem != 0}, {"hebb.ba", &b.ba, c.fast_mem != 0}, {"hebb.bb", &b.bb, c.fast_mem != 0},
                        {"hebb.wa1", &b.wa1, c.fast_mem != 0}, {"hebb.wa2", &b.wa2, c.fast_mem != 0}, {"hebb.wb1", &b.wb1, c.fast_mem != 0}, {"hebb.wb2", &b.wb2, c.fast_mem != 0},
                        {"hebb.off", &b.off, c.fast_mem != 0}, {"hebb.vres", &b.vres, c.fast_mem && c.value_residual && i > 0}, {"eng.norm", &b.eng_norm, i == c.eng_block},
                        {"mlp.norm", &b.mlp_norm, true}, {"dense", &b.dense, c.dense != 0},
                        {"parts.stp.u_param", &b.stp_u, c.stp != 0}, {"parts.stp.f_param", &b.stp_f, c.stp != 0},
                        {"parts.stp.d_param", &b.stp_d, c.stp != 0}, {"parts.stp.mix", &b.stp_mix, c.stp != 0},
                        {"v51.dend_a", &b.dend_a, c.dendrite && c.fast_mem}, {"v51.dend_b", &b.dend_b, c.dendrite && c.fast_mem},
                        {"v51.rh_w", &b.rh_w, c.rhythm && c.fast_mem}, {"v51.rh_r", &b.rh_r, c.rhythm && c.fast_mem},
                        {"v51.da_w", &b.da_w, c.dopamine && i > 0}, {"v51.da_c", &b.da_c, c.dopamine && i > 0},
                        {"v51.mood_g", &b.mood_g, c.mood > 0 && i > 0}};
        for (const F& f : fs)
            if (f.need && f.v->empty()) return fail(p + f.n);
        struct Q { const char* n; const QW* q; bool need; };
        const Q qs[] = {{"mem.win", &b.win, true}, {"mem.wout", &b.wout, true}, {"hebb.wq", &b.wq, c.fast_mem != 0}, {"hebb.wk", &b.wk, c.fast_mem != 0},
                        {"hebb.wv", &b.wv, c.fast_mem != 0}, {"hebb.we", &b.we, c.fast_mem != 0}, {"hebb.wg", &b.wg, c.fast_mem && c.out_gate}, {"hebb.wo", &b.wo, c.fast_mem != 0},
                        {"eng.wq", &b.ewq, i == c.eng_block}, {"eng.wk", &b.ewk, i == c.eng_block}, {"eng.wv", &b.ewv, i == c.eng_block},
                        {"eng.wo", &b.ewo, i == c.eng_block}, {"mlp.w1", &b.w1, true}, {"mlp.w2", &b.w2, true}};
        for (const Q& q : qs)
            if (q.need && !q.q->ok()) return fail(p + q.n);
    }
    derive(m);
    return 0;
}

orc_state* orc_state_new(const orc_model* m, int rows) {
    orc_state* s = new orc_state();
    s->m = m;
    s->rows.resize(rows);
    const orc_config& c = m->cfg;
    const size_t fl = c.fast_mem ? (size_t)m->nh() * c.head_size * c.head_size : 0;
    for (RowState& r : s->rows) {
        r.v.assign(c.n_blocks, std::vector<float>(c.d, 0.f));
        r.s.assign(c.n_blocks, std::vector<float>(c.d, 0.f));
        r.a.assign(c.n_blocks, std::vector<float>(c.alif ? c.d : 0, 0.f));
        r.f.assign(c.n_blocks, std::vector<float>(fl, 0.f));
        r.ms.assign(c.n_blocks, std::vector<float>(c.mem_momentum > 0.f ? fl : 0, 0.f));
        r.su.assign(c.n_blocks, std::vector<float>(c.stp ? c.d : 0, 0.f));  // u = 0, x = 1 (nn/parts/src/stp.rs:69-70)
        r.sx.assign(c.n_blocks, std::vector<float>(c.stp ? c.d : 0, 1.f));
        r.prev.assign((c.dopamine || c.mood > 0) ? c.d : 0, 0.f);  // src/v51.rs:1029-1036
        r.mood.assign(c.mood, 0.f);
        r.rh.assign(c.rhythm ? 2 : 0, 0.f);
        r.pvalid.assign((c.dopamine || c.mood > 0) ? 1 : 0, 0.f);
        r.last_s.assign((c.dopamine || c.mood > 0) ? 1 : 0, 0.f);
    }
    return s;
}
void orc_state_free(orc_state* s) { delete s; }
int orc_state_rows(const orc_state* s) { return (int)s->rows.size(); }
orc_state* orc_state_select(const orc_state* s, const int32_t* idx, int n) {
    orc_state* o = new orc_state();
    o->m = s->m;
    for (int i = 0; i < n; ++i) {
        if (idx[i] < 0 || idx[i] >= (int)s->rows.size()) {
            delete o;
            return nullptr;
        }
        o->rows.push_back(s->rows[idx[i]]);
    }
    return o;
}
int64_t orc_state_len(const orc_state* s, int row, const char* name) {
    const std::vector<float>* v = nullptr;
    if (row < 0 || row >= (int)s->rows.size() || !parse_state_name(s, row, name, &v)) return -1;
    return (int64_t)v->size();
}
int orc_state_get(const orc_state* s, int row, const char* name, float* out) {
    const std::vector<float>* v = nullptr;
    if (row < 0 || row >= (int)s->rows.size() || !parse_state_name(s, row, name, &v)) return -1;
    std::copy(v->begin(), v->end(), out);
    return 0;
}
int orc_state_put(orc_state* s, int row, const char* name, const float* in, int64_t n) {
    const std::vector<float>* v = nullptr;
    if (row < 0 || row >= (int)s->rows.size() || !parse_state_name(s, row, name, &v)) return -1;
    std::vector<float>* w = const_cast<std::vector<float>*>(v);
    const std::string nm = name;
    if (nm == "eng.k" || nm == "eng.v") {
        const int per = s->m->enh() * s->m->cfg.eng_head_size;
        if (n % per != 0) return -1;
        w->assign(in, in + n);
        s->rows[row].eng_n = (int)(n / per);
        return 0;
    }
    if ((int64_t)w->size() != n) return -1;
    std::copy(in, in + n, w->begin());
    return 0;
}
int64_t orc_state_seen(const orc_state* s, int row) { return s->rows[row].seen; }

int orc_step(const orc_model* m, orc_state* s, const uint32_t* tok, float* logits) {
    derive(m);
    const int rows = (int)s->rows.size();
    std::vector<RowState*> rp(rows);
    for (int r = 0; r < rows; ++r) rp[r] = &s->rows[r];
    return step_rows(m, rp.data(), rows, tok, logits, m->cfg.vocab, g_trace.on);
}

int orc_forward(const orc_model* m, orc_state* s, const uint32_t* ids, int t, int last_only, float* logits) {
    derive(m);
    const int rows = (int)s->rows.size(), V = m->cfg.vocab;
    std::vector<RowState*> rp(rows);
    for (int r = 0; r < rows; ++r) rp[r] = &s->rows[r];
    std::vector<float> scratch(last_only ? (size_t)rows * V : 0);
    std::vector<uint32_t> tk(rows);
    int rc = 0;
    for (int j = 0; j < t; ++j) {
        for (int r = 0; r < rows; ++r) tk[r] = ids[(size_t)r * t + j];
        int one;
        if (last_only)
            one = step_rows(m, rp.data(), rows, tk.data(), j == t - 1 ? logits : scratch.data(), V, false);
        else
            one = step_rows(m, rp.data(), rows, tk.data(), logits + (size_t)j * V, (size_t)t * V, false);
        if (one < 0) return one;
        rc = std::max(rc, one);
    }
    return rc;
}

void orc_trace_enable(int on) {
    g_trace.on = on != 0;
    if (!on) g_trace.t.clear();
}
int64_t orc_trace_len(const char* name, int block) {
    auto it = g_trace.t.find({name, block});
    return it == g_trace.t.end() ? -1 : (int64_t)it->second.size();
}
int orc_trace_get(const char* name, int block, float* out) {
    auto it = g_trace.t.find({name, block});
    if (it == g_trace.t.end()) return -1;
    std::copy(it->second.begin(), it->second.end(), out);
    return 0;
}

}  // extern "C"

// CPU oracle, part two: the chunk-parallel forms of the fast-weight memory.  TEST INFRASTRUCTURE ONLY: nothing in the
// product library includes, links or runs this file.
//
// A restatement in plain loops of the reference's chunked delta rules, function by function, for ONE head
// (the reference folds batch and heads into one leading dimension; every head is independent):
//   orc_inv_unit_lower   design-tests/nn/gpu/src/model.rs:720-742   (I + A)^-1 by block doubling
//   orc_delta_rule_from  design-tests/nn/gpu/src/model.rs:744-799   chunk-64 WY form of the plain (v0.2) delta rule
//   orc_delta_rec        design-tests/nn/gpu/src/arch.rs:1091-1136  the Ava-0.4 rule token by token (the sequential side)
//   orc_delta_chunk      design-tests/nn/gpu/src/arch.rs:1151-1173,1243-1327  the same rule in chunks (`chunk_core`)
// The reference states these as tensor operations (matmuls in whatever order its backend sums); the loops below sum in
// index order in f32.  Chunked and sequential forms agree to rounding only, which is what the reference's own tests
// ask of them (src/arch/tests.rs:700-753: 1e-4 of max(1, max|ref|); tests/smoke.rs:373-391: 1e-3 with repeated keys).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

using Mat = std::vector<float>;

// C [m, n] = A [m, k] . B [k, n], row-major, summed in k order
void mm(const float* a, const float* b, int m, int k, int n, float* c) {
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float s = 0.f;
            for (int l = 0; l < k; ++l) s += a[(size_t)i * k + l] * b[(size_t)l * n + j];
            c[(size_t)i * n + j] = s;
        }
}
// C [m, n] = A^T . B with A [k, m], B [k, n]
void mm_tn(const float* a, const float* b, int k, int m, int n, float* c) {
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float s = 0.f;
            for (int l = 0; l < k; ++l) s += a[(size_t)l * m + i] * b[(size_t)l * n + j];
            c[(size_t)i * n + j] = s;
        }
}
// C [m, n] = A . B^T with A [m, k], B [n, k]
void mm_nt(const float* a, const float* b, int m, int k, int n, float* c) {
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float s = 0.f;
            for (int l = 0; l < k; ++l) s += a[(size_t)i * k + l] * b[(size_t)j * k + l];
            c[(size_t)i * n + j] = s;
        }
}

// model.rs:720-742: t = I - level(1); for s = 2, 4, ... < c: t = t - t . level(s) . t, where level(s) keeps A's
// lower-left s-block inside each diagonal 2s-block
void inv_unit_lower(const float* a, int c, float* t) {
    auto level = [&](int s, Mat& out) {
        out.assign((size_t)c * c, 0.f);
        for (int i = 0; i < c; ++i)
            for (int j = 0; j < c; ++j)
                if (i / (2 * s) == j / (2 * s) && (i / s) % 2 == 1 && (j / s) % 2 == 0) out[(size_t)i * c + j] = a[(size_t)i * c + j];
    };
    Mat e, te((size_t)c * c), tet((size_t)c * c);
    level(1, e);
    for (int i = 0; i < c; ++i)
        for (int j = 0; j < c; ++j) t[(size_t)i * c + j] = -e[(size_t)i * c + j] + (i == j ? 1.f : 0.f);
    for (int s = 2; s < c; s *= 2) {
        level(s, e);
        mm(t, e.data(), c, c, c, te.data());
        mm(te.data(), t, c, c, c, tet.data());
        for (size_t i = 0; i < (size_t)c * c; ++i) t[i] = t[i] - tet[i];
    }
}

}  // namespace

extern "C" {

void orc_inv_unit_lower(const float* a, int c, float* t) { inv_unit_lower(a, c, t); }

// model.rs:761-799 for one head: q, k, v [t, hs] (q, k unit length), log alpha and beta [t]; f0 [hs, hs] or null (zeros).
// y [t, hs], f1 [hs, hs].  Chunk length: the largest power of two <= 64 dividing t (model.rs:705-711).
void orc_delta_rule_from(int t, int hs, const float* q, const float* k, const float* v, const float* la, const float* beta, const float* f0,
                         float* y, float* f1) {
    int c = 64;
    while (t % c != 0) c /= 2;
    const int nc = t / c;
    Mat f((size_t)hs * hs, 0.f);
    if (f0) f.assign(f0, f0 + (size_t)hs * hs);
    Mat cum(c), dmat((size_t)c * c), a((size_t)c * c), ad((size_t)c * c), ti((size_t)c * c), tu((size_t)c * c), kb((size_t)c * hs), vb((size_t)c * hs),
        w((size_t)c * hs), u((size_t)c * hs), qk((size_t)c * c), qkm((size_t)c * c), qkd((size_t)c * c), wf((size_t)c * hs), qf((size_t)c * hs),
        t1((size_t)c * hs), t2((size_t)c * hs), ut((size_t)c * hs), fresh((size_t)hs * hs), kwf((size_t)hs * hs);
    for (int r = 0; r < nc; ++r) {
        const float *qc = q + (size_t)r * c * hs, *kc = k + (size_t)r * c * hs, *vc = v + (size_t)r * c * hs;
        const float *lac = la + (size_t)r * c, *bc = beta + (size_t)r * c;
        float run = 0.f;
        for (int i = 0; i < c; ++i) cum[i] = (run += lac[i]);  // log Gamma, restarting every chunk
        for (int i = 0; i < c; ++i)
            for (int j = 0; j < c; ++j) dmat[(size_t)i * c + j] = j <= i ? std::exp(cum[i] - cum[j]) : 0.f;  // D o M
        mm_nt(kc, kc, c, hs, c, a.data());
        for (int i = 0; i < c; ++i)
            for (int j = 0; j < c; ++j) a[(size_t)i * c + j] = j < i ? a[(size_t)i * c + j] * bc[i] : 0.f;  // beta_i k_i.k_j, strictly below
        for (size_t i = 0; i < (size_t)c * c; ++i) ad[i] = a[i] * dmat[i];
        for (int i = 0; i < c; ++i)
            for (int x = 0; x < hs; ++x) {
                kb[(size_t)i * hs + x] = kc[(size_t)i * hs + x] * bc[i];
                vb[(size_t)i * hs + x] = vc[(size_t)i * hs + x] * bc[i];
            }
        inv_unit_lower(a.data(), c, ti.data());
        mm(ti.data(), kb.data(), c, c, hs, w.data());
        inv_unit_lower(ad.data(), c, tu.data());
        mm(tu.data(), vb.data(), c, c, hs, u.data());
        mm_nt(qc, kc, c, hs, c, qk.data());
        for (int i = 0; i < c; ++i)
            for (int j = 0; j < c; ++j) {
                qkm[(size_t)i * c + j] = j <= i ? qk[(size_t)i * c + j] : 0.f;
                qkd[(size_t)i * c + j] = qk[(size_t)i * c + j] * dmat[(size_t)i * c + j];
            }
        const float last = cum[c - 1];
        // y = (q F - qkm (W F)) * gam + qkd U
        mm(w.data(), f.data(), c, hs, hs, wf.data());
        mm(qc, f.data(), c, hs, hs, qf.data());
        mm(qkm.data(), wf.data(), c, c, hs, t1.data());
        mm(qkd.data(), u.data(), c, c, hs, t2.data());
        for (int i = 0; i < c; ++i)
            for (int x = 0; x < hs; ++x)
                y[((size_t)r * c + i) * hs + x] = (qf[(size_t)i * hs + x] - t1[(size_t)i * hs + x]) * std::exp(cum[i]) + t2[(size_t)i * hs + x];
        // f = (f - K^T (W F)) * gam_c + K^T (U * tail)
        for (int i = 0; i < c; ++i)
            for (int x = 0; x < hs; ++x) ut[(size_t)i * hs + x] = u[(size_t)i * hs + x] * std::exp(last - cum[i]);
        mm_tn(kc, ut.data(), c, hs, hs, fresh.data());
        mm_tn(kc, wf.data(), c, hs, hs, kwf.data());
        const float gc = std::exp(last);
        for (size_t i = 0; i < (size_t)hs * hs; ++i) f[i] = (f[i] - kwf[i]) * gc + fresh[i];
    }
    std::memcpy(f1, f.data(), (size_t)hs * hs * sizeof(float));
}

// arch.rs:1091-1136 for one head: q, k, e, v [t, hs]; la, b [t, g] (g = 1 per head, hs per channel); momentum m (0: none);
// f0, s0 [hs, hs] or null.  cap: the bound on the state (mem_gen::MEM_CAP, 1e5).  y [t, hs]; f1, s1 [hs, hs] (s1 may be null).
void orc_delta_rec(int t, int hs, int g, const float* q, const float* k, const float* e, const float* v, const float* la, const float* b, float m,
                   const float* f0, const float* s0, float cap, float* y, float* f1, float* s1) {
    Mat f((size_t)hs * hs, 0.f), s((size_t)hs * hs, 0.f), pred(hs), upd((size_t)hs * hs);
    if (f0) f.assign(f0, f0 + (size_t)hs * hs);
    if (s0 && m > 0.f) s.assign(s0, s0 + (size_t)hs * hs);
    for (int i = 0; i < t; ++i) {
        const float *qi = q + (size_t)i * hs, *ki = k + (size_t)i * hs, *ei = e + (size_t)i * hs, *vi = v + (size_t)i * hs;
        auto al = [&](int row) { return std::exp(la[(size_t)i * g + (g == 1 ? 0 : row)]); };
        auto bw = [&](int row) { return b[(size_t)i * g + (g == 1 ? 0 : row)]; };
        for (int x = 0; x < hs; ++x) {  // pred = e^T F
            float sum = 0.f;
            for (int r = 0; r < hs; ++r) sum += ei[r] * f[(size_t)r * hs + x];
            pred[x] = sum;
        }
        for (int r = 0; r < hs; ++r)
            for (int x = 0; x < hs; ++x) upd[(size_t)r * hs + x] = (ki[r] * bw(r)) * vi[x] - ((ei[r] * bw(r)) * pred[x]) * al(r);
        for (int r = 0; r < hs; ++r)
            for (int x = 0; x < hs; ++x) {
                const size_t at = (size_t)r * hs + x;
                const float fa = f[at] * al(r);
                float nf;
                if (m > 0.f) {
                    s[at] = s[at] * m + upd[at];
                    nf = fa + s[at];
                } else {
                    nf = fa + upd[at];
                }
                f[at] = std::min(std::max(nf, -cap), cap);
            }
        for (int x = 0; x < hs; ++x) {
            float sum = 0.f;
            for (int r = 0; r < hs; ++r) sum += qi[r] * f[(size_t)r * hs + x];
            y[(size_t)i * hs + x] = sum;
        }
    }
    std::memcpy(f1, f.data(), (size_t)hs * hs * sizeof(float));
    if (s1 && m > 0.f) std::memcpy(s1, s.data(), (size_t)hs * hs * sizeof(float));
}

// arch.rs:1151-1173 + 1243-1327 (`delta_chunk` -> `chunk_core`) for one head, same arguments as orc_delta_rec (no cap: the
// chunked form cannot hold it, arch.rs:1139-1141).  Chunk length: 64 per head gates, 16 per channel, halved until it
// divides t (arch.rs:1167-1173).
void orc_delta_chunk(int t, int hs, int g, const float* q, const float* k, const float* e, const float* v, const float* la, const float* b, float m,
                     const float* f0, const float* s0, float* y, float* f1, float* s1) {
    int c = g == 1 ? 64 : 16;
    while (t % c != 0) c /= 2;
    const int nc = t / c;
    const bool mom = m > 0.f;
    Mat f((size_t)hs * hs, 0.f), s((size_t)hs * hs, 0.f);
    if (f0) f.assign(f0, f0 + (size_t)hs * hs);
    if (s0 && mom) s.assign(s0, s0 + (size_t)hs * hs);
    const size_t ch = (size_t)c * hs, cg = (size_t)c * g, ccg = (size_t)c * c * g, cc = (size_t)c * c;
    Mat w(ch), ah(ch), cum(cg), cumex(cg), dm(ccg), kk(ccg), kp(ccg), qw(cc), qa(cc), ke(cc), ae(cc), tinv(cc), x1(ch), p1(ch), kev(ch), r0(ch), qg(ch),
        qwv(ch), wl(ch), alk(ch), wlv((size_t)hs * hs), al((size_t)hs * c), gs(cg), gsx(cg), wmu(ch), amu(ch), wm((size_t)hs * hs), am((size_t)hs * c), p2(ch),
        qs(ch), rr(ch), t1(ch), t2(ch), t3(ch), alr((size_t)hs * hs), amr((size_t)hs * hs);
    auto G = [&](int ch_) { return g == 1 ? 0 : ch_; };
    for (int r = 0; r < nc; ++r) {
        const float *qc = q + (size_t)r * ch, *kc = k + (size_t)r * ch, *ec = e + (size_t)r * ch, *vc = v + (size_t)r * ch;
        const float *lac = la + (size_t)r * cg, *bc = b + (size_t)r * cg;
        for (int i = 0; i < c; ++i)
            for (int x = 0; x < hs; ++x) {
                const float bw = bc[(size_t)i * g + G(x)], lv = lac[(size_t)i * g + G(x)];
                w[(size_t)i * hs + x] = kc[(size_t)i * hs + x] * bw;                 // write key
                ah[(size_t)i * hs + x] = ec[(size_t)i * hs + x] * (bw * std::exp(lv));  // erase key alpha*b*e
            }
        for (int z = 0; z < g; ++z) {
            float run = 0.f;
            for (int i = 0; i < c; ++i) {
                cumex[(size_t)i * g + z] = run;  // cum - la: the sum before the position (taken before the add: the same value)
                run += lac[(size_t)i * g + z];
                cum[(size_t)i * g + z] = run;
                cumex[(size_t)i * g + z] = cum[(size_t)i * g + z] - lac[(size_t)i * g + z];
            }
        }
        for (int i = 0; i < c; ++i)
            for (int mm_ = 0; mm_ < c; ++mm_)
                for (int z = 0; z < g; ++z)
                    dm[((size_t)i * c + mm_) * g + z] = mm_ <= i ? std::exp(cum[(size_t)i * g + z] - cum[(size_t)mm_ * g + z]) : 0.f;
        if (mom) {  // K_ij = sum_m D_im M^(m-j) for m >= j
            for (int i = 0; i < c; ++i)
                for (int j = 0; j < c; ++j)
                    for (int z = 0; z < g; ++z) {
                        float sum = 0.f;
                        for (int mm_ = 0; mm_ < c; ++mm_)
                            if (mm_ >= j) sum += dm[((size_t)i * c + mm_) * g + z] * (float)std::pow((double)m, mm_ - j);
                        kk[((size_t)i * c + j) * g + z] = sum;
                    }
        } else {
            kk = dm;
        }
        for (int i = 0; i < c; ++i)
            for (int j = 0; j < c; ++j)
                for (int z = 0; z < g; ++z) kp[((size_t)i * c + j) * g + z] = i > 0 ? kk[((size_t)(i - 1) * c + j) * g + z] : 0.f;
        // sum over channels of x_i K_ij y_j
        auto pair = [&](const float* x, const Mat& kern, const float* yv, Mat& out) {
            for (int i = 0; i < c; ++i)
                for (int j = 0; j < c; ++j) {
                    float sum = 0.f;
                    if (g == 1) {
                        for (int z = 0; z < hs; ++z) sum += x[(size_t)i * hs + z] * yv[(size_t)j * hs + z];
                        sum *= kern[(size_t)i * c + j];
                    } else {
                        for (int z = 0; z < hs; ++z) sum += (x[(size_t)i * hs + z] * kern[((size_t)i * c + j) * g + z]) * yv[(size_t)j * hs + z];
                    }
                    out[(size_t)i * c + j] = sum;
                }
        };
        pair(qc, kk, w.data(), qw);
        pair(qc, kk, ah.data(), qa);
        pair(ec, kp, w.data(), ke);
        pair(ec, kp, ah.data(), ae);
        inv_unit_lower(ae.data(), c, tinv.data());
        for (int i = 0; i < c; ++i)
            for (int x = 0; x < hs; ++x) {
                x1[(size_t)i * hs + x] = ec[(size_t)i * hs + x] * std::exp(cumex[(size_t)i * g + G(x)]);
                qg[(size_t)i * hs + x] = qc[(size_t)i * hs + x] * std::exp(cum[(size_t)i * g + G(x)]);
            }
        mm(tinv.data(), x1.data(), c, c, hs, p1.data());
        mm(ke.data(), vc, c, c, hs, kev.data());
        mm(tinv.data(), kev.data(), c, c, hs, r0.data());
        mm(qw.data(), vc, c, c, hs, qwv.data());
        for (int j = 0; j < c; ++j)
            for (int x = 0; x < hs; ++x) {
                const float kl = kk[((size_t)(c - 1) * c + j) * g + G(x)];  // K_{c-1, j}
                wl[(size_t)j * hs + x] = w[(size_t)j * hs + x] * kl;
                alk[(size_t)j * hs + x] = ah[(size_t)j * hs + x] * kl;
            }
        mm_tn(wl.data(), vc, c, hs, hs, wlv.data());
        for (int j = 0; j < c; ++j)
            for (int x = 0; x < hs; ++x) al[(size_t)x * c + j] = alk[(size_t)j * hs + x];
        if (mom) {
            for (int i = 0; i < c; ++i)
                for (int z = 0; z < g; ++z) {
                    gs[(size_t)i * g + z] = kk[((size_t)i * c + 0) * g + z] * m;   // M K_i0
                    gsx[(size_t)i * g + z] = kp[((size_t)i * c + 0) * g + z] * m;
                }
            for (int p = 0; p < c; ++p) {
                const float mu = (float)std::pow((double)m, c - 1 - p);
                for (int x = 0; x < hs; ++x) {
                    wmu[(size_t)p * hs + x] = w[(size_t)p * hs + x] * mu;
                    amu[(size_t)p * hs + x] = ah[(size_t)p * hs + x] * mu;
                }
            }
            mm_tn(wmu.data(), vc, c, hs, hs, wm.data());
            for (int j = 0; j < c; ++j)
                for (int x = 0; x < hs; ++x) am[(size_t)x * c + j] = amu[(size_t)j * hs + x];
            for (int i = 0; i < c; ++i)
                for (int x = 0; x < hs; ++x) {
                    x1[(size_t)i * hs + x] = ec[(size_t)i * hs + x] * gsx[(size_t)i * g + G(x)];
                    qs[(size_t)i * hs + x] = qc[(size_t)i * hs + x] * gs[(size_t)i * g + G(x)];
                }
            mm(tinv.data(), x1.data(), c, c, hs, p2.data());
        }
        // the recalls, the reads, the new state
        mm(p1.data(), f.data(), c, hs, hs, rr.data());
        for (size_t i = 0; i < ch; ++i) rr[i] = rr[i] + r0[i];
        if (mom) {
            mm(p2.data(), s.data(), c, hs, hs, t1.data());
            for (size_t i = 0; i < ch; ++i) rr[i] = rr[i] + t1[i];
        }
        mm(qg.data(), f.data(), c, hs, hs, t1.data());
        mm(qa.data(), rr.data(), c, c, hs, t2.data());
        for (size_t i = 0; i < ch; ++i) t1[i] = (t1[i] + qwv[i]) - t2[i];
        if (mom) {
            mm(qs.data(), s.data(), c, hs, hs, t3.data());
            for (size_t i = 0; i < ch; ++i) t1[i] = t1[i] + t3[i];
        }
        std::memcpy(y + (size_t)r * ch, t1.data(), ch * sizeof(float));
        mm(al.data(), rr.data(), hs, c, hs, alr.data());
        if (mom) mm(am.data(), rr.data(), hs, c, hs, amr.data());
        const float mc = (float)std::pow((double)m, c);
        for (int row = 0; row < hs; ++row)
            for (int x = 0; x < hs; ++x) {
                const size_t at = (size_t)row * hs + x;
                const float gcv = std::exp(cum[(size_t)(c - 1) * g + G(row)]);  // Gamma_c as row scales
                float fn = (f[at] * gcv + wlv[at]) - alr[at];
                if (mom) {
                    fn = fn + s[at] * gs[(size_t)(c - 1) * g + G(row)];
                    s[at] = (s[at] * mc + wm[at]) - amr[at];
                }
                f[at] = fn;
            }
    }
    std::memcpy(f1, f.data(), (size_t)hs * hs * sizeof(float));
    if (s1 && mom) std::memcpy(s1, s.data(), (size_t)hs * hs * sizeof(float));
}

}  // extern "C"

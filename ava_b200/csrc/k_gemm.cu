// The int8-weight products of the block step for a batch of rows (sm_100a, CUDA cores).
//
// The reference keeps activations in f32 and sums x[j] * (f32) q[j][c] with one fused multiply-add per term in the
// order j = 0, 1, ..., d_in - 1 from +0, then multiplies by the column's scale (design-tests/nn/gpu/src/int8.rs:3-8,
// 315-331).  Any other summation order rounds differently, and one flipped spike or k-WTA winner sends a spiking
// model down another path, so this kernel keeps that order: each thread owns a 4x4 block of outputs and walks k
// upwards, never splitting K.  The int8 tile is widened to f32 once when it is staged in shared memory and reused by
// every row of the tile.
#include <algorithm>
#include <cstdlib>

#include "ava_math.h"
#include "kernels.cuh"
#include "row_sums.cuh"

namespace ava {

namespace {

constexpr int BK = 16;

// Four int8 weights packed in a word, widened to f32 without the (quarter-rate) integer-to-float unit: a byte b + 128
// placed in the mantissa of 2^23 is the float 8388608 + b + 128 exactly, and subtracting 8388736 leaves b.
__device__ __forceinline__ void widen4(int w, float* f) {
    const unsigned u = (unsigned)w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)) - 8388736.0f;
}

// One LIF update of one channel (src/model/fstep/arch.rs:173-228) with the hard spike count taken directly (as the
// reference's own GPU kernel does; the CPU's soft + (hard - soft) equals it).  v, s, a: the carried state, in and out.
// ne: --neuromod's NE signal of the row (1 without it: a product with 1 is exact), applied after --lif-scale.
// MG: --mood's gain of this (token-row, channel) after NE (src/model/fstep/arch.rs:646-650); only the scan kernel has it.
template <bool MG = false>
__device__ __forceinline__ void lif_math(int spikes, int lif_scale, bool adaptive, float beta, float th, float rho, float gain, float ne, float cur,
                                         float& v, float& s, float& a, float mg = 1.0f) {
    if (lif_scale) cur = mul(cur, add(mul(beta, -1.0f), 1.0f));
    cur = mul(cur, ne);
    if (MG) cur = mul(cur, mg);
    float th_prev = th, th_t = th;
    if (adaptive) {
        th_prev = add(th, mul(a, gain));
        a = add(mul(a, rho), mul(fabsf(s), add(mul(rho, -1.0f), 1.0f)));
        th_t = add(th, mul(a, gain));
    }
    const float vv = sub(add(mul(v, beta), cur), mul(s, th_prev));
    v = vv;
    if (spikes == 0) {
        s = sub(vv, th_t) >= 0.0f ? 1.0f : 0.0f;
    } else {
        const int levels = spikes == 2 ? 2 : 1;
        float n = 0.0f;
        for (int k = 1; k <= levels; ++k) {
            const float kth = add(mul(th_t, (float)k), 0.0f);
            const float up = sub(vv, kth), down = sub(-vv, kth);
            n += (up >= 0.0f ? 1.0f : 0.0f) - (down >= 0.0f ? 1.0f : 0.0f);
        }
        s = n;
    }
}

template <bool MG = false>
__device__ __forceinline__ void lif_core(const LifParams& p, int c, float ne, float cur, float& v, float& s, float& a, float mg = 1.0f) {
    lif_math<MG>(p.spikes, p.lif_scale, p.rho != nullptr, p.beta[c], p.theta ? p.theta[c] : 1.0f, p.rho ? p.rho[c] : 0.0f, p.rho ? p.gain[c] : 0.0f, ne,
                 cur, v, s, a, mg);
}

__device__ __forceinline__ void lif_update(const LifParams& p, int r, int c, int d, float cur) {
    const size_t i = (size_t)r * d + c;
    float v = p.v[i], s = p.s[i], a = p.rho ? p.a[i] : 0.0f;
    lif_core(p, c, p.ne ? p.ne[(size_t)r * NM_STRIDE] : 1.0f, cur, v, s, a);
    p.v[i] = v;
    p.s[i] = s;
    if (p.rho) p.a[i] = a;
}

// The LIF over a chunk of T tokens: one thread per (row, channel) walks the tokens in order with the membrane, last
// spike and trace in registers (the reset makes the recurrence nonlinear, so time stays sequential; the parallelism is
// rows x channels).  cur and spikes are time-major [T][M][d]; so is cur_gain (--mood's gain of the current, or nullptr).
__global__ void lif_scan_kernel(const float* __restrict__ cur, const LifParams p, int M, int d, int T, float* __restrict__ spikes,
                                const float* __restrict__ cur_gain) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t Md = (size_t)M * d;
    if (i >= Md) return;
    const int c = (int)(i % d);
    float v = p.v[i], s = p.s[i], a = p.rho ? p.a[i] : 0.0f;
    float nxt = cur[i];
    for (int t = 0; t < T; ++t) {
        const float x = nxt;
        if (t + 1 < T) nxt = cur[(size_t)(t + 1) * Md + i];
        // the NE signal belongs to the token-row: row (t, i / d) of the chunk
        const float ne = p.ne ? p.ne[((size_t)t * M + i / d) * NM_STRIDE] : 1.0f;
        if (cur_gain)
            lif_core<true>(p, c, ne, x, v, s, a, cur_gain[(size_t)t * Md + i]);
        else
            lif_core(p, c, ne, x, v, s, a);
        spikes[(size_t)t * Md + i] = s;
    }
    p.v[i] = v;
    p.s[i] = s;
    if (p.rho) p.a[i] = a;
}

// Tile BM x BN per block, TM x TN outputs per thread (TM = 4; TN = 4 or 2).  Wide products use 64x64 tiles of 4x4; the
// narrow ones (N = d) use 32x64 tiles of 4x2 so that twice the warps share the same work and cover each other's
// shared-memory latency.
template <int BM, int BN, int TM, int TN, int EPI>
__global__ void __launch_bounds__((BM / TM) * (BN / TN)) q8_gemm_kernel(const GemmArgs g) {
    pdl_enter();
    static_assert((TM == 4 || TM == 8) && (TN == 8 || TN == 4 || TN == 2), "micro-tile");
    constexpr int T = (BM / TM) * (BN / TN);
    constexpr int AS = BM + 4;  // padded row length of the k-major A tile
    __shared__ __align__(16) float As[2][BK][AS];
    __shared__ __align__(16) float Ws[2][BK][BN];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nk = g.K / BK;

    constexpr int KQ = BK / 4;                      // float4 per A-tile row
    constexpr int A_N = BM * KQ, W_N = BK * BN / 4; // float4 of the A tile, words of the W tile
    constexpr int A_LOADS = (A_N + T - 1) / T;      // float4 per thread
    constexpr int W_LOADS = (W_N + T - 1) / T;      // char4 per thread
    constexpr int PF = 4;                           // tiles fetched ahead into registers (global latency cover)
    float4 ra[PF][A_LOADS];
    int rw[PF][W_LOADS];

    auto load_global = [&](int kt, float4* fa, int* fw) {
#pragma unroll
        for (int i = 0; i < A_LOADS; ++i) {
            const int idx = tid + i * T;
            const int row = idx / KQ, kq = idx % KQ;
            fa[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (kt < nk && idx < A_N && m0 + row < g.M)
                fa[i] = *reinterpret_cast<const float4*>(g.A + (size_t)(m0 + row) * g.lda + kt * BK + kq * 4);
        }
#pragma unroll
        for (int i = 0; i < W_LOADS; ++i) {
            const int idx = tid + i * T;
            const int k = idx / (BN / 4), n4 = idx % (BN / 4);
            fw[i] = 0;
            if (kt < nk && idx < W_N && n0 + n4 * 4 < g.N)
                fw[i] = __ldg(reinterpret_cast<const int*>(g.W + (size_t)(kt * BK + k) * g.ldw + n0 + n4 * 4));
        }
    };
    auto store_smem = [&](int buf, const float4* fa, const int* fw) {
#pragma unroll
        for (int i = 0; i < A_LOADS; ++i) {
            const int idx = tid + i * T;
            const int row = idx / KQ, kq = idx % KQ;
            if (idx < A_N) {
                As[buf][kq * 4 + 0][row] = fa[i].x;
                As[buf][kq * 4 + 1][row] = fa[i].y;
                As[buf][kq * 4 + 2][row] = fa[i].z;
                As[buf][kq * 4 + 3][row] = fa[i].w;
            }
        }
#pragma unroll
        for (int i = 0; i < W_LOADS; ++i) {
            const int idx = tid + i * T;
            const int k = idx / (BN / 4), n4 = idx % (BN / 4);
            if (idx < W_N) {
                float f[4];
                widen4(fw[i], f);
                *reinterpret_cast<float4*>(&Ws[buf][k][n4 * 4]) = make_float4(f[0], f[1], f[2], f[3]);
            }
        }
    };
    auto frag = [&](int buf, int k, float* av, float* bv) {
#pragma unroll
        for (int i = 0; i < TM; i += 4) {
            const float4 a = *reinterpret_cast<const float4*>(&As[buf][k][ty * TM + i]);
            av[i] = a.x; av[i + 1] = a.y; av[i + 2] = a.z; av[i + 3] = a.w;
        }
        if (TN >= 4) {
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const float4 b = *reinterpret_cast<const float4*>(&Ws[buf][k][tx * TN + j]);
                bv[j] = b.x; bv[j + 1] = b.y; bv[j + 2] = b.z; bv[j + 3] = b.w;
            }
        } else {
            const float2 b = *reinterpret_cast<const float2*>(&Ws[buf][k][tx * TN]);
            bv[0] = b.x; bv[1] = b.y;
        }
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

#pragma unroll
    for (int s = 0; s < PF; ++s) load_global(s, ra[s], rw[s]);
    store_smem(0, ra[0], rw[0]);
    __syncthreads();
    // tile kt sits in shared buffer kt & 1 and its registers (slot kt % PF) are free again: they take tile kt + PF
    for (int kt0 = 0; kt0 < nk; kt0 += PF) {
#pragma unroll
        for (int s = 0; s < PF; ++s) {
            const int kt = kt0 + s;
            if (kt < nk) {
                load_global(kt + PF, ra[s], rw[s]);
                // the fragments of step k + 1 are fetched before the multiply-adds of step k
                float av[2][TM], bv[2][TN];
                frag(s & 1, 0, av[0], bv[0]);
#pragma unroll
                for (int k = 0; k < BK; ++k) {
                    if (k + 1 < BK) frag(s & 1, k + 1, av[(k + 1) & 1], bv[(k + 1) & 1]);
#pragma unroll
                    for (int i = 0; i < TM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) acc[i][j] = fma(av[k & 1][i], bv[k & 1][j], acc[i][j]);
                }
                if (kt + 1 < nk) store_smem((s + 1) & 1, ra[(s + 1) % PF], rw[(s + 1) % PF]);
                __syncthreads();
            }
        }
    }

    const int c0 = n0 + tx * TN;
    if (c0 >= g.N) return;
    float scv[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) scv[j] = g.scale[c0 + j];
    float lbeta[TN], lth[TN], lrho[TN], lgain[TN];  // the LIF's per-channel parameters of this thread's columns
    if (EPI == EPI_LIF) {
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            lbeta[j] = g.lif.beta[c0 + j];
            lth[j] = g.lif.theta ? g.lif.theta[c0 + j] : 1.0f;
            lrho[j] = g.lif.rho ? g.lif.rho[c0 + j] : 0.0f;
            lgain[j] = g.lif.rho ? g.lif.gain[c0 + j] : 0.0f;
        }
    }
    float resid[TM][TN];  // EPI_ADD: what the product is added to, read for the whole micro-tile before any row is written
    if (EPI == EPI_ADD) {
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = m0 + ty * TM + i;
            const float* src = g.C + (size_t)(r < g.M ? r : 0) * g.ldc + c0;
            if (TN >= 4) {
#pragma unroll
                for (int j = 0; j < TN; j += 4) {
                    const float4 x = *reinterpret_cast<const float4*>(src + j);
                    resid[i][j] = x.x; resid[i][j + 1] = x.y; resid[i][j + 2] = x.z; resid[i][j + 3] = x.w;
                }
            } else {
                const float2 x = *reinterpret_cast<const float2*>(src);
                resid[i][0] = x.x; resid[i][1] = x.y;
            }
        }
    }
    if (EPI == EPI_LIF) {
        // The carried state of the whole micro-tile is read before any of it is written: the stores would otherwise
        // fence the next element's loads, and every element would wait a memory round trip of its own.
        const LifParams& p = g.lif;
        float v[TM][TN], sp[TM][TN], tr[TM][TN], lne[TM];
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = m0 + ty * TM + i;
            lne[i] = p.ne ? p.ne[(size_t)(r < g.M ? r : 0) * NM_STRIDE] : 1.0f;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const size_t at = (size_t)(r < g.M ? r : 0) * g.N + c0 + j;
                v[i][j] = p.v[at];
                sp[i][j] = p.s[at];
                tr[i][j] = p.rho ? p.a[at] : 0.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j)
                lif_math(p.spikes, p.lif_scale, p.rho != nullptr, lbeta[j], lth[j], lrho[j], lgain[j], lne[i], mul(acc[i][j], scv[j]), v[i][j], sp[i][j],
                         tr[i][j]);
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = m0 + ty * TM + i;
            if (r >= g.M) continue;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const size_t at = (size_t)r * g.N + c0 + j;
                p.v[at] = v[i][j];
                p.s[at] = sp[i][j];
                if (p.rho) p.a[at] = tr[i][j];
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = m0 + ty * TM + i;
        if (r >= g.M) continue;
        float o[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) o[j] = mul(acc[i][j], scv[j]);
        if (EPI == EPI_ADD && g.lif.ne) {
            const float rg = g.lif.ne[(size_t)r * NM_STRIDE];
#pragma unroll
            for (int j = 0; j < TN; ++j) o[j] = mul(o[j], rg);
        }
        if (EPI == EPI_LIF) {
            // handled above for the whole micro-tile
        } else {
            float* dst = g.C + (size_t)r * g.ldc + c0;
            if (TN >= 4) {
#pragma unroll
                for (int j = 0; j < TN; j += 4) {
                    float4* d4 = reinterpret_cast<float4*>(dst + j);
                    if (EPI == EPI_ADD) {
                        o[j] = add(resid[i][j], o[j]); o[j + 1] = add(resid[i][j + 1], o[j + 1]);
                        o[j + 2] = add(resid[i][j + 2], o[j + 2]); o[j + 3] = add(resid[i][j + 3], o[j + 3]);
                    }
                    *d4 = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
                }
            } else {
                float2* d2 = reinterpret_cast<float2*>(dst);
                if (EPI == EPI_ADD) {
                    o[0] = add(resid[i][0], o[0]); o[1] = add(resid[i][1], o[1]);
                }
                *d2 = make_float2(o[0], o[1]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------- few rows
// The same product when there are only a few rows (one sequence talking, a handful generating): the tiled kernel above
// then spends its time on 48 rounds of load-sync-multiply per output, one after another.  Here a block takes 64 output
// columns and ALL K rows of their weights: the K x 64 int8 tile is requested at once (cp.async, every thread copies, one
// latency for the lot) and sits in shared memory; then one thread per (row pair, four columns) walks k = 0, 1, ... with
// its 8 accumulators, weights read from shared memory, inputs from a staged copy of the rows.  The sums are the same
// fma chains in the same order, so the same bits.
constexpr int RT_COLS = 64, RT_THREADS = 256, RT_ROWS = 32;  // rows per block: 16 row lanes x 2 rows

template <int EPI>
__global__ void __launch_bounds__(RT_THREADS) q8_resident_kernel(const GemmArgs g) {
    pdl_enter();
    extern __shared__ __align__(16) unsigned char rt_smem[];
    int8_t* wt = reinterpret_cast<int8_t*>(rt_smem);                            // [K][64]
    float* xs = reinterpret_cast<float*>(rt_smem + (size_t)g.K * RT_COLS);      // [rows][K]
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * RT_COLS, m0 = blockIdx.y * RT_ROWS;
    const int rows = min(RT_ROWS, g.M - m0);
    // the weights: K rows of 64 bytes, 16 bytes per copy
    for (int i = tid; i < g.K * 4; i += RT_THREADS) {
        const int k = i >> 2, q = i & 3;
        if (n0 + q * 16 < g.N)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(wt + (size_t)k * RT_COLS + q * 16)),
                         "l"(g.W + (size_t)k * g.ldw + n0 + q * 16)
                         : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    // the rows' inputs
    for (int i = tid; i < rows * (g.K / 4); i += RT_THREADS) {
        const int r = i / (g.K / 4), k4 = i - r * (g.K / 4);
        reinterpret_cast<float4*>(xs + (size_t)r * g.K)[k4] = *reinterpret_cast<const float4*>(g.A + (size_t)(m0 + r) * g.lda + 4 * k4);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const int cg = tid & 15, rl = tid >> 4;  // four columns cg * 4 .., rows rl and rl + 16
    const int c0 = n0 + cg * 4;
    if (c0 >= g.N || rl >= rows) return;
    const bool two = rl + 16 < rows;
    const float* x0 = xs + (size_t)rl * g.K;
    const float* x1 = xs + (size_t)(two ? rl + 16 : rl) * g.K;
    const int* wp = reinterpret_cast<const int*>(wt + cg * 4);
    float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
    auto lds_w = [&](int k) {
        int w;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w) : "r"((uint32_t)__cvta_generic_to_shared(wp + (size_t)k * (RT_COLS / 4))));
        return w;
    };
    auto lds_x = [&](const float* p) {
        float4 v;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"((uint32_t)__cvta_generic_to_shared(p)));
        return v;
    };
    // four k at a time, the next four on their way
    int w[4];
    float4 xa = lds_x(x0), xb = lds_x(x1);
#pragma unroll
    for (int u = 0; u < 4; ++u) w[u] = lds_w(u);
    for (int k = 0; k < g.K; k += 4) {
        const int kn = k + 4 < g.K ? k + 4 : k;
        int nw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) nw[u] = lds_w(kn + u);
        const float4 nxa = lds_x(x0 + kn), nxb = lds_x(x1 + kn);
        const float va[4] = {xa.x, xa.y, xa.z, xa.w}, vb[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float f[4];
            widen4(w[u], f);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                a0[j] = fma(va[u], f[j], a0[j]);
                a1[j] = fma(vb[u], f[j], a1[j]);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) w[u] = nw[u];
        xa = nxa;
        xb = nxb;
    }
    const float4 sc = *reinterpret_cast<const float4*>(g.scale + c0);
    const float scv[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (h == 1 && !two) break;
        const int r = m0 + rl + 16 * h;
        const float* acc = h ? a1 : a0;
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = mul(acc[j], scv[j]);
        if (EPI == EPI_ADD && g.lif.ne) {
            const float rg = g.lif.ne[(size_t)r * NM_STRIDE];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = mul(o[j], rg);
        }
        if (EPI == EPI_LIF) {
#pragma unroll
            for (int j = 0; j < 4; ++j) lif_update(g.lif, r, c0 + j, g.N, o[j]);
        } else {
            float4* d4 = reinterpret_cast<float4*>(g.C + (size_t)r * g.ldc + c0);
            if (EPI == EPI_ADD) {
                const float4 x = *d4;
                o[0] = add(x.x, o[0]); o[1] = add(x.y, o[1]); o[2] = add(x.z, o[2]); o[3] = add(x.w, o[3]);
            }
            *d4 = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

// false: shape not covered (the tile and the rows must fit shared memory; N a multiple of 16; 16-byte aligned rows)
bool launch_resident(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi) {
    const int rows = a.M < RT_ROWS ? a.M : RT_ROWS;
    const size_t smem = (size_t)a.K * RT_COLS + (size_t)rows * a.K * sizeof(float);
    if (smem > 220 * 1024 || a.N % 16 || a.K % 4 || a.ldw % 16 || a.lda % 4) return false;
    dim3 grid((a.N + RT_COLS - 1) / RT_COLS, (a.M + RT_ROWS - 1) / RT_ROWS);
    auto go = [&](auto kernel) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(kernel, grid, dim3(RT_THREADS), smem, st, a);
    };
    switch (epi) {
        case EPI_STORE: go(q8_resident_kernel<EPI_STORE>); break;
        case EPI_ADD: go(q8_resident_kernel<EPI_ADD>); break;
        case EPI_LIF: go(q8_resident_kernel<EPI_LIF>); break;
    }
    return true;
}

// ------------------------------------------------------------------------------------------- a few rows (one sequence)
// With one sequence (or a handful) a product is a chain of K dependent multiply-adds per output and nothing else, so the
// kernel is laid out for latency: a block owns 32 output columns, all its threads request the [K][32] strip of weights
// at once (the weights do not depend on the kernel before, so they are requested BEFORE the wait for it), and then one
// warp per row walks k with one column per lane: one shared-memory byte, one conversion, one multiply-add per step.
constexpr int GV_COLS = 32, GV_THREADS = 256, GV_ROWS = GV_THREADS / 32;

template <int EPI>
__global__ void __launch_bounds__(GV_THREADS) q8_gemv_kernel(const GemmArgs g, const GemvPro pro) {
    extern __shared__ __align__(16) unsigned char gv_smem[];
    int8_t* wt = reinterpret_cast<int8_t*>(gv_smem);                          // [K][32]
    float* xs = reinterpret_cast<float*>(gv_smem + (size_t)g.K * GV_COLS);    // [rows][K]
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * GV_COLS, m0 = blockIdx.y * GV_ROWS;
    const int rows = min(GV_ROWS, g.M - m0);
    for (int i = tid; i < g.K * 2; i += GV_THREADS) {
        const int k = i >> 1, q = i & 1;
        if (n0 + q * 16 < g.N)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(wt + (size_t)k * GV_COLS + q * 16)),
                         "l"(g.W + (size_t)k * g.ldw + n0 + q * 16)
                         : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    pdl_enter();
    for (int i = tid; i < rows * (g.K / 4); i += GV_THREADS) {
        const int r = i / (g.K / 4), k4 = i - r * (g.K / 4);
        reinterpret_cast<float4*>(xs + (size_t)r * g.K)[k4] = *reinterpret_cast<const float4*>(g.A + (size_t)(m0 + r) * g.lda + 4 * k4);
    }
    // the prologue's own vectors come in with the rows (one latency for all): the norm's gain [K], or the rows' gates [rows][K]
    float* aux = xs + (size_t)rows * g.K;
    if (pro.kind == PRO_RMS) {
        for (int i = tid; i < g.K / 4; i += GV_THREADS) reinterpret_cast<float4*>(aux)[i] = reinterpret_cast<const float4*>(pro.gain)[i];
    } else if (pro.kind == PRO_POST && pro.gate) {
        for (int i = tid; i < rows * (g.K / 4); i += GV_THREADS) {
            const int r = i / (g.K / 4), k4 = i - r * (g.K / 4);
            reinterpret_cast<float4*>(aux + (size_t)r * g.K)[k4] = *reinterpret_cast<const float4*>(pro.gate + (size_t)(m0 + r) * pro.ldg + 4 * k4);
        }
    }
    const int cl = tid & 31, rl = tid >> 5, c = n0 + cl;
    if (pro.kind != PRO_NONE) {
        // one thread per ordered sum (a row's, or a head's of a row), all of them side by side; then every thread of the
        // block scales its share of the elements.  The weights are still arriving meanwhile.
        float* inv_sh = aux + (pro.kind == PRO_RMS ? g.K : (pro.gate ? (size_t)rows * g.K : 0));   // [rows] or [rows][heads]
        __syncthreads();
        if (pro.kind == PRO_RMS) {
            if (cl == 0 && rl < rows) inv_sh[rl] = inv_rms_seq(xs + (size_t)rl * g.K, g.K);
            __syncthreads();
            for (int i = tid; i < rows * g.K; i += GV_THREADS) {
                const int r = i / g.K, col = i - r * g.K;
                const float v = mul(mul(xs[i], inv_sh[r]), aux[col]);
                xs[i] = v;
                if (pro.out && blockIdx.x == 0) pro.out[(size_t)(m0 + r) * g.K + col] = v;
            }
        } else {
            const int nh = g.K / pro.hs;
            // lane 0 of each warp takes a sum at a time (sums side by side in one warp would meet in one shared-memory bank)
            for (int p = rl; p < rows * nh; p += GV_THREADS / 32)
                if (cl == 0) inv_sh[p] = inv_rms_seq(xs + (size_t)p * pro.hs, pro.hs);   // row p / nh, head p % nh
            __syncthreads();
            for (int i = tid; i < rows * g.K; i += GV_THREADS) {
                const int r = i / g.K, col = i - r * g.K;
                float v = mul(xs[i], inv_sh[i / pro.hs]);
                if (pro.gate) {
                    const float gt = aux[i];
                    v = mul(v, div(gt, add(1.0f, expf_(-gt))));
                }
                xs[i] = v;
                if (pro.out && blockIdx.x == 0) pro.out[(size_t)(m0 + r) * g.K + col] = v;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (c >= g.N || rl >= rows) return;
    const float* x = xs + (size_t)rl * g.K;
    const int8_t* wp = wt + cl;
    // what the epilogue reads from global memory is requested before the chain: its latency passes under it
    const int r = m0 + rl;
    const float sc = g.scale[c];
    float* dst = EPI == EPI_LIF ? nullptr : g.C + (size_t)r * g.ldc + c;
    const float before = EPI == EPI_ADD ? *dst : 0.0f;
    const float row_gain = (EPI == EPI_ADD && g.lif.ne) ? g.lif.ne[(size_t)r * NM_STRIDE] : 1.0f;
    // (the LIF update's state and parameters of this channel too: lif_update's loads, made early)
    const size_t li = (size_t)r * g.N + c;
    float lv = 0.f, ls = 0.f, la = 0.f, l_beta = 0.f, l_th = 1.0f, l_rho = 0.f, l_gain = 0.f, l_ne = 1.0f;
    if (EPI == EPI_LIF) {
        const LifParams& p = g.lif;
        lv = p.v[li];
        ls = p.s[li];
        la = p.rho ? p.a[li] : 0.0f;
        l_beta = p.beta[c];
        l_th = p.theta ? p.theta[c] : 1.0f;
        l_rho = p.rho ? p.rho[c] : 0.0f;
        l_gain = p.rho ? p.gain[c] : 0.0f;
        l_ne = p.ne ? p.ne[(size_t)r * NM_STRIDE] : 1.0f;
    }
    const float acc = chain_s8<GV_COLS>(x, wp, g.K, 0.f);
    float o = mul(acc, sc);
    if (EPI == EPI_ADD && g.lif.ne) o = mul(o, row_gain);
    if (EPI == EPI_LIF) {
        const LifParams& p = g.lif;
        lif_math(p.spikes, p.lif_scale, p.rho != nullptr, l_beta, l_th, l_rho, l_gain, l_ne, o, lv, ls, la);
        p.v[li] = lv;
        p.s[li] = ls;
        if (p.rho) p.a[li] = la;
    } else {
        if (EPI == EPI_ADD) o = add(before, o);
        *dst = o;
    }
}

// false: shape not covered (the strip and the rows must fit shared memory; N a multiple of 16; 16-byte aligned rows)
// the shared-memory size of the launch, or 0 when the shape is not covered
size_t gemv_smem(const GemmArgs& a, const GemvPro& pro) {
    const int rows = a.M < GV_ROWS ? a.M : GV_ROWS;
    if (pro.kind == PRO_POST && (pro.hs <= 0 || a.K % pro.hs || pro.hs % 4)) return 0;
    size_t aux = pro.kind == PRO_RMS ? (size_t)a.K * sizeof(float) : (pro.kind == PRO_POST && pro.gate) ? (size_t)rows * a.K * sizeof(float) : 0;
    if (pro.kind == PRO_RMS) aux += (size_t)rows * sizeof(float);                       // the rows' norms
    if (pro.kind == PRO_POST) aux += (size_t)rows * (a.K / pro.hs) * sizeof(float);    // the heads' norms
    aux = (aux + 15) & ~(size_t)15;
    const size_t smem = (size_t)a.K * GV_COLS + (size_t)rows * a.K * sizeof(float) + aux;
    if (pro.kind == PRO_RMS && (reinterpret_cast<uintptr_t>(pro.gain) & 15)) return 0;
    if (pro.kind == PRO_POST && pro.gate && ((reinterpret_cast<uintptr_t>(pro.gate) & 15) || pro.ldg % 4)) return 0;
    if (smem > 200 * 1024 || a.N % 16 || a.K % 4 || a.ldw % 16 || a.lda % 4 || (reinterpret_cast<uintptr_t>(a.W) & 15) || (reinterpret_cast<uintptr_t>(a.A) & 15)) return 0;
    return smem;
}

bool launch_gemv(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, const GemvPro& pro = GemvPro()) {
    const size_t smem = gemv_smem(a, pro);
    if (!smem) return false;
    dim3 grid((a.N + GV_COLS - 1) / GV_COLS, (a.M + GV_ROWS - 1) / GV_ROWS);
    auto go = [&](auto kernel) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(kernel, grid, dim3(GV_THREADS), smem, st, a, pro);
    };
    switch (epi) {
        case EPI_STORE: go(q8_gemv_kernel<EPI_STORE>); break;
        case EPI_ADD: go(q8_gemv_kernel<EPI_ADD>); break;
        case EPI_LIF: go(q8_gemv_kernel<EPI_LIF>); break;
    }
    return true;
}

// ---------------------------------------------------------------------------------------------------- event sums
// A mostly-zero row (the LIF spikes, the k-WTA'd MLP units) sums over its non-zero inputs only, in increasing order:
// fma(0, q, acc) = acc exactly, so this is the dense sum bit for bit (src/int8.rs:10-13; -0 counts as zero, NaN does
// not, :261-269).  One block per (row, 256 output columns): the block lists the row's non-zero inputs in order in
// shared memory, then every thread walks the list with four columns' accumulators, eight weight loads in flight.
constexpr int EV_THREADS = 64, EV_COLS = EV_THREADS * 4;

template <int EPI, bool GAIN>
__global__ void __launch_bounds__(EV_THREADS) q8_event_kernel(const GemmArgs g, const MixArgs mx) {
    pdl_enter();
    extern __shared__ unsigned char ev_smem[];
    float* vals = reinterpret_cast<float*>(ev_smem);                  // [K]
    unsigned short* idx = reinterpret_cast<unsigned short*>(vals + g.K);  // [K]
    __shared__ int warp_off[EV_THREADS / 32 + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = blockIdx.z * gridDim.y + blockIdx.y, c0 = blockIdx.x * EV_COLS + tid * 4;  // rows beyond a grid dimension's 65535 go on in z
    if (r >= g.M) return;
    const float* xr = g.A + (size_t)r * g.lda;
    // ordered compaction, coalesced: each warp takes a contiguous part of the row 32 inputs at a time; first the
    // warps count, then each writes its part of the list behind the parts before it
    constexpr int NW = EV_THREADS / 32;
    const int part = ((g.K + NW * 32 - 1) / (NW * 32)) * 32;  // inputs per warp, a multiple of 32
    const int j0 = warp * part, j1 = min(g.K, j0 + part);
    int cnt = 0;
    for (int j = j0 + lane; j < j1; j += 32) cnt += xr[j] != 0.0f;
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) warp_off[warp + 1] = cnt;
    __syncthreads();
    if (tid == 0) {
        warp_off[0] = 0;
        for (int w = 1; w <= NW; ++w) warp_off[w] += warp_off[w - 1];
    }
    __syncthreads();
    int at = warp_off[warp];
    for (int j = j0; j < j1; j += 32) {
        const float v = (j + lane < j1) ? xr[j + lane] : 0.0f;
        const unsigned m = __ballot_sync(0xffffffffu, v != 0.0f);
        if (v != 0.0f) {
            const int pos = at + __popc(m & ((1u << lane) - 1u));
            vals[pos] = v;
            idx[pos] = (unsigned short)(j + lane);
        }
        at += __popc(m);
    }
    __syncthreads();
    const int nnz = warp_off[NW];
    if (c0 >= g.N) return;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int8_t* wp = g.W + c0;
    auto step = [&](int w, float x) {
        float f[4];
        widen4(w, f);
        acc[0] = fma(x, f[0], acc[0]);
        acc[1] = fma(x, f[1], acc[1]);
        acc[2] = fma(x, f[2], acc[2]);
        acc[3] = fma(x, f[3], acc[3]);
    };
    int i = 0;
    if (nnz >= 32) {
        // thirty-two weight words in flight while the thirty-two before them are summed
        int w[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) w[u] = __ldg(reinterpret_cast<const int*>(wp + (size_t)idx[u] * g.ldw));
        for (; i + 64 <= nnz; i += 32) {
            int nx[32];
#pragma unroll
            for (int u = 0; u < 32; ++u) nx[u] = __ldg(reinterpret_cast<const int*>(wp + (size_t)idx[i + 32 + u] * g.ldw));
#pragma unroll
            for (int u = 0; u < 32; ++u) step(w[u], vals[i + u]);
#pragma unroll
            for (int u = 0; u < 32; ++u) w[u] = nx[u];
        }
#pragma unroll
        for (int u = 0; u < 32; ++u) step(w[u], vals[i + u]);
        i += 32;
    }
    for (; i + 4 <= nnz; i += 4) {
        int w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) w[u] = __ldg(reinterpret_cast<const int*>(wp + (size_t)idx[i + u] * g.ldw));
#pragma unroll
        for (int u = 0; u < 4; ++u) step(w[u], vals[i + u]);
    }
    for (; i < nnz; ++i) step(__ldg(reinterpret_cast<const int*>(wp + (size_t)idx[i] * g.ldw)), vals[i]);
    const float4 sc = *reinterpret_cast<const float4*>(g.scale + c0);
    float o[4] = {mul(acc[0], sc.x), mul(acc[1], sc.y), mul(acc[2], sc.z), mul(acc[3], sc.w)};
    if (GAIN) {
        const float rg = g.lif.ne[(size_t)r * NM_STRIDE];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = mul(o[j], rg);
    }
    float4* dst = reinterpret_cast<float4*>(g.C + (size_t)r * g.ldc + c0);
    if (EPI == EPI_ADD) {
        const float4 x = *dst;
        o[0] = add(x.x, o[0]);
        o[1] = add(x.y, o[1]);
        o[2] = add(x.z, o[2]);
        o[3] = add(x.w, o[3]);
    }
    if (EPI == EPI_ADD && mx.streams) {
        // the dense mix (dense_mix_kernel) of these four elements: x + sum_j stream_j w_j in order, the block's output
        // joining the streams; every load before the first store
        const int64_t MD = (int64_t)g.M * g.N, i = (int64_t)r * g.N + c0;
        float mix[4] = {o[0], o[1], o[2], o[3]};
        for (int j = 0; j < mx.n_streams - 1; ++j) {
            const float4 sj = *reinterpret_cast<const float4*>(mx.streams + (int64_t)j * MD + i);
            const float wj = mx.w[j];
            mix[0] = add(mix[0], mul(sj.x, wj));
            mix[1] = add(mix[1], mul(sj.y, wj));
            mix[2] = add(mix[2], mul(sj.z, wj));
            mix[3] = add(mix[3], mul(sj.w, wj));
        }
        const float wl = mx.w[mx.n_streams - 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) mix[j] = add(mix[j], mul(o[j], wl));
        *reinterpret_cast<float4*>(mx.streams + (int64_t)(mx.n_streams - 1) * MD + i) = make_float4(o[0], o[1], o[2], o[3]);
        *dst = make_float4(mix[0], mix[1], mix[2], mix[3]);
        return;
    }
    *dst = make_float4(o[0], o[1], o[2], o[3]);
}

// The event sum for a few rows: one block per (row, 32 output columns).  The block lists the row's non-zero inputs in
// order (eight warps, a contiguous part of the row each), requests the listed weight rows' 32 bytes all at once into
// shared memory (one latency for the whole list instead of one per 32 events), and one warp then walks the list with a
// column per lane.
constexpr int EVS_COLS = 32, EVS_THREADS = 256;

template <int EPI, bool GAIN>
__global__ void __launch_bounds__(EVS_THREADS) q8_event_small_kernel(const GemmArgs g, const MixArgs mx) {
    pdl_enter();
    extern __shared__ __align__(16) unsigned char evs_smem[];
    int8_t* wt = reinterpret_cast<int8_t*>(evs_smem);                                   // [K][32], the first nnz rows used
    float* vals = reinterpret_cast<float*>(evs_smem + (size_t)g.K * EVS_COLS);          // [K]
    unsigned short* idx = reinterpret_cast<unsigned short*>(vals + g.K);                // [K]
    constexpr int NW = EVS_THREADS / 32;
    __shared__ int warp_off[NW + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = blockIdx.y, n0 = blockIdx.x * EVS_COLS;
    const float* xr = g.A + (size_t)r * g.lda;
    if (mx.kw_u) {
        // the row is the k winners of the pre-activations (kwta_kernel's selection and arithmetic), made here
        float* us = reinterpret_cast<float*>(idx + g.K);   // [K]
        uint32_t* keys = reinterpret_cast<uint32_t*>(vals);  // [K], free until the list is written
        __shared__ int hist[256];
        __shared__ int warp_sum[8];
        __shared__ uint32_t sel_prefix;
        __shared__ int sel_k;
        const int n = g.K, k = mx.kw_k;
        const float* ur = mx.kw_u + (size_t)r * n;
        for (int i = tid; i < n; i += EVS_THREADS) us[i] = ur[i];
        __syncthreads();
        if (k >= n) {
            for (int i = tid; i < n; i += EVS_THREADS) {
                const float v = fmaxf(mul(us[i], 1.0f), 0.0f);
                us[i] = mx.kw_relu2 ? mul(v, v) : v;
            }
        } else {
            for (int i = tid; i < n; i += EVS_THREADS) keys[i] = order_key(us[i]);
            uint32_t thr = 0;
            int k_rem = k;
            for (int shift = 24; shift >= 0; shift -= 8) {
                hist[tid] = 0;
                __syncthreads();
                const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
                for (int i = tid; i < n; i += EVS_THREADS) {
                    const uint32_t key = keys[i];
                    if ((key & mask) == thr) atomicAdd(&hist[(key >> shift) & 255u], 1);
                }
                __syncthreads();
                const int h = hist[tid];
                int sfx = h;  // keys in bins tid .. 255
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_down_sync(0xffffffffu, sfx, o);
                    if (lane + o < 32) sfx += up;
                }
                if (lane == 0) warp_sum[warp] = sfx;
                __syncthreads();
                for (int w = warp + 1; w < 8; ++w) sfx += warp_sum[w];
                if (sfx >= k_rem && sfx - h < k_rem) {  // exactly one bin: the suffix sums fall as the bin index rises
                    sel_prefix = thr | ((uint32_t)tid << shift);
                    sel_k = k_rem - (sfx - h);
                }
                __syncthreads();
                thr = sel_prefix;
                k_rem = sel_k;
            }
            const float kth = key_value(thr);
            for (int i = tid; i < n; i += EVS_THREADS) {
                const float v = us[i];
                const float o = fmaxf(mul(v, sub(v, kth) >= 0.0f ? 1.0f : 0.0f), 0.0f);
                us[i] = mx.kw_relu2 ? mul(o, o) : o;
            }
        }
        __syncthreads();
        xr = us;
    }
    const int part = ((g.K + NW * 32 - 1) / (NW * 32)) * 32;  // inputs per warp, a multiple of 32
    const int j0 = min(g.K, warp * part), j1 = min(g.K, j0 + part);
    int cnt = 0;
    for (int j = j0 + lane; j < j1; j += 32) cnt += xr[j] != 0.0f;
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) warp_off[warp + 1] = cnt;
    __syncthreads();
    if (tid == 0) {
        warp_off[0] = 0;
        for (int w = 1; w <= NW; ++w) warp_off[w] += warp_off[w - 1];
    }
    __syncthreads();
    int at = warp_off[warp];
    for (int j = j0; j < j1; j += 32) {
        const float v = (j + lane < j1) ? xr[j + lane] : 0.0f;
        const unsigned m = __ballot_sync(0xffffffffu, v != 0.0f);
        if (v != 0.0f) {
            const int pos = at + __popc(m & ((1u << lane) - 1u));
            vals[pos] = v;
            idx[pos] = (unsigned short)(j + lane);
        }
        at += __popc(m);
    }
    __syncthreads();
    const int nnz = warp_off[NW];
    for (int i = tid; i < nnz * 2; i += EVS_THREADS) {
        const int ev = i >> 1, q = i & 1;
        if (n0 + q * 16 < g.N)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(wt + (size_t)ev * EVS_COLS + q * 16)),
                         "l"(g.W + (size_t)idx[ev] * g.ldw + n0 + q * 16)
                         : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const int c = n0 + lane;
    if (warp != 0 || c >= g.N) return;
    const int8_t* wp = wt + lane;
    // the mix's stream values of this element are requested before the chain, so that their latency passes under it
    constexpr int MIX_PRE = 16;
    float sv[MIX_PRE];
    if (EPI == EPI_ADD && mx.streams) {
        const int64_t MD = (int64_t)g.M * g.N, i = (int64_t)r * g.N + c;
#pragma unroll
        for (int j = 0; j < MIX_PRE; ++j) sv[j] = j < mx.n_streams - 1 ? mx.streams[(int64_t)j * MD + i] : 0.0f;
    }
    // so is everything else the epilogue reads
    const float sc = g.scale[c];
    const float row_gain = GAIN ? g.lif.ne[(size_t)r * NM_STRIDE] : 1.0f;
    float* dst = g.C + (size_t)r * g.ldc + c;
    const float before = EPI == EPI_ADD ? *dst : 0.0f;
    float mw[MIX_PRE + 1];
    if (EPI == EPI_ADD && mx.streams) {
#pragma unroll
        for (int j = 0; j <= MIX_PRE; ++j) mw[j] = j < mx.n_streams ? mx.w[j] : 0.0f;
    }
    const float acc = chain_s8<EVS_COLS>(vals, wp, nnz, 0.f);
    float o = mul(acc, sc);
    if (GAIN) o = mul(o, row_gain);
    if (EPI == EPI_ADD) o = add(before, o);
    if (EPI == EPI_ADD && mx.streams) {
        // the dense mix (dense_mix_kernel): x + sum_j stream_j w_j in order, the block's output joining the streams
        const int64_t MD = (int64_t)g.M * g.N, i = (int64_t)r * g.N + c;
        float mix = o;
        float w_last = 0.0f;
#pragma unroll
        for (int j = 0; j < MIX_PRE; ++j)
            if (j < mx.n_streams - 1) mix = add(mix, mul(sv[j], mw[j]));
#pragma unroll
        for (int j = 0; j <= MIX_PRE; ++j)
            if (j == mx.n_streams - 1) w_last = mw[j];
        mix = add(mix, mul(o, w_last));
        mx.streams[(int64_t)(mx.n_streams - 1) * MD + i] = o;
        o = mix;
    }
    *dst = o;
}

template <int BM, int BN, int TM, int TN>
void launch_tile(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi) {
    dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM);
    dim3 block((BM / TM) * (BN / TN));
    switch (epi) {
        case EPI_STORE: launch_k(q8_gemm_kernel<BM, BN, TM, TN, EPI_STORE>, dim3(grid), dim3(block), 0, st, a); break;
        case EPI_ADD: launch_k(q8_gemm_kernel<BM, BN, TM, TN, EPI_ADD>, dim3(grid), dim3(block), 0, st, a); break;
        case EPI_LIF: launch_k(q8_gemm_kernel<BM, BN, TM, TN, EPI_LIF>, dim3(grid), dim3(block), 0, st, a); break;
    }
}

// --stp: the spikes through the synapse, one thread per (row, channel), the tokens of a chunk in order
__global__ void stp_kernel(const float* spikes, const float* __restrict__ U, const float* __restrict__ F, const float* __restrict__ D,
                           const float* __restrict__ mix, float* u_st, float* x_st, int M, int d, int T, float* out) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t Md = (size_t)M * d;
    if (i >= Md) return;
    const int c = (int)(i % d);
    const float uu = U[c], df = F[c], dd = D[c], mx = mix[c];
    float u = u_st[i], x = x_st[i];
    for (int t = 0; t < T; ++t) {
        const float sv = spikes[(size_t)t * Md + i];
        // the event size: s k + (clamp(|s|, 0, 1) - s k), k = 1 on [0, 1], -1 on [-1, 0), 0 beyond (nn/parts/src/stp.rs:42-54)
        const float k = ((sv >= 0.0f && sv <= 1.0f) ? 1.0f : 0.0f) - ((sv < 0.0f && sv >= -1.0f) ? 1.0f : 0.0f);
        const float sk = mul(sv, k);
        const float a = fminf(fmaxf(fabsf(sv), 0.0f), 1.0f);
        const float ev = add(sk, sub(a, sk));
        const float u_plus = add(u, mul(mul(add(mul(u, -1.0f), 1.0f), uu), ev));
        const float e = mul(u_plus, x);
        const float eff = div(e, uu);
        const float x_used = sub(x, mul(e, ev));
        u = mul(u_plus, df);
        x = add(mul(mul(add(mul(x_used, -1.0f), 1.0f), dd), -1.0f), 1.0f);
        out[(size_t)t * Md + i] = add(sv, mul(sub(mul(sv, eff), sv), mx));
    }
    u_st[i] = u;
    x_st[i] = x;
}

__global__ void fill_kernel(float* p, int64_t n, float v) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

__global__ void lif_kernel(const float* cur, const LifParams p, int M, int d) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * d) return;
    lif_update(p, (int)(i / d), (int)(i % d), d, cur[i]);
}

}  // namespace

int g_gemm_force = 0;  // tuning override (0: choose by shape)
int g_gemv_max_rows = 8;       // up to this many rows the one-column-per-lane kernel takes the dense products
int g_resident_max_rows = 16;  // up to this many rows the resident-tile kernel takes the dense products (measured: 19-21 us
                                // against 23 us for the tiled kernel at 1-8 rows, slower from 32 rows on)
thread_local cudaError_t g_launch_error = cudaSuccess;
int g_pdl = 1;         // programmatic dependent launch on every kernel of the step (kernels.cuh)

void prefer_max_shared(const void* kernel, int percent_for_this) {
    // once per kernel and device (a handful of kernels: a linear scan of a small table)
    struct Seen { const void* k; int dev; };
    static Seen seen[512];
    static int n = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    for (int i = 0; i < n; ++i)
        if (seen[i].k == kernel && seen[i].dev == dev) return;
    // half of it as shared memory: measured best for the step as a whole (all of it starves the kernels that lean on L1)
    const int percent = 50;
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, percent_for_this >= 0 ? percent_for_this : percent);
    if (n < 512) seen[n++] = {kernel, dev};
}

int gemv_max_rows() { return g_gemm_force == 0 ? g_gemv_max_rows : 0; }

bool q8_gemv_pro_covers(const GemmArgs& a, const GemvPro& pro) { return a.M <= gemv_max_rows() && gemv_smem(a, pro) != 0; }

bool launch_q8_gemv_pro(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, const GemvPro& pro) {
    return a.M <= gemv_max_rows() && launch_gemv(st, a, epi, pro);
}

void launch_q8_gemm(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, int sm_count) {
    switch (g_gemm_force) {
        case 1: return launch_tile<64, 64, 4, 4>(st, a, epi);
        case 2: return launch_tile<64, 64, 8, 4>(st, a, epi);
        case 3: return launch_tile<32, 64, 4, 4>(st, a, epi);
        case 4: return launch_tile<32, 64, 4, 2>(st, a, epi);
        case 6:
            if (launch_resident(st, a, epi)) return;
            break;
        default: break;
    }
    // one sequence or a handful: a column per lane, the weights' strip requested before the wait for the kernel before
    if (g_gemm_force == 0 && a.M <= g_gemv_max_rows && launch_gemv(st, a, epi)) return;
    // a few rows: the whole-K tile in shared memory, one latency instead of one per k-tile
    if (g_gemm_force == 0 && a.M <= g_resident_max_rows && launch_resident(st, a, epi)) return;
    // Measured on B200 at 256 rows (the machine is short of warps at this batch, so the choice is about filling SMs):
    // very wide products take 64x64 tiles of 8x4, wide ones 64x64 of 4x4, then 32x64 of 4x4, narrow ones 32x64 of 4x2.
    const long tiles64 = (long)((a.N + 63) / 64) * ((a.M + 63) / 64);
    if (tiles64 >= 4L * sm_count)
        launch_tile<64, 64, 8, 4>(st, a, epi);
    else if (2 * tiles64 >= 3L * sm_count)
        launch_tile<64, 64, 4, 4>(st, a, epi);
    else if (tiles64 >= sm_count)
        launch_tile<32, 64, 4, 4>(st, a, epi);
    else
        launch_tile<32, 64, 4, 2>(st, a, epi);
}

bool event_small_covers(const GemmArgs& a, GemmEpilogue epi) {
    // (the k winners' copy of the row is counted in: K * 4 bytes more)
    const size_t smem_small = (size_t)a.K * (2 * sizeof(float) + sizeof(unsigned short) + EVS_COLS);
    return epi != EPI_LIF && a.K <= 65535 && a.M <= g_gemv_max_rows && smem_small <= 200 * 1024 && a.N % 16 == 0 && a.ldw % 16 == 0 && a.K % 4 == 0 &&
           !(reinterpret_cast<uintptr_t>(a.W) & 15);
}

bool event_takes_mix(const GemmArgs& a, GemmEpilogue epi, int n_streams) {
    // either event kernel takes it: the few-row one keeps up to 16 stream values in registers, the other walks the streams
    if (epi != EPI_ADD || n_streams < 1 || a.K > 65535 || a.ldc != a.N || a.N % 4) return false;
    const size_t smem = (size_t)a.K * (sizeof(float) + sizeof(unsigned short));
    if (smem > 200 * 1024) return false;
    return event_small_covers(a, epi) ? n_streams - 1 <= 16 : true;
}

bool launch_q8_event(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, const MixArgs* mix) {
    if (a.K > 65535 || epi == EPI_LIF) return false;
    const size_t smem = (size_t)a.K * (sizeof(float) + sizeof(unsigned short));
    if (smem > 200 * 1024) return false;
    const size_t smem_small = smem + (size_t)a.K * EVS_COLS + (mix && mix->kw_u ? (size_t)a.K * sizeof(float) : 0);
    if (mix && mix->kw_u && !event_small_covers(a, epi)) return false;   // only the kernel for a few rows makes the k winners itself
    if (event_small_covers(a, epi)) {
        dim3 grid((a.N + EVS_COLS - 1) / EVS_COLS, a.M);
        MixArgs mx;
        if (mix && mix->streams && event_takes_mix(a, epi, mix->n_streams)) mx = *mix;
        if (mix && mix->kw_u) {
            mx.kw_u = mix->kw_u;
            mx.kw_k = mix->kw_k;
            mx.kw_relu2 = mix->kw_relu2;
        } else {
            mx.kw_u = nullptr;
        }
        auto go = [&](auto kernel) {
            if (smem_small > 32 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_small);
            launch_k(kernel, dim3(grid), dim3(EVS_THREADS), smem_small, st, a, mx);
        };
        if (epi == EPI_ADD && a.lif.ne)
            go(q8_event_small_kernel<EPI_ADD, true>);
        else if (epi == EPI_ADD)
            go(q8_event_small_kernel<EPI_ADD, false>);
        else
            go(q8_event_small_kernel<EPI_STORE, false>);
        return true;
    }
    const int gy = std::min(a.M, 32768);
    dim3 grid((a.N + EV_COLS - 1) / EV_COLS, gy, (a.M + gy - 1) / gy);
    MixArgs mx;
    if (mix && mix->streams && event_takes_mix(a, epi, mix->n_streams)) mx = *mix;
    auto go = [&](auto kernel) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(kernel, dim3(grid), dim3(EV_THREADS), smem, st, a, mx);
    };
    if (epi == EPI_ADD && a.lif.ne)
        go(q8_event_kernel<EPI_ADD, true>);
    else if (epi == EPI_ADD)
        go(q8_event_kernel<EPI_ADD, false>);
    else
        go(q8_event_kernel<EPI_STORE, false>);
    return true;
}

void launch_lif_scan(cudaStream_t st, const float* cur, const LifParams& p, int M, int d, int T, float* spikes, const float* cur_gain) {
    const size_t n = (size_t)M * d;
    launch_k(lif_scan_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, st, cur, p, M, d, T, spikes, cur_gain);
}

void launch_stp(cudaStream_t st, const float* spikes, const float* U, const float* F, const float* D, const float* mix, float* u, float* x, int M, int d,
                int T, float* out) {
    const size_t n = (size_t)M * d;
    launch_k(stp_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, spikes, U, F, D, mix, u, x, M, d, T, out);
}

void launch_fill(cudaStream_t st, float* p, int64_t n, float v) {
    launch_k(fill_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, p, n, v);
}

void launch_lif(cudaStream_t st, const float* cur, const LifParams& p, int M, int d) {
    const size_t n = (size_t)M * d;
    launch_k(lif_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, cur, p, M, d);
}

}  // namespace ava

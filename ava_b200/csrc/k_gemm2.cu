// The dense int8-weight products for a batch of rows, second form (sm_100a, CUDA cores, packed f32x2 multiply-adds).
//
// Same arithmetic as k_gemm.cu: y[r][c] = scale[c] * (fma chain over k = 0, 1, ... from +0 of x[r][k] * (f32) q[k][c]),
// the reference's order (design-tests/nn/gpu/src/int8.rs:315-331), so the same bits.  What changes is how the operands
// reach the multiply-add units.  An SM can bring 32 words per clock from shared memory into registers and do 128
// multiply-adds per clock, so every word fetched has to serve four multiply-adds or more.  Here
//   * the weights stay int8 in shared memory: one 32-bit word holds a thread's four neighbouring columns of one k and is
//     widened in registers (byte permute + one packed subtract), so a TM x 4 block of outputs costs TM + 1 words per k;
//   * the multiply-adds are issued as fma.rn.f32x2 (two IEEE fused multiply-adds per instruction: the same roundings
//     as two scalar ones), which halves the issue slots the sums take and leaves room for the widening;
//   * tiles arrive by cp.async in a four-stage ring, 32 k per stage: one barrier per 32 k.
#include <cstdlib>

#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int G2_BK = 32;
constexpr int G2_STAGES = 4;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// four int8 in a word -> two packed float pairs, exactly: byte + 128 in the mantissa of 2^23, minus (2^23 + 128)
__device__ __forceinline__ void widen4x2(int w, float2& lo, float2& hi) {
    const unsigned u = (unsigned)w ^ 0x80808080u;
    const float2 m = make_float2(-8388736.0f, -8388736.0f);
    lo = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)), __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441))), m);
    hi = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)), __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443))), m);
}

// One LIF update (the same function as in k_gemm.cu; src/model/fstep/arch.rs:173-228)
__device__ __forceinline__ void lif_math2(int spikes, int lif_scale, bool adaptive, float beta, float th, float rho, float gain, float ne, float cur, float& v,
                                          float& s, float& a) {
    if (lif_scale) cur = mul(cur, add(mul(beta, -1.0f), 1.0f));
    cur = mul(cur, ne);
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

// Block tile BM x BN, thread tile TM x TN (TN = 4 or 8: one or two packed words of weights per k).
template <int BM, int BN, int TM, int TN, int EPI>
__global__ void __launch_bounds__((BM / TM) * (BN / TN)) q8_gemm2_kernel(const GemmArgs g) {
    pdl_enter();
    static_assert(TN == 4 || TN == 8, "thread tile width");
    constexpr int TX = BN / TN, TY = BM / TM, NT = TX * TY;
    constexpr int AP = G2_BK + 4;  // floats per staged A row: rows stay 16-byte aligned, neighbours fall in other banks
    constexpr int WQ = TN / 4;
    constexpr int A_STAGE = BM * AP;            // floats
    constexpr int W_STAGE = G2_BK * BN;         // bytes
    extern __shared__ __align__(16) unsigned char g2_smem[];
    float* As = reinterpret_cast<float*>(g2_smem);
    int8_t* Ws = reinterpret_cast<int8_t*>(As + G2_STAGES * A_STAGE);

    const int tid = threadIdx.x;
    const int tx = tid % TX, ty = tid / TX;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nk = g.K / G2_BK;

    auto load_stage = [&](int kt, int s) {
        constexpr int AC = BM * (G2_BK / 4);  // 16-byte pieces of the A tile
        float* as = As + s * A_STAGE;
#pragma unroll
        for (int i = 0; i < (AC + NT - 1) / NT; ++i) {
            const int idx = tid + i * NT;
            if (AC % NT == 0 || idx < AC) {
                const int row = idx / (G2_BK / 4), c = idx % (G2_BK / 4);
                const int r = m0 + row < g.M ? m0 + row : g.M - 1;
                cp_async16(as + row * AP + c * 4, g.A + (size_t)r * g.lda + kt * G2_BK + c * 4);
            }
        }
        constexpr int WC = G2_BK * (BN / 16);
        int8_t* ws = Ws + s * W_STAGE;
#pragma unroll
        for (int i = 0; i < (WC + NT - 1) / NT; ++i) {
            const int idx = tid + i * NT;
            if (WC % NT == 0 || idx < WC) {
                const int k = idx / (BN / 16), c = idx % (BN / 16);
                const int col = n0 + c * 16 < g.N ? n0 + c * 16 : 0;
                cp_async16(ws + k * BN + c * 16, g.W + (size_t)(kt * G2_BK + k) * g.ldw + col);
            }
        }
    };

    float2 acc[TM][TN / 2];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) acc[i][j] = make_float2(0.0f, 0.0f);

#pragma unroll
    for (int s = 0; s < G2_STAGES - 1; ++s) {
        if (s < nk) load_stage(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < nk; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(G2_STAGES - 2) : "memory");
        __syncthreads();  // tile kt has landed for every thread, and everyone is done with tile kt - 1
        if (kt + G2_STAGES - 1 < nk) load_stage(kt + G2_STAGES - 1, (kt + G2_STAGES - 1) % G2_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const float* as = As + (kt % G2_STAGES) * A_STAGE + (ty * TM) * AP;
        const int* ws = reinterpret_cast<const int*>(Ws + (kt % G2_STAGES) * W_STAGE) + tx * WQ;
#pragma unroll
        for (int k4 = 0; k4 < G2_BK / 4; ++k4) {
            float4 a4[TM];
#pragma unroll
            for (int i = 0; i < TM; ++i) a4[i] = *reinterpret_cast<const float4*>(as + i * AP + k4 * 4);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                float2 wf[TN / 2];
#pragma unroll
                for (int q = 0; q < WQ; ++q) widen4x2(ws[(k4 * 4 + kk) * (BN / 4) + q], wf[2 * q], wf[2 * q + 1]);
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const float a = kk == 0 ? a4[i].x : kk == 1 ? a4[i].y : kk == 2 ? a4[i].z : a4[i].w;
                    const float2 a2 = make_float2(a, a);
#pragma unroll
                    for (int j = 0; j < TN / 2; ++j) acc[i][j] = __ffma2_rn(a2, wf[j], acc[i][j]);
                }
            }
        }
    }

    const int c0 = n0 + tx * TN;
    if (c0 >= g.N) return;
    float accs[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) {
            accs[i][2 * j] = acc[i][j].x;
            accs[i][2 * j + 1] = acc[i][j].y;
        }
    float scv[TN];
#pragma unroll
    for (int j = 0; j < TN; j += 4) {
        const float4 s4 = *reinterpret_cast<const float4*>(g.scale + c0 + j);
        scv[j] = s4.x; scv[j + 1] = s4.y; scv[j + 2] = s4.z; scv[j + 3] = s4.w;
    }
    const int r0 = m0 + ty * TM;
    if (EPI == EPI_LIF) {
        // the carried state of the whole thread tile is read before any of it is written (a store would otherwise fence
        // the next element's loads)
        const LifParams& p = g.lif;
        float lbeta[TN], lth[TN], lrho[TN], lgain[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            lbeta[j] = p.beta[c0 + j];
            lth[j] = p.theta ? p.theta[c0 + j] : 1.0f;
            lrho[j] = p.rho ? p.rho[c0 + j] : 0.0f;
            lgain[j] = p.rho ? p.gain[c0 + j] : 0.0f;
        }
        float v[TM][TN], sp[TM][TN], tr[TM][TN], lne[TM];
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = r0 + i < g.M ? r0 + i : g.M - 1;
            lne[i] = p.ne ? p.ne[(size_t)r * NM_STRIDE] : 1.0f;
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const size_t at = (size_t)r * g.N + c0 + j;
                const float4 v4 = *reinterpret_cast<const float4*>(p.v + at), s4 = *reinterpret_cast<const float4*>(p.s + at);
                v[i][j] = v4.x; v[i][j + 1] = v4.y; v[i][j + 2] = v4.z; v[i][j + 3] = v4.w;
                sp[i][j] = s4.x; sp[i][j + 1] = s4.y; sp[i][j + 2] = s4.z; sp[i][j + 3] = s4.w;
                if (p.rho) {
                    const float4 a4 = *reinterpret_cast<const float4*>(p.a + at);
                    tr[i][j] = a4.x; tr[i][j + 1] = a4.y; tr[i][j + 2] = a4.z; tr[i][j + 3] = a4.w;
                } else {
                    tr[i][j] = tr[i][j + 1] = tr[i][j + 2] = tr[i][j + 3] = 0.0f;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j)
                lif_math2(p.spikes, p.lif_scale, p.rho != nullptr, lbeta[j], lth[j], lrho[j], lgain[j], lne[i], mul(accs[i][j], scv[j]), v[i][j], sp[i][j],
                          tr[i][j]);
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            if (r0 + i >= g.M) continue;
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const size_t at = (size_t)(r0 + i) * g.N + c0 + j;
                *reinterpret_cast<float4*>(p.v + at) = make_float4(v[i][j], v[i][j + 1], v[i][j + 2], v[i][j + 3]);
                *reinterpret_cast<float4*>(p.s + at) = make_float4(sp[i][j], sp[i][j + 1], sp[i][j + 2], sp[i][j + 3]);
                if (p.rho) *reinterpret_cast<float4*>(p.a + at) = make_float4(tr[i][j], tr[i][j + 1], tr[i][j + 2], tr[i][j + 3]);
            }
        }
        return;
    }
    float resid[TM][TN];
    if (EPI == EPI_ADD) {
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int r = r0 + i < g.M ? r0 + i : g.M - 1;
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const float4 x = *reinterpret_cast<const float4*>(g.C + (size_t)r * g.ldc + c0 + j);
                resid[i][j] = x.x; resid[i][j + 1] = x.y; resid[i][j + 2] = x.z; resid[i][j + 3] = x.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = r0 + i;
        if (r >= g.M) continue;
        float o[TN];
#pragma unroll
        for (int j = 0; j < TN; ++j) o[j] = mul(accs[i][j], scv[j]);
        if (EPI == EPI_ADD && g.lif.ne) {
            const float rg = g.lif.ne[(size_t)r * NM_STRIDE];
#pragma unroll
            for (int j = 0; j < TN; ++j) o[j] = mul(o[j], rg);
        }
        if (EPI == EPI_ADD) {
#pragma unroll
            for (int j = 0; j < TN; ++j) o[j] = add(resid[i][j], o[j]);
        }
#pragma unroll
        for (int j = 0; j < TN; j += 4) *reinterpret_cast<float4*>(g.C + (size_t)r * g.ldc + c0 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
    }
}

template <int BM, int BN, int TM, int TN>
void launch_tile2(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi) {
    constexpr size_t smem = (size_t)G2_STAGES * (BM * (G2_BK + 4) * sizeof(float) + G2_BK * BN);
    dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM);
    dim3 block((BM / TM) * (BN / TN));
    auto go = [&](auto kernel) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(kernel, grid, block, smem, st, a);
    };
    switch (epi) {
        case EPI_STORE: go(q8_gemm2_kernel<BM, BN, TM, TN, EPI_STORE>); break;
        case EPI_ADD: go(q8_gemm2_kernel<BM, BN, TM, TN, EPI_ADD>); break;
        case EPI_LIF: go(q8_gemm2_kernel<BM, BN, TM, TN, EPI_LIF>); break;
    }
}

}  // namespace

int g_gemm2_force = 0;  // tuning override (0: choose by shape)

// false: shape not covered (K a multiple of 32, N of 16, 16-byte aligned rows of A and W)
bool launch_q8_gemm2(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, int sm_count) {
    if (a.K % G2_BK || a.N % 16 || a.ldw % 16 || a.lda % 4 || a.ldc % 4 || a.M < 1) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.W) | reinterpret_cast<uintptr_t>(a.C) | reinterpret_cast<uintptr_t>(a.scale)) & 15) return false;
    switch (g_gemm2_force) {
        case 1: launch_tile2<64, 64, 8, 4>(st, a, epi); return true;
        case 2: launch_tile2<128, 64, 8, 4>(st, a, epi); return true;
        case 3: launch_tile2<64, 128, 8, 8>(st, a, epi); return true;
        case 4: launch_tile2<32, 64, 4, 4>(st, a, epi); return true;
        case 5: launch_tile2<64, 32, 8, 4>(st, a, epi); return true;
        case 6: launch_tile2<32, 128, 4, 4>(st, a, epi); return true;
        case 7: launch_tile2<64, 64, 4, 4>(st, a, epi); return true;
        case 8: launch_tile2<128, 128, 8, 8>(st, a, epi); return true;
        case 9: launch_tile2<32, 32, 4, 4>(st, a, epi); return true;
        default: break;
    }
    (void)sm_count;
    // Measured on B200 (one decode step's products are short of warps, so the choice is about filling the SMs; the
    // wide-tile forms win once there are rows enough):
    //   thousands of rows (a prompt chunk): 64x128 tiles of 8x8 (the LIF epilogue keeps 8x4);
    //   129..1023 rows: very wide products 64x64 of 8x4, wide ones 128x64 of 8x4, the rest 32x64 of 4x4;
    //   65..128 rows: wide products 64x64 of 8x4, narrow ones 32x64 of 4x4;  up to 64 rows: 32x32 of 4x4 when wide.
    if (a.M >= 1024) {
        if (epi == EPI_LIF) launch_tile2<64, 64, 8, 4>(st, a, epi); else launch_tile2<64, 128, 8, 8>(st, a, epi);
    } else if (a.M > 128) {
        if (a.N >= 8192) launch_tile2<64, 64, 8, 4>(st, a, epi);
        else if (a.N >= 3584) launch_tile2<128, 64, 8, 4>(st, a, epi);
        else launch_tile2<32, 64, 4, 4>(st, a, epi);
    } else if (a.M > 64) {
        if (a.N >= 1024) launch_tile2<64, 64, 8, 4>(st, a, epi); else launch_tile2<32, 64, 4, 4>(st, a, epi);
    } else {
        if (a.N >= 1024) launch_tile2<32, 32, 4, 4>(st, a, epi); else launch_tile2<32, 64, 4, 4>(st, a, epi);
    }
    return true;
}

}  // namespace ava

// The int8-weight products of the block step for a batch of rows (sm_100a, CUDA cores).
//
// The reference keeps activations in f32 and sums x[j] * (f32) q[j][c] with one fused multiply-add per term in the
// order j = 0, 1, ..., d_in - 1 from +0, then multiplies by the column's scale (design-tests/nn/gpu/src/int8.rs:3-8,
// 315-331).  Any other summation order rounds differently, and one flipped spike or k-WTA winner sends a spiking
// model down another path, so this kernel keeps that order: each thread owns a 4x4 block of outputs and walks k
// upwards, never splitting K.  The int8 tile is widened to f32 once when it is staged in shared memory and reused by
// every row of the tile.
#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int BK = 16;

__device__ __forceinline__ void lif_update(const LifParams& p, int r, int c, int d, float cur) {
    // src/model/fstep/arch.rs:173-228 with the hard spike count taken directly (as the reference's own GPU kernel
    // does; the CPU's soft + (hard - soft) equals it).
    const float beta = p.beta[c];
    if (p.lif_scale) cur = mul(cur, add(mul(beta, -1.0f), 1.0f));
    const size_t i = (size_t)r * d + c;
    const float th = p.theta ? p.theta[c] : 1.0f;
    const float v0 = p.v[i], s0 = p.s[i];
    float th_prev = th, th_t = th;
    if (p.rho) {
        const float a_prev = p.a[i];
        const float rho = p.rho[c], gain = p.gain[c];
        th_prev = add(th, mul(a_prev, gain));
        const float an = add(mul(a_prev, rho), mul(fabsf(s0), add(mul(rho, -1.0f), 1.0f)));
        p.a[i] = an;
        th_t = add(th, mul(an, gain));
    }
    const float vv = sub(add(mul(v0, beta), cur), mul(s0, th_prev));
    p.v[i] = vv;
    float s;
    if (p.spikes == 0) {
        s = sub(vv, th_t) >= 0.0f ? 1.0f : 0.0f;
    } else {
        const int levels = p.spikes == 2 ? 2 : 1;
        s = 0.0f;
        for (int k = 1; k <= levels; ++k) {
            const float kth = add(mul(th_t, (float)k), 0.0f);
            const float up = sub(vv, kth), down = sub(-vv, kth);
            s += (up >= 0.0f ? 1.0f : 0.0f) - (down >= 0.0f ? 1.0f : 0.0f);
        }
    }
    p.s[i] = s;
}

template <int BM, int BN, int EPI>
__global__ void __launch_bounds__((BM / 4) * (BN / 4)) q8_gemm_kernel(const GemmArgs g) {
    constexpr int T = (BM / 4) * (BN / 4);
    constexpr int AS = BM + 4;  // padded row length of the k-major A tile
    __shared__ __align__(16) float As[2][BK][AS];
    __shared__ __align__(16) float Ws[2][BK][BN];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / 4), ty = tid / (BN / 4);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nk = g.K / BK;

    constexpr int A_LOADS = (BM * 4 + T - 1) / T;   // float4 per thread
    constexpr int W_LOADS = (BN * 4 + T - 1) / T;   // char4 per thread
    constexpr int PF = 4;                           // tiles fetched ahead into registers (global latency cover)
    float4 ra[PF][A_LOADS];
    int rw[PF][W_LOADS];

    auto load_global = [&](int kt, float4* fa, int* fw) {
#pragma unroll
        for (int i = 0; i < A_LOADS; ++i) {
            const int idx = tid + i * T;
            const int row = idx >> 2, kq = idx & 3;
            fa[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (kt < nk && idx < BM * 4 && m0 + row < g.M)
                fa[i] = *reinterpret_cast<const float4*>(g.A + (size_t)(m0 + row) * g.lda + kt * BK + kq * 4);
        }
#pragma unroll
        for (int i = 0; i < W_LOADS; ++i) {
            const int idx = tid + i * T;
            const int k = idx / (BN / 4), n4 = idx % (BN / 4);
            fw[i] = 0;
            if (kt < nk && idx < BN * 4 && n0 + n4 * 4 < g.N)
                fw[i] = __ldg(reinterpret_cast<const int*>(g.W + (size_t)(kt * BK + k) * g.ldw + n0 + n4 * 4));
        }
    };
    auto store_smem = [&](int buf, const float4* fa, const int* fw) {
#pragma unroll
        for (int i = 0; i < A_LOADS; ++i) {
            const int idx = tid + i * T;
            const int row = idx >> 2, kq = idx & 3;
            if (idx < BM * 4) {
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
            if (idx < BN * 4) {
                const int w = fw[i];
                float4 f;
                f.x = (float)(int8_t)(w & 0xff);
                f.y = (float)(int8_t)((w >> 8) & 0xff);
                f.z = (float)(int8_t)((w >> 16) & 0xff);
                f.w = (float)(int8_t)((w >> 24) & 0xff);
                *reinterpret_cast<float4*>(&Ws[buf][k][n4 * 4]) = f;
            }
        }
    };

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

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
#pragma unroll
                for (int k = 0; k < BK; ++k) {
                    const float4 a = *reinterpret_cast<const float4*>(&As[s & 1][k][ty * 4]);
                    const float4 b = *reinterpret_cast<const float4*>(&Ws[s & 1][k][tx * 4]);
                    const float av[4] = {a.x, a.y, a.z, a.w};
                    const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[i][j] = fma(av[i], bv[j], acc[i][j]);
                }
                if (kt + 1 < nk) store_smem((s + 1) & 1, ra[(s + 1) % PF], rw[(s + 1) % PF]);
                __syncthreads();
            }
        }
    }

    const int c0 = n0 + tx * 4;
    if (c0 >= g.N) return;
    const float4 sc = *reinterpret_cast<const float4*>(g.scale + c0);
    const float scv[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r >= g.M) continue;
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = mul(acc[i][j], scv[j]);
        if (EPI == EPI_LIF) {
#pragma unroll
            for (int j = 0; j < 4; ++j) lif_update(g.lif, r, c0 + j, g.N, o[j]);
        } else {
            float4* dst = reinterpret_cast<float4*>(g.C + (size_t)r * g.ldc + c0);
            if (EPI == EPI_ADD) {
                const float4 x = *dst;
                o[0] = add(x.x, o[0]);
                o[1] = add(x.y, o[1]);
                o[2] = add(x.z, o[2]);
                o[3] = add(x.w, o[3]);
            }
            *dst = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------- event sums
// A mostly-zero row (the LIF spikes, the k-WTA'd MLP units) sums over its non-zero inputs only, in increasing order:
// fma(0, q, acc) = acc exactly, so this is the dense sum bit for bit (src/int8.rs:10-13; -0 counts as zero, NaN does
// not, :261-269).  One block per (row, 256 output columns): the block lists the row's non-zero inputs in order in
// shared memory, then every thread walks the list with four columns' accumulators, eight weight loads in flight.
constexpr int EV_THREADS = 64, EV_COLS = EV_THREADS * 4;

template <int EPI>
__global__ void __launch_bounds__(EV_THREADS) q8_event_kernel(const GemmArgs g) {
    extern __shared__ unsigned char ev_smem[];
    float* vals = reinterpret_cast<float*>(ev_smem);                  // [K]
    unsigned short* idx = reinterpret_cast<unsigned short*>(vals + g.K);  // [K]
    __shared__ int warp_off[EV_THREADS / 32 + 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = blockIdx.y, c0 = blockIdx.x * EV_COLS + tid * 4;
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
        acc[0] = fma(x, (float)(int8_t)(w & 0xff), acc[0]);
        acc[1] = fma(x, (float)(int8_t)((w >> 8) & 0xff), acc[1]);
        acc[2] = fma(x, (float)(int8_t)((w >> 16) & 0xff), acc[2]);
        acc[3] = fma(x, (float)(int8_t)((w >> 24) & 0xff), acc[3]);
    };
    int i = 0;
    for (; i + 32 <= nnz; i += 32) {
        int w[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) w[u] = __ldg(reinterpret_cast<const int*>(wp + (size_t)idx[i + u] * g.ldw));
#pragma unroll
        for (int u = 0; u < 32; ++u) step(w[u], vals[i + u]);
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
    float4* dst = reinterpret_cast<float4*>(g.C + (size_t)r * g.ldc + c0);
    if (EPI == EPI_ADD) {
        const float4 x = *dst;
        o[0] = add(x.x, o[0]);
        o[1] = add(x.y, o[1]);
        o[2] = add(x.z, o[2]);
        o[3] = add(x.w, o[3]);
    }
    *dst = make_float4(o[0], o[1], o[2], o[3]);
}

template <int BM, int BN>
void launch_tile(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi) {
    dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM);
    dim3 block((BM / 4) * (BN / 4));
    switch (epi) {
        case EPI_STORE: q8_gemm_kernel<BM, BN, EPI_STORE><<<grid, block, 0, st>>>(a); break;
        case EPI_ADD: q8_gemm_kernel<BM, BN, EPI_ADD><<<grid, block, 0, st>>>(a); break;
        case EPI_LIF: q8_gemm_kernel<BM, BN, EPI_LIF><<<grid, block, 0, st>>>(a); break;
    }
}

__global__ void lif_kernel(const float* cur, const LifParams p, int M, int d) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * d) return;
    lif_update(p, (int)(i / d), (int)(i % d), d, cur[i]);
}

}  // namespace

void launch_q8_gemm(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi, int sm_count) {
    // 64x64 tiles when they fill the SMs, else 32x64 so that a narrow product still spreads out
    const long tiles64 = (long)((a.N + 63) / 64) * ((a.M + 63) / 64);
    if (tiles64 >= sm_count)
        launch_tile<64, 64>(st, a, epi);
    else
        launch_tile<32, 64>(st, a, epi);
}

bool launch_q8_event(cudaStream_t st, const GemmArgs& a, GemmEpilogue epi) {
    if (a.K > 65535 || epi == EPI_LIF) return false;
    const size_t smem = (size_t)a.K * (sizeof(float) + sizeof(unsigned short));
    if (smem > 200 * 1024) return false;
    dim3 grid((a.N + EV_COLS - 1) / EV_COLS, a.M);
    if (epi == EPI_ADD) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(q8_event_kernel<EPI_ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        q8_event_kernel<EPI_ADD><<<grid, EV_THREADS, smem, st>>>(a);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(q8_event_kernel<EPI_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        q8_event_kernel<EPI_STORE><<<grid, EV_THREADS, smem, st>>>(a);
    }
    return true;
}

void launch_lif(cudaStream_t st, const float* cur, const LifParams& p, int M, int d) {
    const size_t n = (size_t)M * d;
    lif_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(cur, p, M, d);
}

}  // namespace ava

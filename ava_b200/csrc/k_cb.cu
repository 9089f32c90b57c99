// --cerebellum-head: the correction of the final normed state before the head (src/model/fstep/arch_f3.rs:207-283,
// src/v51b.rs:327-360).  Per token-row: G granule units each sum four fixed inputs of [xf, rmsnorm(embedding)] (from 0,
// in order), the top G/32 are kept and rectified (the k-WTA kernel), the code is brought to unit length with its squares
// summed in unit order, and the kept units' rows of the read-out are summed per channel in unit order.
#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

__global__ void cb_gather_kernel(const float* __restrict__ tok_emb, const uint32_t* __restrict__ tok, int R, int d, int V, float* __restrict__ out) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * d) return;
    const uint32_t t = tok[i / d];
    out[i] = t < (uint32_t)V ? tok_emb[(size_t)t * d + i % d] : 0.0f;  // a bad id was already reported by the embedding kernel
}

__global__ void cb_units_kernel(const float* __restrict__ xf, const float* __restrict__ en, const uint32_t* __restrict__ idx,
                                const float* __restrict__ sgn, int g, int d, int R, float* __restrict__ h) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * g) return;
    const size_t r = i / g;
    const int j = (int)(i % g);
    const uint4 ix = *reinterpret_cast<const uint4*>(idx + (size_t)j * 4);
    const float4 w = *reinterpret_cast<const float4*>(sgn + (size_t)j * 4);
    auto in = [&](uint32_t q) { return q < (uint32_t)d ? xf[r * d + q] : en[r * d + (q - d)]; };
    float s = 0.0f;
    s = add(s, mul(in(ix.x), w.x));
    s = add(s, mul(in(ix.y), w.y));
    s = add(s, mul(in(ix.z), w.z));
    s = add(s, mul(in(ix.w), w.w));
    h[i] = s;
}

constexpr int CB_THREADS = 256;

// one block per token-row: the non-zero units in unit order (their indices and values), then the code a / len with
// len = sqrt(sum of squares in unit order) * 1 + 1e-6
__global__ void __launch_bounds__(CB_THREADS) cb_code_kernel(const float* __restrict__ a, int g, int* __restrict__ list_j, float* __restrict__ list_c,
                                                             int* __restrict__ count) {
    pdl_enter();
    __shared__ int part[CB_THREADS + 1];
    __shared__ float s_len;
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* ar = a + (size_t)r * g;
    int* lj = list_j + (size_t)r * g;
    float* lc = list_c + (size_t)r * g;
    const int per = (g + CB_THREADS - 1) / CB_THREADS, i0 = tid * per, i1 = min(g, i0 + per);
    int c = 0;
    for (int i = i0; i < i1; ++i) c += ar[i] != 0.0f;
    part[tid + 1] = c;
    __syncthreads();
    if (tid == 0) {
        part[0] = 0;
        for (int t = 1; t <= CB_THREADS; ++t) part[t] += part[t - 1];
    }
    __syncthreads();
    int at = part[tid];
    for (int i = i0; i < i1; ++i) {
        const float v = ar[i];
        if (v != 0.0f) {
            lj[at] = i;
            lc[at] = v;
            ++at;
        }
    }
    __syncthreads();
    const int n = part[CB_THREADS];
    if (tid == 0) {
        float s2 = 0.0f;
        for (int i = 0; i < n; ++i) s2 = add(s2, mul(lc[i], lc[i]));
        s_len = add(mul(root(s2), 1.0f), 1e-6f);
        count[r] = n;
    }
    __syncthreads();
    const float len = s_len;
    for (int i = tid; i < n; i += CB_THREADS) lc[i] = div(lc[i], len);
}

// one thread per (token-row, channel): corr = 0 + W[j0] c0 + W[j1] c1 + ... over the units whose code is not zero, in unit
// order (0 + W[0] * 0 when there is none), xf + corr
__global__ void cb_read_kernel(const int* __restrict__ list_j, const float* __restrict__ list_c, const int* __restrict__ count,
                               const float* __restrict__ W, int g, int R, int d, float* __restrict__ xf) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)R * d) return;
    const size_t r = i / d;
    const int ch = (int)(i % d);
    const int n = count[r];
    const int* lj = list_j + r * g;
    const float* lc = list_c + r * g;
    float corr = 0.0f;
    bool any = false;
    // eight rows of the read-out in flight while the chain adds the eight before them (a slot past the list has code 0)
    for (int e0 = 0; e0 < n; e0 += 8) {
        float c[8], w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int e = e0 + u;
            c[u] = e < n ? lc[e] : 0.0f;
            w[u] = W[(size_t)(e < n ? lj[e] : 0) * d + ch];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (c[u] != 0.0f) {
                corr = add(corr, mul(w[u], c[u]));
                any = true;
            }
    }
    if (!any) corr = add(corr, mul(W[ch], 0.0f));
    xf[i] = add(xf[i], corr);
}

}  // namespace

void launch_cb_inputs(cudaStream_t st, const float* tok_emb, const uint32_t* tok, int R, int d, int V, float* emb_rows) {
    const size_t n = (size_t)R * d;
    launch_k(cb_gather_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, tok_emb, tok, R, d, V, emb_rows);
}

void launch_cb_units(cudaStream_t st, const float* xf, const float* en, const uint32_t* idx, const float* sgn, int g, int d, int R, float* h) {
    const size_t n = (size_t)R * g;
    launch_k(cb_units_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, xf, en, idx, sgn, g, d, R, h);
}

void launch_cb_read(cudaStream_t st, const float* a, int g, int* list_j, float* list_c, int* count, const float* W, int R, int d, float* xf) {
    launch_k(cb_code_kernel, dim3(R), dim3(CB_THREADS), 0, st, a, g, list_j, list_c, count);
    const size_t n = (size_t)R * d;
    launch_k(cb_read_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const int*)list_j, (const float*)list_c, (const int*)count, W, g, R, d, xf);
}

}  // namespace ava

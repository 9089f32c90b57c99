// Kernels of the Ava-0.4 parts that hang off the surprise and the clocks: --dopamine and --mood (the surprise at each
// token and what follows from it: src/model/fstep/arch_f3.rs:106-186, src/model/fstep/arch_f4.rs:131-143) and --rhythm
// (src/model/fstep/arch_f4.rs:39-108).  Every value is the one the reference's one-token step computes: the cross
// entropy of the head's logits for block 0's normed output at the position before, with the exponentials summed in
// index order by one thread (the reference's loop); the mood's and the clocks' one-step scans token after token.
#include <cmath>

#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int SUR_THREADS = 256;

__device__ __forceinline__ float4 lds4u(const float* p) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
}

// one block per token-row: s = ((max + ln(sum exp(logit - max))) - logit[token]) * valid, z = s * inv_lnv + 0
__global__ void __launch_bounds__(SUR_THREADS) surprise_kernel(const float* __restrict__ logits, int V, const uint32_t* __restrict__ tok,
                                                               const float* __restrict__ valid, int rows, float inv_lnv, float* __restrict__ s_out,
                                                               float* __restrict__ z_out) {
    pdl_enter();
    extern __shared__ __align__(16) float sur_e[];  // [V] padded to a multiple of 4
    __shared__ float red[SUR_THREADS / 32];
    __shared__ float s_max;
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* lr = logits + (size_t)r * V;
    const int Vp = (V + 3) & ~3;
    float m = -INFINITY;
    for (int i = tid; i < V; i += SUR_THREADS) m = fmaxf(m, lr[i]);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (tid == 0) {
        float mm = red[0];
        for (int w = 1; w < SUR_THREADS / 32; ++w) mm = fmaxf(mm, red[w]);
        s_max = mm;
    }
    __syncthreads();
    const float mx = s_max;
    for (int i = tid; i < Vp; i += SUR_THREADS) sur_e[i] = i < V ? expf_(sub(lr[i], mx)) : 0.0f;
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;  // in index order; the padding adds +0 at the end
        float4 a = lds4u(sur_e);
        for (int i = 0; i < Vp; i += 4) {
            const float4 nx = lds4u(sur_e + (i + 4 < Vp ? i + 4 : i));
            sum = add(sum, a.x);
            sum = add(sum, a.y);
            sum = add(sum, a.z);
            sum = add(sum, a.w);
            a = nx;
        }
        const float lse = add(mx, logf_(sum));
        const uint32_t t = tok[r];
        const float ce = t < (uint32_t)V ? sub(lse, lr[t]) : 0.0f;
        const float v = r < rows ? valid[r] : 1.0f;  // the chunk's first token of each row carries the state's flag
        const float s = mul(ce, v);
        s_out[r] = s;
        z_out[r] = add(mul(s, inv_lnv), 0.0f);
    }
}

// one thread per (row, unit): m = (exp(0 ll) 1)((z win + bin) oml) + m exp(1 ll), ll = log_sigmoid(lam), oml = sigmoid(-lam)
__global__ void mood_kernel(const float* __restrict__ z, int rows, int T, int k, const float* __restrict__ lam, const float* __restrict__ win,
                            const float* __restrict__ bin, float* __restrict__ mood_state, float* __restrict__ mood_all) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * k) return;
    const int r = i / k, j = i % k;
    const float ll = log_sigmoid(lam[j]), oml = sigmoid(-lam[j]);
    const float p = mul(expf_(mul(0.0f, ll)), 1.0f), keep = expf_(mul(1.0f, ll));
    const float w = win[j], b = bin[j];
    float m = mood_state[i];
    for (int t = 0; t < T; ++t) {
        const float u = add(mul(z[(size_t)t * rows + r], w), b);
        m = add(mul(p, mul(u, oml)), mul(m, keep));
        mood_all[((size_t)t * rows + r) * k + j] = m;
    }
    mood_state[i] = m;
}

// the one-row product's order (w0 x0, then one fused multiply-add per further input; two inputs: w1 x1 + w0 x0)
__global__ void mood_gain_kernel(const float* __restrict__ mood_all, int k, const float* __restrict__ G, int M, int d, float* __restrict__ gain) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * d) return;
    const int c = (int)(i % d);
    const float* mv = mood_all + (i / d) * k;
    float zc;
    if (k == 1) {
        zc = mul(G[c], mv[0]);
    } else if (k == 2) {
        zc = add(mul(G[d + c], mv[1]), mul(G[c], mv[0]));
    } else {
        zc = mul(G[c], mv[0]);
        for (int j = 1; j < k; ++j) zc = fma(G[(size_t)j * d + c], mv[j], zc);
    }
    gain[i] = add(mul(tanhf_(zc), 1.0f), 1.0f);
}

__global__ void da_add_kernel(float* x, const float* __restrict__ y, const float* __restrict__ z, const float* __restrict__ w,
                              const float* __restrict__ c, const float* __restrict__ row_gain, int M, int d) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * d) return;
    const size_t r = i / d;
    const int ch = (int)(i % d);
    float o = mul(y[i], add(mul(tanhf_(add(mul(z[r], w[ch]), c[ch])), 1.0f), 1.0f));
    if (row_gain) o = mul(o, row_gain[r * NM_STRIDE]);
    x[i] = add(x[i], o);
}

// --rhythm, one thread per (row, clock): l = log_sigmoid(-(pre + br)) = ln(1 - reset), the one-step scan written as the
// reference's chunk form at one token (big = l 1, before = big - l, diff = big - before, w = exp(min(diff, 0)) 1,
// time = w + exp(big) time), phase = time exp(lw), features cos and sin
__global__ void rhythm_kernel(const float* __restrict__ pre, const float* __restrict__ br, const float* __restrict__ lw, int rows, int T,
                              float* __restrict__ times, float* __restrict__ f) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * 2) return;
    const int r = i >> 1, o = i & 1;
    const float b = br[o], w_ph = expf_(lw[o]);
    float a = times[i];
    for (int t = 0; t < T; ++t) {
        const size_t row = (size_t)t * rows + r;
        const float p = add(pre[row * 4 + o], b);
        const float l = log_sigmoid(-p);
        const float big = mul(l, 1.0f), before = sub(big, l), diff = sub(big, before);
        const float w = mul(expf_(diff > 0.0f ? 0.0f : diff), 1.0f);
        a = add(w, mul(expf_(big), a));
        const float ph = mul(a, w_ph);
        f[row * 4 + 2 * o] = cosf_(ph);
        f[row * 4 + 2 * o + 1] = sinf_(ph);
    }
    times[i] = a;
}

__global__ void rhythm_gates_kernel(const float* __restrict__ f, const float* __restrict__ Gw, const float* __restrict__ Gr, int M, int nh,
                                    float* __restrict__ gw, float* __restrict__ gr) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * nh) return;
    const int r = i / nh, e = i % nh;
    const float4 fv = *reinterpret_cast<const float4*>(f + (size_t)r * 4);
    float zw = mul(Gw[e], fv.x), zr = mul(Gr[e], fv.x);
    zw = fma(Gw[nh + e], fv.y, zw);
    zr = fma(Gr[nh + e], fv.y, zr);
    zw = fma(Gw[2 * nh + e], fv.z, zw);
    zr = fma(Gr[2 * nh + e], fv.z, zr);
    zw = fma(Gw[3 * nh + e], fv.w, zw);
    zr = fma(Gr[3 * nh + e], fv.w, zr);
    gw[i] = add(mul(tanhf_(zw), 1.0f), 1.0f);
    gr[i] = add(mul(tanhf_(zr), 1.0f), 1.0f);
}

}  // namespace

void launch_rhythm(cudaStream_t st, const float* pre, const float* br, const float* lw, int rows, int T, float* times, float* f) {
    launch_k(rhythm_kernel, dim3((rows * 2 + 127) / 128), dim3(128), 0, st, pre, br, lw, rows, T, times, f);
}

void launch_rhythm_gates(cudaStream_t st, const float* f, const float* Gw, const float* Gr, int M, int nh, float* gw, float* gr) {
    launch_k(rhythm_gates_kernel, dim3((M * nh + 127) / 128), dim3(128), 0, st, f, Gw, Gr, M, nh, gw, gr);
}

bool launch_surprise(cudaStream_t st, const float* logits, int V, const uint32_t* tok, const float* valid, int rows, int T, float* s, float* z) {
    const size_t smem = (size_t)((V + 3) & ~3) * sizeof(float);
    if (smem > 220 * 1024) return false;
    if (smem > 32 * 1024) cudaFuncSetAttribute(surprise_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const float inv_lnv = (float)(1.0 / std::log((double)V));
    launch_k(surprise_kernel, dim3(rows * T), dim3(SUR_THREADS), smem, st, logits, V, tok, valid, rows, inv_lnv, s, z);
    return true;
}

void launch_mood(cudaStream_t st, const float* z, int rows, int T, int k, const float* lam, const float* win, const float* bin, float* mood_state,
                 float* mood_all) {
    launch_k(mood_kernel, dim3((rows * k + 127) / 128), dim3(128), 0, st, z, rows, T, k, lam, win, bin, mood_state, mood_all);
}

void launch_mood_gain(cudaStream_t st, const float* mood_all, int k, const float* G, int M, int d, float* gain) {
    const size_t n = (size_t)M * d;
    launch_k(mood_gain_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, mood_all, k, G, M, d, gain);
}

void launch_da_add(cudaStream_t st, float* x, const float* y, const float* z, const float* w, const float* c, const float* row_gain, int M, int d) {
    const size_t n = (size_t)M * d;
    launch_k(da_add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, y, z, w, c, row_gain, M, d);
}

}  // namespace ava

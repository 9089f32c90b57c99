// The engram: one softmax attention read per token over every key/value stored so far (sm_100a).
//
// Follows the reference's one-token read (design-tests/nn/gpu/src/model/fstep.rs:303-356 and
// src/model/fstep/arch.rs:909-974): this token's key and value join the store first, then per head the scores
// K_j . q (row 0's product, then fma over the head's dimensions) times 1/sqrt(hs), the maximum, exp(s - max), the
// sum taken in key order from 0, each weight divided by it, and the mix p . V in gemm's one-row order over the keys.
// One block of threads per row; the scores of all heads live in shared memory.  The store is a ring per row so that
// an oldest-first cap (src/state.rs:526-538) drops a token by moving the start.
#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

template <bool BF16>
__device__ __forceinline__ float kv_load(const void* base, size_t i) {
    if (BF16) return bf16_to_f(reinterpret_cast<const uint16_t*>(base)[i]);
    return reinterpret_cast<const float*>(base)[i];
}
template <bool BF16>
__device__ __forceinline__ void kv_store(void* base, size_t i, float v) {
    if (BF16)
        reinterpret_cast<uint16_t*>(base)[i] = f_to_bf16(v);
    else
        reinterpret_cast<float*>(base)[i] = v;
}

template <bool BF16>
__global__ void engram_kernel(const EngramArgs a) {
    extern __shared__ float sm[];
    __shared__ int s_n, s_start;
    const int d = a.d, hs = a.hs, nh = d / hs, cap = a.cap;
    const int r = blockIdx.x, tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarp = T >> 5;
    const float* qkv = a.qkv + (size_t)r * 3 * d;
    const size_t row_base = (size_t)r * nh * cap * hs;

    // this token's key and value join the store
    if (tid == 0) {
        int n = a.n[r];
        if (n >= cap) {
            atomicOr(a.status, ST_ENGRAM_FULL);
            n = cap - 1;  // keep the kernel in bounds; the host reports the error
        }
        s_n = n;
        s_start = a.start[r];
    }
    __syncthreads();
    const int n0 = s_n, start = s_start, n = n0 + 1;
    const int slot = (start + n0) % cap;
    for (int c = tid; c < d; c += T) {
        const int hh = c / hs, dd = c % hs;
        const size_t o = row_base + ((size_t)hh * cap + slot) * hs + dd;
        kv_store<BF16>(a.k, o, qkv[d + c]);
        kv_store<BF16>(a.v, o, qkv[2 * d + c]);
    }
    float* q = sm;              // [d]
    float* mx = q + d;          // [nh]
    float* den = mx + nh;       // [nh]
    float* sc = den + nh;       // [nh][n]
    for (int c = tid; c < d; c += T) q[c] = qkv[c];
    __syncthreads();  // the stores above are visible to this block's loads below

    const float scale = (float)(1.0 / sqrt((double)hs));
    for (int idx = tid; idx < nh * n; idx += T) {
        const int hh = idx / n, j = idx % n;
        const size_t o = row_base + ((size_t)hh * cap + (start + j) % cap) * hs;
        const float* qh = q + hh * hs;
        float s = mul(kv_load<BF16>(a.k, o), qh[0]);
        for (int x = 1; x < hs; ++x) s = fma(kv_load<BF16>(a.k, o + x), qh[x], s);
        sc[(size_t)hh * n + j] = add(mul(s, scale), 0.0f);
    }
    __syncthreads();
    for (int hh = warp; hh < nh; hh += nwarp) {
        float m = -INFINITY;
        for (int j = lane; j < n; j += 32) m = fmaxf(m, sc[(size_t)hh * n + j]);
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) mx[hh] = m;
    }
    __syncthreads();
    for (int idx = tid; idx < nh * n; idx += T) sc[idx] = expf_(sub(sc[idx], mx[idx / n]));
    __syncthreads();
    for (int hh = tid; hh < nh; hh += T) {
        float s = 0.0f;
        const float* p = sc + (size_t)hh * n;
        for (int j = 0; j < n; ++j) s = add(s, p[j]);
        den[hh] = s;
    }
    __syncthreads();
    for (int idx = tid; idx < nh * n; idx += T) sc[idx] = div(sc[idx], den[idx / n]);
    __syncthreads();
    // o = p . V: per output the chain over the keys (src/model/fstep.rs:222-257 with k = n)
    for (int c = tid; c < d; c += T) {
        const int hh = c / hs, dd = c % hs;
        const float* p = sc + (size_t)hh * n;
        const size_t hb = row_base + (size_t)hh * cap * hs + dd;
        auto V = [&](int j) { return kv_load<BF16>(a.v, hb + (size_t)((start + j) % cap) * hs); };
        float out;
        if (n == 1) {
            out = mul(V(0), p[0]);
        } else if (n == 2) {
            out = add(mul(V(1), p[1]), mul(V(0), p[0]));
        } else {
            out = mul(V(0), p[0]);
            for (int j = 1; j < n; ++j) out = fma(V(j), p[j], out);
        }
        a.o[(size_t)r * d + c] = out;
    }
    // the read saw every token including the oldest; a capped store then drops the oldest (src/state.rs:526-538)
    if (tid == 0) {
        if (n > a.keep) {
            a.n[r] = a.keep;
            a.start[r] = (start + (n - a.keep)) % cap;
        } else {
            a.n[r] = n;
        }
    }
}

}  // namespace

bool launch_engram(cudaStream_t st, const EngramArgs& a, int n_max) {
    const int nh = a.d / a.hs;
    const size_t smem = ((size_t)a.d + 2 * nh + (size_t)nh * n_max) * sizeof(float);
    if (smem > 227 * 1024 - 64) return false;
    int threads = ((a.d + 31) / 32) * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 128) threads = 128;
    if (a.bf16) {
        cudaFuncSetAttribute(engram_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        engram_kernel<true><<<a.M, threads, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(engram_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        engram_kernel<false><<<a.M, threads, smem, st>>>(a);
    }
    return true;
}

}  // namespace ava

// The per-row kernels of the block step (sm_100a): embedding gather, RMS norm, the memory's gate preparation and
// head norm + output gate, k-winners-take-all, the dense residual mix, greedy argmax.
//
// Sums that the reference takes "one value after another from 0" (design-tests/nn/gpu/src/model/fstep.rs:12-14) are
// taken in that order by one thread, and the small f32 products follow gemm's one-row order (fstep.rs:17-23,222-257):
// out = w0 * x0, then fma(w_j, x_j, out).  The chains are short next to the memory traffic of the step, and keeping
// them makes every value the bits of the reference's arithmetic.
#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr float NORM_EPS = 1e-5f;  // src/model.rs:36

// sum of x[i]^2 one after another from 0; x in shared memory, 16-byte aligned.  Eight values are fetched ahead of the
// chain so that the loads overlap; the order of the additions is the reference's.
__device__ __forceinline__ float sumsq_seq(const float* x, int n) {
    float s = 0.0f;
    int i = 0;
    for (; i + 8 <= n; i += 8) {
        const float4 a = *reinterpret_cast<const float4*>(x + i), b = *reinterpret_cast<const float4*>(x + i + 4);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        float p[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) p[k] = mul(v[k], v[k]);
#pragma unroll
        for (int k = 0; k < 8; ++k) s = add(s, p[k]);
    }
    for (; i < n; ++i) s = add(s, mul(x[i], x[i]));
    return s;
}

// sum of a[i] * b[i] one after another from 0 (shared memory, 16-byte aligned)
__device__ __forceinline__ float dot_seq(const float* a, const float* b, int n) {
    float s = 0.0f;
    int i = 0;
    for (; i + 8 <= n; i += 8) {
        const float4 a0 = *reinterpret_cast<const float4*>(a + i), a1 = *reinterpret_cast<const float4*>(a + i + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(b + i), b1 = *reinterpret_cast<const float4*>(b + i + 4);
        const float p[8] = {mul(a0.x, b0.x), mul(a0.y, b0.y), mul(a0.z, b0.z), mul(a0.w, b0.w),
                            mul(a1.x, b1.x), mul(a1.y, b1.y), mul(a1.z, b1.z), mul(a1.w, b1.w)};
#pragma unroll
        for (int k = 0; k < 8; ++k) s = add(s, p[k]);
    }
    for (; i < n; ++i) s = add(s, mul(a[i], b[i]));
    return s;
}

// (mean(x^2) + eps)^-1/2 with the squares summed in order (src/model/fstep.rs:212-220); x in shared memory
__device__ __forceinline__ float inv_rms_seq(const float* x, int n) {
    const float s = sumsq_seq(x, n);
    const float ms = add(mul(s, (float)(1.0 / (double)n)), 0.0f);
    return rsqrtf_(add(mul(ms, 1.0f), NORM_EPS));
}

// (sum(x^2) + 1e-6)^-1/2 (src/model/fstep.rs:271-282)
__device__ __forceinline__ float inv_l2_seq(const float* x, int n) {
    const float s = sumsq_seq(x, n);
    return rsqrtf_(add(mul(s, 1.0f), (float)1e-6));
}

// gemm's one-row product for one output: x [k] (shared), w[j * stride] the column's weights (global).  The weights are
// fetched sixteen at a time ahead of the chain so that their latency overlaps; the chain's order is untouched.
__device__ __forceinline__ float gemv_col(const float* x, int k, const float* __restrict__ w, int stride) {
    if (k == 0) return 0.0f;
    if (k == 1) return mul(w[0], x[0]);
    if (k == 2) return add(mul(w[stride], x[1]), mul(w[0], x[0]));
    float out = mul(w[0], x[0]);
    for (int j = 1; j < k; j += 16) {
        float t[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t[i] = (j + i < k) ? __ldg(w + (size_t)(j + i) * stride) : 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (j + i < k) out = fma(t[i], x[j + i], out);
    }
    return out;
}

__device__ __forceinline__ bool finite_f(float v) { return (f_to_bits(v) & 0x7f800000u) != 0x7f800000u; }

// ---------------------------------------------------------------------------------------------------- embedding
__global__ void embed_kernel(const float* __restrict__ tok_emb, const uint32_t* __restrict__ tok, int M, int d, int vocab, float* x, float* stream0,
                             uint32_t* status) {
    pdl_enter();
    const int r = blockIdx.x;
    uint32_t t = tok[r];
    if (t >= (uint32_t)vocab) {  // stay in bounds; the host reports the token
        if (threadIdx.x == 0) atomicOr(status, ST_BAD_TOKEN);
        t = 0;
    }
    const float4* src = reinterpret_cast<const float4*>(tok_emb + (size_t)t * d);
    float4* dst = reinterpret_cast<float4*>(x + (size_t)r * d);
    float4* dst2 = stream0 ? reinterpret_cast<float4*>(stream0 + (size_t)r * d) : nullptr;
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
        const float4 v = src[i];
        dst[i] = v;
        if (dst2) dst2[i] = v;
    }
}

// ---------------------------------------------------------------------------------------------------- RMS norm
// three bf16 limbs of v (their sum is v exactly) into planes [3][plane], for the tensor-core products
__device__ __forceinline__ void store_limbs(uint16_t* limbs, int64_t plane, int64_t i, float v) {
    const uint16_t hi = f_to_bf16(v);
    const float r1 = sub(v, bf16_to_f(hi));
    const uint16_t mid = f_to_bf16(r1);
    limbs[i] = hi;
    limbs[plane + i] = mid;
    limbs[2 * plane + i] = f_to_bf16(sub(r1, bf16_to_f(mid)));
}

// One warp per row: the row is staged in shared memory, lane 0 takes the ordered sum, every lane scales.
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain, int M, int n, float* __restrict__ y,
                               uint16_t* __restrict__ limbs) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= M) return;
    float* xs = sm + (size_t)warp * n;
    const float* xr = x + (size_t)r * n;
    for (int i = lane; i < n; i += 32) xs[i] = xr[i];
    __syncwarp();
    float inv = 0.0f;
    if (lane == 0) inv = inv_rms_seq(xs, n);
    inv = __shfl_sync(0xffffffffu, inv, 0);
    float* yr = y + (size_t)r * n;
    for (int i = lane; i < n; i += 32) {
        const float v = mul(mul(xs[i], inv), gain[i]);
        yr[i] = v;
        if (limbs) store_limbs(limbs, (int64_t)M * n, (int64_t)r * n + i, v);
    }
}

// ---------------------------------------------------------------------------------------------------- memory: gates
// src/model/fstep/arch.rs:685-803 for one row per block of threads.
__global__ void mem_prep_kernel(const MemPrepArgs a) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int d = a.d, hs = a.hs, nh = d / hs, rk = a.rank;
    const int r = blockIdx.x, tid = threadIdx.x, T = blockDim.x;
    float* h = sm;            // [d]
    float* q = h + d;         // [d] raw, then unit
    float* kr = q + d;        // [d] raw key
    float* ek = kr + d;       // [d] raw erase key, then unit
    float* wv = ek + d;       // [d] w = k b
    float* ahv = wv + d;      // [d] ah = e (b alpha)
    float* lra = ahv + d;     // [d]
    float* lrb = lra + d;     // [d]
    float* inv_q = lrb + d;   // [nh]
    float* inv_k = inv_q + nh;
    float* inv_e = inv_k + nh;
    float* za = inv_e + nh;
    float* zb = za + nh;
    float* z1a = zb + nh;     // [rk]
    float* z1b = z1a + rk;    // [rk]

    const float* pr = a.proj + (size_t)r * a.ldp;
    for (int c = tid; c < d; c += T) {
        h[c] = a.h[(size_t)r * d + c];
        q[c] = pr[c];
        const float kk = pr[d + c];
        kr[c] = kk;
        ek[c] = add(kk, pr[3 * d + c]);
    }
    __syncthreads();
    // The ordered chains.  The gate projections h . [wa | wb | wa1 | wb1] (gemm's one-row order: row 0's product,
    // then fma down the rows) take one thread per output column; their weights come through shared memory a chunk of
    // rows at a time (every thread copies, cp.async, double buffered), so a chain never waits on global memory.  The
    // three sums of squares per head run in the warps after them while the first chunk is in flight.
    {
        const int ncols = 2 * nh + 2 * rk, ncp = a.gate_cols;  // real and padded column count
        const int CR = a.gate_chunk, nchunk = d / CR;
        float* stage = z1b + rk;                               // [2][CR * ncp], 16-byte aligned (see the launcher)
        stage += (4 - ((5 * nh + 2 * rk) & 3)) & 3;
        const int per_chunk4 = CR * ncp / 4;
        auto fetch = [&](int c) {
            float* dst = stage + (size_t)(c & 1) * CR * ncp;
            const float* src = a.gate_w + (size_t)c * CR * ncp;
            for (int i = tid; i < per_chunk4; i += T)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst + 4 * i)), "l"(src + 4 * i) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        fetch(0);
        float out = -0.0f;  // fma(w, x, -0) is the plain rounded product: the chain's first term
        const int first_sq = ((ncols + 31) / 32) * 32;         // sums of squares start at a warp boundary
        for (int c = 0; c < nchunk; ++c) {
            if (c + 1 < nchunk) {
                fetch(c + 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
            if (tid < ncols) {
                const float* wcol = stage + (size_t)(c & 1) * CR * ncp + tid;
                const float* hx = h + c * CR;
                for (int r0 = 0; r0 < CR; r0 += 8) {
                    float w8[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) w8[i] = wcol[(size_t)(r0 + i) * ncp];
                    const float4 x0 = *reinterpret_cast<const float4*>(hx + r0), x1 = *reinterpret_cast<const float4*>(hx + r0 + 4);
                    const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) out = fma(w8[i], xv[i], out);
                }
            } else if (c == 0) {
                for (int it = tid - first_sq; it >= 0 && it < 3 * nh; it += T - first_sq) {
                    const int which = it / nh, e = it % nh;
                    const float* src = (which == 0 ? q : which == 1 ? kr : ek) + e * hs;
                    (which == 0 ? inv_q : which == 1 ? inv_k : inv_e)[e] = inv_l2_seq(src, hs);
                }
            }
            __syncthreads();
        }
        if (tid < nh) za[tid] = add(out, a.ba[tid]);
        else if (tid < 2 * nh) zb[tid - nh] = add(out, a.bb[tid - nh]);
        else if (tid < 2 * nh + rk) z1a[tid - 2 * nh] = out;
        else if (tid < ncols) z1b[tid - 2 * nh - rk] = out;
    }
    __syncthreads();
    for (int c = tid; c < d; c += T) {
        lra[c] = gemv_col(z1a, rk, a.wa2 + c, d);
        lrb[c] = gemv_col(z1b, rk, a.wb2 + c, d);
    }
    __syncthreads();
    bool bad = false;
    for (int c = tid; c < d; c += T) {
        const int e = c / hs;
        const size_t o = (size_t)r * d + c;
        const float la = log_sigmoid(add(add(za[e], a.off[c]), lra[c]));
        const float be = add(mul(sigmoid(add(zb[e], lrb[c])), 2.0f), 0.0f);
        const float ex = expf_(la);
        const float qn = mul(q[c], inv_q[e]);
        const float kn = mul(kr[c], inv_k[e]);
        const float en = mul(ek[c], inv_e[e]);
        float v = pr[2 * d + c];
        if (a.first) {
            a.v_first[o] = v;
        } else if (a.vres) {
            // (1 + p0) v + p1 v0 (src/model/fstep/arch.rs:697-702)
            const float p0 = add(mul(a.vres[0], 1.0f), 1.0f);
            v = add(mul(v, p0), mul(a.v_first[o], a.vres[1]));
        }
        const float w = mul(kn, be);
        const float ah = mul(en, mul(be, ex));
        const float qg = mul(qn, ex);
        bad |= !(finite_f(la) && finite_f(en) && finite_f(w) && finite_f(ah) && finite_f(qn) && finite_f(v));
        a.e[o] = en;
        a.v[o] = v;
        a.w[o] = w;
        a.ah[o] = ah;
        a.qg[o] = qg;
        a.ex[o] = ex;
        if (a.qs) a.qs[o] = mul(qn, add(mul(1.0f, a.mom), 0.0f));  // q * (1 * M + 0) (src/model/fstep/arch.rs:784)
        q[c] = qn;
        wv[c] = w;
        ahv[c] = ah;
    }
    if (bad) atomicOr(a.status, ST_NONFINITE);
    __syncthreads();
    // q.w and q.ah, each summed in order from 0 (src/model/fstep/arch.rs:789-797)
    for (int role = tid; role < 2 * nh; role += T) {
        const int e = role % nh;
        const float* b = role < nh ? wv : ahv;
        (role < nh ? a.qw : a.qa)[(size_t)r * nh + e] = dot_seq(q + e * hs, b + e * hs, hs);
    }
}

// ---------------------------------------------------------------------------------------------------- memory: output
// head norm, then the silu output gate (src/model/fstep/arch.rs:842-852)
__global__ void mem_post_kernel(const float* __restrict__ y_raw, const float* __restrict__ gate, int ldg, int M, int d, int hs, float* __restrict__ y,
                                uint16_t* __restrict__ limbs) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int nh = d / hs, r = blockIdx.x, tid = threadIdx.x, T = blockDim.x;
    float* ys = sm;
    float* inv = sm + d;
    for (int c = tid; c < d; c += T) ys[c] = y_raw[(size_t)r * d + c];
    __syncthreads();
    for (int e = tid; e < nh; e += T) inv[e] = inv_rms_seq(ys + e * hs, hs);
    __syncthreads();
    for (int c = tid; c < d; c += T) {
        float v = mul(ys[c], inv[c / hs]);
        if (gate) {
            const float g = gate[(size_t)r * ldg + c];
            v = mul(v, div(g, add(1.0f, expf_(-g))));
        }
        y[(size_t)r * d + c] = v;
        if (limbs) store_limbs(limbs, (int64_t)M * d, (int64_t)r * d + c, v);
    }
}

// ---------------------------------------------------------------------------------------------------- kWTA
// The k-th largest value found exactly, one byte of its order-preserving key per round (256 threads, one per
// histogram bin): the result is the largest key T with count(keys >= T) >= k.  Every unit at or above it is kept (ties included), negatives dropped, squared on request
// (src/model/fstep.rs:295-299, src/model/fstep/arch.rs:982-989).
__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = f_to_bits(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) { return bits_to_f((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

__global__ void kwta_kernel(const float* __restrict__ u, int M, int n, int k, int relu2, float* __restrict__ out) {
    pdl_enter();
    extern __shared__ uint32_t keys[];  // [n] keys
    const int r = blockIdx.x, tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5;
    const float* ur = u + (size_t)r * n;
    float* orow = out + (size_t)r * n;
    if (k >= n) {
        for (int i = tid; i < n; i += T) {
            float v = fmaxf(mul(ur[i], 1.0f), 0.0f);
            orow[i] = relu2 ? mul(v, v) : v;
        }
        return;
    }
    for (int i = tid; i < n; i += T) keys[i] = order_key(ur[i]);
    // radix select, one byte of the key per pass from the top: a 256-bin histogram of the keys that share the prefix
    // found so far, a suffix sum over the bins (one bin per thread), and the bin that holds the k-th largest
    __shared__ int hist[256];
    __shared__ int warp_sum[8];
    __shared__ uint32_t sel_prefix;
    __shared__ int sel_k;
    uint32_t thr = 0;
    int k_rem = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        hist[tid] = 0;
        __syncthreads();
        const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < n; i += T) {
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
    for (int i = tid; i < n; i += T) {
        const float v = ur[i];
        float o = fmaxf(mul(v, sub(v, kth) >= 0.0f ? 1.0f : 0.0f), 0.0f);
        orow[i] = relu2 ? mul(o, o) : o;
    }
}

// ---------------------------------------------------------------------------------------------------- dense mix
// src/model/fstep/arch.rs:1014-1024: the block's output joins the streams, then x <- x + sum_j stream_j w_j in order.
__global__ void dense_mix_kernel(float* x, float* streams, const float* __restrict__ w, int n_streams, int64_t MD) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= MD) return;
    const float xv = x[i];
    streams[(int64_t)(n_streams - 1) * MD + i] = xv;
    float mix = xv;
    for (int j = 0; j < n_streams - 1; ++j) mix = add(mix, mul(streams[(int64_t)j * MD + i], w[j]));
    mix = add(mix, mul(xv, w[n_streams - 1]));
    x[i] = mix;
}

// ---------------------------------------------------------------------------------------------------- argmax
__global__ void argmax_kernel(const float* __restrict__ logits, int M, int V, uint32_t* next) {
    pdl_enter();
    __shared__ float bv[32];
    __shared__ uint32_t bi[32];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* lr = logits + (size_t)r * V;
    float best = -INFINITY;
    uint32_t idx = 0xffffffffu;
    for (int i = tid; i < V; i += blockDim.x) {
        const float v = lr[i];
        if (v > best || (v == best && (uint32_t)i < idx) || idx == 0xffffffffu) {
            best = v;
            idx = i;
        }
    }
    auto better = [](float v, uint32_t i, float bv_, uint32_t bi_) { return bi_ == 0xffffffffu || (i != 0xffffffffu && (v > bv_ || (v == bv_ && i < bi_))); };
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) {
            best = ov;
            idx = oi;
        }
    }
    if (lane == 0) {
        bv[warp] = best;
        bi[warp] = idx;
    }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < (blockDim.x >> 5); ++w)
            if (better(bv[w], bi[w], best, idx)) {
                best = bv[w];
                idx = bi[w];
            }
        next[r] = idx == 0xffffffffu ? 0u : idx;
    }
}

__global__ void math_kernel(int which, const float* x, int64_t n, float* y) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    y[i] = which == 0 ? expf_(x[i]) : which == 1 ? logf_(x[i]) : rsqrtf_(x[i]);
}

__global__ void round_bf16_kernel(const float* x, int64_t n, uint16_t* y) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = f_to_bf16(x[i]);
}
__global__ void widen_bf16_kernel(const uint16_t* x, int64_t n, float* y) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = bf16_to_f(x[i]);
}

template <typename K>
void opt_in_smem(K kernel, size_t bytes) {
    if (bytes > 32 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace

void launch_embed(cudaStream_t st, const float* tok_emb, const uint32_t* tok, int M, int d, int vocab, float* x, float* stream0, uint32_t* status) {
    launch_k(embed_kernel, dim3(M), dim3(128), 0, st, tok_emb, tok, M, d, vocab, x, stream0, status);
}

void launch_rmsnorm(cudaStream_t st, const float* x, const float* gain, int M, int n, float* y, uint16_t* limbs) {
    const int warps = 4;
    const size_t smem = (size_t)warps * n * sizeof(float);
    opt_in_smem(rmsnorm_kernel, smem);
    launch_k(rmsnorm_kernel, dim3((M + warps - 1) / warps), dim3(warps * 32), smem, st, x, gain, M, n, y, limbs);
}

void launch_mem_prep(cudaStream_t st, const MemPrepArgs& a) {
    const int nh = a.d / a.hs;
    const size_t smem = ((size_t)8 * a.d + 5 * nh + 2 * a.rank + 4 + 2 * (size_t)a.gate_chunk * a.gate_cols) * sizeof(float);
    opt_in_smem(mem_prep_kernel, smem);
    launch_k(mem_prep_kernel, dim3(a.M), dim3(256), smem, st, a);
}

void launch_mem_post(cudaStream_t st, const float* y_raw, const float* gate, int ldg, int M, int d, int hs, float* y, uint16_t* limbs) {
    const size_t smem = ((size_t)d + d / hs) * sizeof(float);
    opt_in_smem(mem_post_kernel, smem);
    launch_k(mem_post_kernel, dim3(M), dim3(256), smem, st, y_raw, gate, ldg, M, d, hs, y, limbs);
}

void launch_kwta(cudaStream_t st, const float* u, int M, int n, int k, int relu2, float* a) {
    const size_t smem = (size_t)n * sizeof(uint32_t);
    opt_in_smem(kwta_kernel, smem);
    launch_k(kwta_kernel, dim3(M), dim3(256), smem, st, u, M, n, k, relu2, a);
}

void launch_dense_mix(cudaStream_t st, float* x, float* streams, const float* w, int n_streams, int64_t MD) {
    launch_k(dense_mix_kernel, dim3((unsigned)((MD + 255) / 256)), dim3(256), 0, st, x, streams, w, n_streams, MD);
}

void launch_argmax(cudaStream_t st, const float* logits, int M, int V, uint32_t* next) { launch_k(argmax_kernel, dim3(M), dim3(256), 0, st, logits, M, V, next); }

void launch_math(cudaStream_t st, int which, const float* x, int64_t n, float* y) {
    launch_k(math_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, which, x, n, y);
}
void launch_round_bf16(cudaStream_t st, const float* x, int64_t n, uint16_t* y) {
    launch_k(round_bf16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, n, y);
}
void launch_widen_bf16(cudaStream_t st, const uint16_t* x, int64_t n, float* y) {
    launch_k(widen_bf16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, n, y);
}

}  // namespace ava

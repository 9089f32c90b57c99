// The token sampler on the device: `diary::pick` (design-tests/nn/gpu/src/diary.rs:686-718) for every row of a step at
// once, so that a sampled generation loop does not copy the logits to the host (16.8 MB per step at 256 rows of 16384)
// nor sort them there.  One block per row; every value is the one ava_pick (generate.cpp) computes on the host from
// the same logits and the same uniform number: softmax(logits * (1 / temperature)) in f32 with the largest value taken
// out, the exponentials summed in index order by one thread, the top_k most likely kept with ties in index order,
// their mass summed in f64 in that order, one draw walked down the list.
//
// The k-th largest probability is found by radix select (as the k-WTA does), the candidates are compacted in index
// order and sorted by (probability down, index up) with a bitonic network in shared memory; top_k is limited to 1024.
#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int SAMPLE_THREADS = 256, SAMPLE_MAX_K = 1024;

__device__ __forceinline__ float4 lds4s(const float* p) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits, int V, float inv_t, int top_k,
                                                                const double* __restrict__ uniform, uint32_t* __restrict__ next) {
    pdl_enter();
    extern __shared__ __align__(16) unsigned char smem[];
    float* p = reinterpret_cast<float*>(smem);                                   // [V] (padded to a multiple of 4)
    const int Vp = (V + 3) & ~3;
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(p + Vp);    // [SAMPLE_MAX_K] sort keys
    __shared__ float red[SAMPLE_THREADS / 32];
    __shared__ float s_max, s_sum;
    __shared__ int hist[256];
    __shared__ int warp_sum[SAMPLE_THREADS / 32];
    __shared__ uint32_t sel_prefix;
    __shared__ int sel_k, n_gt, n_eq_take;
    __shared__ int part[SAMPLE_THREADS + 1];
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* lr = logits + (size_t)r * V;

    // z = logit * (1 / T) + 0 and its maximum
    float m = -INFINITY;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float z = add(mul(lr[i], inv_t), 0.0f);
        p[i] = z;
        m = fmaxf(m, z);
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (tid == 0) {
        float mm = red[0];
        for (int w = 1; w < SAMPLE_THREADS / 32; ++w) mm = fmaxf(mm, red[w]);
        s_max = mm;
    }
    __syncthreads();
    const float mx = s_max;
    for (int i = tid; i < Vp; i += SAMPLE_THREADS) p[i] = i < V ? expf_(sub(p[i], mx)) : 0.0f;
    __syncthreads();
    if (tid == 0) {  // the sum in index order, as the host's loop takes it (the padding adds +0 at the end: no change)
        float s = 0.0f;
        float4 a = lds4s(p);
        for (int i = 0; i < Vp; i += 4) {
            const float4 nx = lds4s(p + (i + 4 < Vp ? i + 4 : i));
            s = add(s, a.x);
            s = add(s, a.y);
            s = add(s, a.z);
            s = add(s, a.w);
            a = nx;
        }
        s_sum = s;
    }
    __syncthreads();
    const float sum = s_sum;
    for (int i = tid; i < V; i += SAMPLE_THREADS) p[i] = div(p[i], sum);
    __syncthreads();

    // the k-th largest probability: radix select over the bit patterns (non-negative floats order as unsigned integers)
    const int k = top_k < 1 ? 1 : (top_k > V ? V : top_k);
    uint32_t thr = 0;
    int k_rem = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        hist[tid] = 0;
        __syncthreads();
        const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const uint32_t key = f_to_bits(p[i]);
            if ((key & mask) == thr) atomicAdd(&hist[(key >> shift) & 255u], 1);
        }
        __syncthreads();
        const int h = hist[tid];
        int sfx = h;
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_down_sync(0xffffffffu, sfx, o);
            if (lane + o < 32) sfx += up;
        }
        if (lane == 0) warp_sum[warp] = sfx;
        __syncthreads();
        for (int w = warp + 1; w < SAMPLE_THREADS / 32; ++w) sfx += warp_sum[w];
        if (sfx >= k_rem && sfx - h < k_rem) {
            sel_prefix = thr | ((uint32_t)tid << shift);
            sel_k = k_rem - (sfx - h);
        }
        __syncthreads();
        thr = sel_prefix;
        k_rem = sel_k;  // how many of the values equal to the threshold are kept: those with the lowest indices
    }
    // candidates in index order: every p above the threshold, and the first k_rem equal to it.  Each thread owns a
    // contiguous range of indices; counts, then an exclusive scan, then the writes.
    const int per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS, i0 = tid * per, i1 = min(V, i0 + per);
    int c_gt = 0, c_eq = 0;
    for (int i = i0; i < i1; ++i) {
        const uint32_t key = f_to_bits(p[i]);
        c_gt += key > thr;
        c_eq += key == thr;
    }
    // scan of the equal counts first (which equals are taken), then of the taken totals
    part[tid + 1] = c_eq;
    __syncthreads();
    if (tid == 0) {
        part[0] = 0;
        for (int t = 1; t <= SAMPLE_THREADS; ++t) part[t] += part[t - 1];
    }
    __syncthreads();
    const int eq_before = part[tid];
    const int eq_take = max(0, min(c_eq, k_rem - eq_before));
    __syncthreads();
    part[tid + 1] = c_gt + eq_take;
    __syncthreads();
    if (tid == 0) {
        part[0] = 0;
        for (int t = 1; t <= SAMPLE_THREADS; ++t) part[t] += part[t - 1];
    }
    __syncthreads();
    {
        int at = part[tid], eq_left = eq_take;
        for (int i = i0; i < i1; ++i) {
            const uint32_t key = f_to_bits(p[i]);
            bool take = key > thr;
            if (key == thr && eq_left > 0) {
                take = true;
                --eq_left;
            }
            // sort key: probability high to low, then index low to high
            if (take) cand[at++] = ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
        }
    }
    __syncthreads();
    // pad to a power of two with zeros (they sort to the end) and sort descending
    int n2 = 1;
    while (n2 < k) n2 <<= 1;
    for (int i = k + tid; i < n2; i += SAMPLE_THREADS) cand[i] = 0ull;
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < n2; i += SAMPLE_THREADS) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool desc = (i & size) == 0;
                    const unsigned long long a = cand[i], b = cand[j];
                    if (desc ? a < b : a > b) {
                        cand[i] = b;
                        cand[j] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
    if (tid == 0) {
        double total = 0.0;
        for (int j = 0; j < k; ++j) total += (double)bits_to_f((uint32_t)(cand[j] >> 32));
        double rr = uniform[r] * total;
        uint32_t out = 0xffffffffu - (uint32_t)(cand[k - 1] & 0xffffffffull);
        for (int j = 0; j < k; ++j) {
            rr -= (double)bits_to_f((uint32_t)(cand[j] >> 32));
            if (rr <= 0.0) {
                out = 0xffffffffu - (uint32_t)(cand[j] & 0xffffffffull);
                break;
            }
        }
        next[r] = out;
    }
}

}  // namespace

static size_t sample_smem(int V) { return (size_t)((V + 3) & ~3) * sizeof(float) + SAMPLE_MAX_K * sizeof(unsigned long long); }

bool sample_covered(int V, int top_k) {
    const int k = top_k < 1 ? 1 : (top_k > V ? V : top_k);
    return V > 0 && k <= SAMPLE_MAX_K && sample_smem(V) <= 220 * 1024;
}

bool launch_sample(cudaStream_t st, const float* logits, int M, int V, float temperature, int top_k, const double* uniform, uint32_t* next) {
    const size_t smem = sample_smem(V);
    if (!sample_covered(V, top_k) || !(temperature > 0.0f)) return false;
    const float inv_t = (float)(1.0 / (double)temperature);
    if (smem > 32 * 1024) cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_k(sample_kernel, dim3(M), dim3(SAMPLE_THREADS), smem, st, logits, V, inv_t, top_k, uniform, next);
    return true;
}

}  // namespace ava

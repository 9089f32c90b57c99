// The engram: one softmax attention read per token over every key/value stored so far (sm_100a).
//
// Follows the reference's one-token read (design-tests/nn/gpu/src/model/fstep.rs:303-356 and
// src/model/fstep/arch.rs:909-974): this token's key and value join the store first, then per head the scores
// K_j . q (row 0's product, then fma over the head's dimensions) times 1/sqrt(hs), the maximum, exp(s - max), the
// sum taken in key order from 0, each weight divided by it, and the mix p . V in gemm's one-row order over the keys.
// One block of threads per (row, group of heads); the group's scores live in shared memory.  Key rows are read with
// 16-byte loads, values sixteen keys at a time ahead of the chain, so the loads overlap while every sum keeps the
// reference's order.  The store is a ring per row so that an oldest-first cap (src/state.rs:526-538) drops a token by
// moving the start.
#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int ENG_THREADS = 256;

// Loads written as volatile asm stay where the source puts them: the compiler otherwise sinks a batch of loads down to
// their uses (to save registers) and an ordered chain then waits for each load in turn.  Plain ld.global, not the
// read-only path: the block reads the slot it has just written.
template <bool BF16>
__device__ __forceinline__ float kv_load(const void* base, size_t i) {
    if (BF16) {
        unsigned short h;
        asm volatile("ld.global.u16 %0, [%1];" : "=h"(h) : "l"(reinterpret_cast<const uint16_t*>(base) + i));
        return bf16_to_f(h);
    }
    float v;
    asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(reinterpret_cast<const float*>(base) + i));
    return v;
}
template <bool BF16>
__device__ __forceinline__ void kv_store(void* base, size_t i, float v) {
    if (BF16)
        reinterpret_cast<uint16_t*>(base)[i] = f_to_bf16(v);
    else
        reinterpret_cast<float*>(base)[i] = v;
}

// eight consecutive stored elements starting at element i (i a multiple of 8), widened to f32
template <bool BF16>
__device__ __forceinline__ void kv_load8(const void* base, size_t i, float* out) {
    if (BF16) {
        uint4 u;
        asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(reinterpret_cast<const uint16_t*>(base) + i));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            out[2 * k] = bits_to_f(w[k] << 16);
            out[2 * k + 1] = bits_to_f(w[k] & 0xffff0000u);
        }
    } else {
        float4 a, b;
        asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w) : "l"(reinterpret_cast<const float*>(base) + i));
        asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w) : "l"(reinterpret_cast<const float*>(base) + i + 4));
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    }
}

// out = fma(V_j, p_j, out) for the keys j0 .. j1 - 1, which sit hs elements apart from element `first`; sixteen values
// are fetched ahead of the chain, and the next sixteen while the chain runs.  HS > 0: hs known at compile time.
template <bool BF16, int HS>
__device__ __forceinline__ float pv_run(const void* v, size_t first, int hs_rt, const float* p, int j0, int j1, float out) {
    const int hs = HS ? HS : hs_rt;
    int j = j0;
    size_t at = first;
    if (j + 16 <= j1) {
        float t[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t[i] = kv_load<BF16>(v, at + (size_t)i * hs);
        for (; j + 32 <= j1; j += 16) {
            at += (size_t)16 * hs;
            float u[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) u[i] = kv_load<BF16>(v, at + (size_t)i * hs);
#pragma unroll
            for (int i = 0; i < 16; ++i) out = fma(t[i], p[j + i], out);
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = u[i];
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) out = fma(t[i], p[j + i], out);
        j += 16;
        at += (size_t)16 * hs;
    }
    for (; j < j1; ++j, at += hs) out = fma(kv_load<BF16>(v, at), p[j], out);
    return out;
}

// hg heads per block; grid = M * (nh / hg).  HS > 0: the head size, known at compile time (the loops unroll without
// bounds checks); HS == 0: any head size that is a multiple of 8.
template <bool BF16, int HS>
__global__ void __launch_bounds__(ENG_THREADS, HS ? 3 : 1) engram_kernel(const EngramArgs a, int hg) {
    pdl_enter();
    extern __shared__ float sm[];
    const int d = a.d, hs = HS ? HS : a.hs, nh = d / hs, cap = a.cap;
    const int groups = nh / hg;
    const int r = blockIdx.x / groups, h0 = (blockIdx.x % groups) * hg;
    const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarp = T >> 5;
    const float* qkv = a.qkv + (size_t)r * 3 * d;
    const size_t row_base = (size_t)r * nh * cap * hs;
    const int gd = hg * hs;  // channels of this group

    // the counts are read by every block of the row and written by none: a second small kernel moves them afterwards
    int n0 = a.n[r];
    const int start = a.start[r];
    if (n0 >= cap) {
        if (tid == 0) atomicOr(a.status, ST_ENGRAM_FULL);
        n0 = cap - 1;  // keep the kernel in bounds; the host reports the error
    }
    const int n = n0 + 1;
    int slot = start + n0;
    if (slot >= cap) slot -= cap;
    // this token's key and value join the store
    for (int c = tid; c < gd; c += T) {
        const int hh = h0 + c / hs, dd = c % hs;
        const size_t o = row_base + ((size_t)hh * cap + slot) * hs + dd;
        kv_store<BF16>(a.k, o, qkv[d + h0 * hs + c]);
        kv_store<BF16>(a.v, o, qkv[2 * d + h0 * hs + c]);
    }
    float* q = sm;              // [gd]
    float* mx = q + gd;         // [hg]
    float* den = mx + hg;       // [hg]
    float* sc = den + hg;       // [hg][n]
    for (int c = tid; c < gd; c += T) q[c] = qkv[h0 * hs + c];
    __syncthreads();  // the stores above are visible to this block's loads below

    // the ring as two straight runs: keys j < n1 sit at slots start + j, the others at slots j - n1
    const int n1 = min(n, cap - start);
    const float scale = (float)(1.0 / sqrt((double)hs));
    for (int g = 0; g < hg; ++g) {
        const float* qh = q + g * hs;
        const size_t head_base = row_base + (size_t)(h0 + g) * cap * hs;
        for (int j = tid; j < n; j += T) {
            const size_t o = head_base + (size_t)(j < n1 ? start + j : j - n1) * hs;
            float s = 0.0f;
            if (HS) {
#pragma unroll
                for (int x0 = 0; x0 < (HS ? HS : 8); x0 += 32) {
                    float kv[32];
#pragma unroll
                    for (int b = 0; b < 4; ++b)
                        if (x0 + 8 * b < HS) kv_load8<BF16>(a.k, o + x0 + 8 * b, kv + 8 * b);
#pragma unroll
                    for (int x = 0; x < 32; ++x)
                        if (x0 + x < HS) s = (x0 + x == 0) ? mul(kv[0], qh[0]) : fma(kv[x], qh[x0 + x], s);
                }
            } else {
                for (int x0 = 0; x0 < hs; x0 += 8) {
                    float kv[8];
                    kv_load8<BF16>(a.k, o + x0, kv);
#pragma unroll
                    for (int x = 0; x < 8; ++x) s = (x0 + x == 0) ? mul(kv[0], qh[0]) : fma(kv[x], qh[x0 + x], s);
                }
            }
            sc[(size_t)g * n + j] = add(mul(s, scale), 0.0f);
        }
    }
    __syncthreads();
    for (int g = warp; g < hg; g += nwarp) {
        float m = -INFINITY;
        for (int j = lane; j < n; j += 32) m = fmaxf(m, sc[(size_t)g * n + j]);
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) mx[g] = m;
    }
    __syncthreads();
    for (int g = 0; g < hg; ++g) {
        const float m = mx[g];
        for (int j = tid; j < n; j += T) sc[(size_t)g * n + j] = expf_(sub(sc[(size_t)g * n + j], m));
    }
    __syncthreads();
    for (int g = tid; g < hg; g += T) {
        float s = 0.0f;
        const float* p = sc + (size_t)g * n;
        for (int j = 0; j < n; ++j) s = add(s, p[j]);
        den[g] = s;
    }
    __syncthreads();
    for (int g = 0; g < hg; ++g) {
        const float dn = den[g];
        for (int j = tid; j < n; j += T) sc[(size_t)g * n + j] = div(sc[(size_t)g * n + j], dn);
    }
    __syncthreads();
    // o = p . V: per output the chain over the keys (src/model/fstep.rs:222-257 with k = n)
    for (int c = tid; c < gd; c += T) {
        const int g = c / hs, dd = c % hs;
        const float* p = sc + (size_t)g * n;
        const size_t hb = row_base + (size_t)(h0 + g) * cap * hs + dd;
        auto at = [&](int j) { return hb + (size_t)(j < n1 ? start + j : j - n1) * hs; };
        float out;
        if (n == 1) {
            out = mul(kv_load<BF16>(a.v, at(0)), p[0]);
        } else if (n == 2) {
            out = add(mul(kv_load<BF16>(a.v, at(1)), p[1]), mul(kv_load<BF16>(a.v, at(0)), p[0]));
        } else {
            out = mul(kv_load<BF16>(a.v, at(0)), p[0]);
            if (n1 > 1) out = pv_run<BF16, HS>(a.v, at(1), hs, p, 1, n1, out);
            const int j2 = max(n1, 1);
            if (j2 < n) out = pv_run<BF16, HS>(a.v, at(j2), hs, p, j2, n, out);
        }
        a.o[(size_t)r * d + h0 * hs + c] = out;
    }
}

// ---------------------------------------------------------------------------------------------------- streamed read
// The same read for the benchmark's store (bf16, heads of 64) with the keys and values streamed through shared memory:
// tiles are requested with cp.async one tile ahead of the arithmetic, so the chains never wait on global memory and the
// kernel runs at the rate the store can be read.  Keys: 256 per tile (one per thread), each key's eight 16-byte pieces
// stored at piece ^ (key & 7) so that a thread reading its own key's 128 bytes meets no bank conflict.  Values: 64 keys
// of all four heads per tile, read by one thread per output channel.  Every sum is the one the kernel above takes, in
// the same order: the same bits.
constexpr int ES_KT = 256;            // keys per key tile (one head)
constexpr int ES_VT = 64;             // keys per value tile (four heads)
constexpr int ES_TILE = ES_KT * 128;  // bytes of a tile: 256 keys x 128 B = 4 heads x 64 keys x 128 B

__device__ __forceinline__ void cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 lds_u4(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
}
__device__ __forceinline__ float lds_bf16(const uint16_t* p) {
    unsigned short h;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return bf16_to_f(h);
}

__global__ void __launch_bounds__(ENG_THREADS, 2) engram_stream_kernel(const EngramArgs a) {
    pdl_enter();
    extern __shared__ __align__(16) unsigned char es_smem[];
    constexpr int HS = 64, HG = 4;
    const int d = a.d, nh = d / HS, cap = a.cap, groups = nh / HG;
    const int r = blockIdx.x / groups, h0 = (blockIdx.x % groups) * HG;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* qkv = a.qkv + (size_t)r * 3 * d;
    const size_t row_base = (size_t)r * nh * cap * HS;
    uint16_t* Kst = reinterpret_cast<uint16_t*>(a.k);
    uint16_t* Vst = reinterpret_cast<uint16_t*>(a.v);

    int n0 = a.n[r];
    const int start = a.start[r];
    if (n0 >= cap) {
        if (tid == 0) atomicOr(a.status, ST_ENGRAM_FULL);
        n0 = cap - 1;
    }
    const int n = n0 + 1;
    int slot = start + n0;
    if (slot >= cap) slot -= cap;
    {   // this token's key and value join the store: thread = (head, channel)
        const int hh = h0 + (tid >> 6), dd = tid & 63;
        const size_t o = row_base + ((size_t)hh * cap + slot) * HS + dd;
        Kst[o] = f_to_bf16(qkv[d + h0 * HS + tid]);
        Vst[o] = f_to_bf16(qkv[2 * d + h0 * HS + tid]);
    }
    unsigned char* tile0 = es_smem;                       // two tiles
    float* q = reinterpret_cast<float*>(es_smem + 2 * ES_TILE);  // [256]
    float* mx = q + HG * HS;                              // [4]
    float* den = mx + HG;                                 // [4]
    float* sc = den + HG;                                 // [4][n]
    q[tid] = qkv[h0 * HS + tid];
    __syncthreads();  // the stores above are visible to this block's copies below

    const int n1 = min(n, cap - start);  // keys j < n1 sit at slots start + j, the others at slots j - n1
    auto slot_of = [&](int j) { return j < n1 ? start + j : j - n1; };

    // ---- scores: tiles of 256 keys of one head; tile index t = head * tiles_k + tile
    const int tiles_k = (n + ES_KT - 1) / ES_KT, total_k = HG * tiles_k;
    const int pc = tid & 7, pk = tid >> 3;  // a thread copies piece pc of the keys pk, pk + 32, ... of a tile
    auto fetch_k = [&](int t) {
        unsigned char* dst = tile0 + (size_t)(t & 1) * ES_TILE + pk * 128 + ((pc ^ (pk & 7)) << 4);  // (pk + 32 i) & 7 == pk & 7
        const int g = t / tiles_k, j0 = (t % tiles_k) * ES_KT;
        const uint16_t* head = Kst + row_base + (size_t)(h0 + g) * cap * HS + pc * 8;
        const int last = min(j0 + ES_KT, n) - 1;
        if (j0 >= n1 || last < n1) {
            // the tile's keys sit in one straight run of slots
            const uint16_t* src = head + (size_t)(slot_of(j0) + pk) * HS;
#pragma unroll
            for (int i = 0; i < ES_KT / 32; ++i)
                if (j0 + pk + 32 * i <= last) cp16(dst + i * 32 * 128, src + (size_t)i * 32 * HS);
        } else {
#pragma unroll
            for (int i = 0; i < ES_KT / 32; ++i) {
                const int j = j0 + pk + 32 * i;
                if (j <= last) cp16(dst + i * 32 * 128, head + (size_t)slot_of(j) * HS);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const float scale = (float)(1.0 / sqrt((double)HS));
    fetch_k(0);
    for (int t = 0; t < total_k; ++t) {
        if (t + 1 < total_k) {
            fetch_k(t + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int g = t / tiles_k, j = (t % tiles_k) * ES_KT + tid;
        if (j < n) {
            const unsigned char* key = tile0 + (size_t)(t & 1) * ES_TILE + tid * 128;
            const float* qh = q + g * HS;
            uint4 u[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) u[c] = lds_u4(key + ((c ^ (tid & 7)) << 4));
            float s = -0.0f;  // fma(k, q, -0) is the plain rounded product: the chain's first term
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t w[4] = {u[c].x, u[c].y, u[c].z, u[c].w};
                const float4 qa = *reinterpret_cast<const float4*>(qh + c * 8), qb = *reinterpret_cast<const float4*>(qh + c * 8 + 4);
                const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                for (int k2 = 0; k2 < 4; ++k2) {
                    s = fma(bits_to_f(w[k2] << 16), qv[2 * k2], s);
                    s = fma(bits_to_f(w[k2] & 0xffff0000u), qv[2 * k2 + 1], s);
                }
            }
            sc[(size_t)g * n + j] = add(mul(s, scale), 0.0f);
        }
        __syncthreads();
    }
    // ---- softmax per head, as above
    for (int g = warp; g < HG; g += ENG_THREADS / 32) {
        float m = -INFINITY;
        for (int j = lane; j < n; j += 32) m = fmaxf(m, sc[(size_t)g * n + j]);
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) mx[g] = m;
    }
    __syncthreads();
    // the first value tile is requested now, so that it arrives while the weights are formed
    const int tiles_v = (n + ES_VT - 1) / ES_VT;
    const size_t head_stride = (size_t)cap * HS;
    auto fetch_v = [&](int t) {
        // 4 heads x 64 keys x 8 pieces: a thread copies piece pc of the keys pk and pk + 32 of every head
        unsigned char* dst = tile0 + (size_t)(t & 1) * ES_TILE + pk * 128 + (pc << 4);
        const int j0 = t * ES_VT, last = min(j0 + ES_VT, n) - 1;
        const uint16_t* base = Vst + row_base + (size_t)h0 * head_stride + pc * 8;
        const bool straight = j0 >= n1 || last < n1;
        const int s0 = slot_of(j0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int gg = i >> 1, kk = pk + 32 * (i & 1), j = j0 + kk;
            if (j <= last) cp16(dst + (gg * ES_VT + 32 * (i & 1)) * 128, base + gg * head_stride + (size_t)(straight ? s0 + kk : slot_of(j)) * HS);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch_v(0);
    for (int g = 0; g < HG; ++g) {
        const float m = mx[g];
        for (int j = tid; j < n; j += ENG_THREADS) sc[(size_t)g * n + j] = expf_(sub(sc[(size_t)g * n + j], m));
    }
    __syncthreads();
    if (tid < HG) {
        float s = 0.0f;
        const float* p = sc + (size_t)tid * n;
        for (int j = 0; j < n; ++j) s = add(s, p[j]);
        den[tid] = s;
    }
    __syncthreads();
    for (int g = 0; g < HG; ++g) {
        const float dn = den[g];
        for (int j = tid; j < n; j += ENG_THREADS) sc[(size_t)g * n + j] = div(sc[(size_t)g * n + j], dn);
    }
    __syncthreads();
    // ---- o = p . V: the chain over the keys in order per output channel (src/model/fstep.rs:222-257 with k = n).  The
    // first 128 threads take two channels each (one 32-bit load per key); all threads keep the tiles coming.
    const int g = tid >> 5, pair = tid & 31;  // head and channel pair of a working thread (tid < 128)
    const bool works = tid < 128;
    const float* p = sc + (size_t)(works ? g : 0) * n;
    float o0 = -0.0f, o1 = -0.0f;  // fma from -0: the first term is the plain product (n >= 3; n of 1 and 2 below)
    for (int t = 0; t < tiles_v; ++t) {
        if (t + 1 < tiles_v) {
            fetch_v(t + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (works) {
            const uint32_t* vt = reinterpret_cast<const uint32_t*>(tile0 + (size_t)(t & 1) * ES_TILE) + (size_t)g * ES_VT * 32 + pair;
            const int j0 = t * ES_VT, cnt = min(ES_VT, n - j0);
            auto ldv = [&](int k) {
                uint32_t w;
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w) : "r"((uint32_t)__cvta_generic_to_shared(vt + (size_t)k * 32)));
                return w;
            };
            auto ldp = [&](int j) {
                float v;
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"((uint32_t)__cvta_generic_to_shared(p + j)));
                return v;
            };
            int b = 0;
            for (; b + 16 <= cnt; b += 16) {
                uint32_t w[16];
                float pj[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    w[i] = ldv(b + i);
                    pj[i] = ldp(j0 + b + i);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    o0 = fma(bits_to_f(w[i] << 16), pj[i], o0);
                    o1 = fma(bits_to_f(w[i] & 0xffff0000u), pj[i], o1);
                }
            }
            for (; b < cnt; ++b) {
                const uint32_t w = ldv(b);
                const float pj = ldp(j0 + b);
                o0 = fma(bits_to_f(w << 16), pj, o0);
                o1 = fma(bits_to_f(w & 0xffff0000u), pj, o1);
            }
        }
        __syncthreads();
    }
    if (works) {
        if (n == 2) {
            // two keys: (v1 p1) + (v0 p0), each product rounded (the reference's two-term form)
            const uint16_t* v0 = Vst + row_base + ((size_t)(h0 + g) * cap + slot_of(0)) * HS + 2 * pair;
            const uint16_t* v1 = Vst + row_base + ((size_t)(h0 + g) * cap + slot_of(1)) * HS + 2 * pair;
            o0 = add(mul(bf16_to_f(v1[0]), p[1]), mul(bf16_to_f(v0[0]), p[0]));
            o1 = add(mul(bf16_to_f(v1[1]), p[1]), mul(bf16_to_f(v0[1]), p[0]));
        }
        float* dst = a.o + (size_t)r * d + (h0 + g) * HS + 2 * pair;
        dst[0] = o0;
        dst[1] = o1;
    }
}

// ---------------------------------------------------------------------------------------------------- long stores
// For a store too long for one block's shared memory, or split by position over several GPUs, the read is taken in
// segments: each block takes one (row, head group, segment of keys) and leaves per head the partial softmax statistics
// (m, l, o[hs]): m the segment's largest score, l = sum exp(s - m), o = sum exp(s - m) v.  A second kernel merges the
// partials of all segments (of all GPUs, once gathered) in position order:
//     m = max m_p,  l = sum l_p e^(m_p - m),  o = sum o_p e^(m_p - m) / l.
// Within a segment the sums keep the reference's order; across segments the order of additions differs from the
// reference's single pass, so this path agrees with it to rounding (1e-6 relative), not bit for bit.
// partial layout: [row][head][segment][2 + hs] f32.
template <bool BF16>
__global__ void __launch_bounds__(ENG_THREADS) engram_partial_kernel(const EngramArgs a, int hg, int seg_len, int n_seg_max, float* partial) {
    pdl_enter();
    extern __shared__ float sm[];
    const int d = a.d, hs = a.hs, nh = d / hs, cap = a.cap;
    const int groups = nh / hg;
    const int seg = blockIdx.x % n_seg_max;
    const int r = (blockIdx.x / n_seg_max) / groups, h0 = ((blockIdx.x / n_seg_max) % groups) * hg;
    const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarp = T >> 5;
    const float* qkv = a.qkv + (size_t)r * 3 * d;
    const size_t row_base = (size_t)r * nh * cap * hs;
    const int gd = hg * hs;
    const int n_all = min(a.n[r], cap), start = a.start[r];
    const int j0 = seg * seg_len, n = min(seg_len, n_all - j0);  // this segment's keys: logical positions j0 .. j0 + n
    float* q = sm;          // [gd]
    float* mx = q + gd;     // [hg]
    float* sc = mx + hg;    // [hg][n]
    auto out = [&](int g) { return partial + ((((size_t)r * nh + h0 + g) * n_seg_max + seg) * (2 + hs)); };
    if (n <= 0) {           // an empty segment contributes nothing: m = -inf, l = 0
        for (int c = tid; c < hg * (2 + hs); c += T) out(c / (2 + hs))[c % (2 + hs)] = (c % (2 + hs)) == 0 ? -INFINITY : 0.0f;
        return;
    }
    for (int c = tid; c < gd; c += T) q[c] = qkv[h0 * hs + c];
    __syncthreads();
    const float scale = (float)(1.0 / sqrt((double)hs));
    for (int idx = tid; idx < hg * n; idx += T) {
        const int g = idx / n, j = idx % n;
        int pj = start + j0 + j;
        if (pj >= cap) pj -= cap;
        const size_t o = row_base + ((size_t)(h0 + g) * cap + pj) * hs;
        const float* qh = q + g * hs;
        float s = 0.0f;
        for (int x0 = 0; x0 < hs; x0 += 32) {
            float kv[32];
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (x0 + 8 * b < hs) kv_load8<BF16>(a.k, o + x0 + 8 * b, kv + 8 * b);
#pragma unroll
            for (int x = 0; x < 32; ++x) {
                if (x0 + x < hs) s = (x0 + x == 0) ? mul(kv[0], qh[0]) : fma(kv[x], qh[x0 + x], s);
            }
        }
        sc[(size_t)g * n + j] = add(mul(s, scale), 0.0f);
    }
    __syncthreads();
    for (int g = warp; g < hg; g += nwarp) {
        float m = -INFINITY;
        for (int j = lane; j < n; j += 32) m = fmaxf(m, sc[(size_t)g * n + j]);
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) mx[g] = m;
    }
    __syncthreads();
    for (int idx = tid; idx < hg * n; idx += T) sc[idx] = expf_(sub(sc[idx], mx[idx / n]));
    __syncthreads();
    for (int g = tid; g < hg; g += T) {
        float s = 0.0f;
        const float* p = sc + (size_t)g * n;
        for (int j = 0; j < n; ++j) s = add(s, p[j]);
        out(g)[0] = mx[g];
        out(g)[1] = s;
    }
    for (int c = tid; c < gd; c += T) {
        const int g = c / hs, dd = c % hs;
        const float* p = sc + (size_t)g * n;
        const size_t hb = row_base + (size_t)(h0 + g) * cap * hs + dd;
        auto V = [&](int j) {
            int pj = start + j0 + j;
            if (pj >= cap) pj -= cap;
            return kv_load<BF16>(a.v, hb + (size_t)pj * hs);
        };
        float o = -0.0f;
        int j = 0;
        for (; j + 16 <= n; j += 16) {
            float t[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = V(j + i);
#pragma unroll
            for (int i = 0; i < 16; ++i) o = fma(t[i], p[j + i], o);
        }
        for (; j < n; ++j) o = fma(V(j), p[j], o);
        out(g)[2 + dd] = o;
    }
}

// partial [group][row][head][n_part][2 + hs] -> o [row][nh * hs]; one thread per output channel walks the groups (the
// GPUs a store is split over, in position order) and within each its parts in order
__global__ void engram_combine_kernel(const float* __restrict__ partial, int M, int nh, int hs, int n_part, int n_groups, float* __restrict__ o) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * nh * hs) return;
    const int dd = i % hs, rh = i / hs;  // rh = row * nh + head
    const size_t part = 2 + hs, gstride = (size_t)M * nh * n_part * part;
    const float* p = partial + (size_t)rh * n_part * part;
    float m = -INFINITY;
    for (int g = 0; g < n_groups; ++g)
        for (int k = 0; k < n_part; ++k) m = fmaxf(m, p[g * gstride + (size_t)k * part]);
    float l = 0.0f, acc = 0.0f;
    for (int g = 0; g < n_groups; ++g)
        for (int k = 0; k < n_part; ++k) {
            const float* pk = p + g * gstride + (size_t)k * part;
            if (pk[1] == 0.0f) continue;  // an empty part
            const float w = expf_(sub(pk[0], m));
            l = add(l, mul(pk[1], w));
            acc = add(acc, mul(pk[2 + dd], w));
        }
    o[i] = div(acc, l);
}

// this token's key and value join the store (the long path appends first, then reads every segment)
template <bool BF16>
__global__ void engram_append_kernel(const EngramArgs a) {
    pdl_enter();
    const int d = a.d, hs = a.hs, nh = d / hs, cap = a.cap;
    const int r = blockIdx.x;
    const int n0 = a.n[r];
    if (n0 >= cap) {
        if (threadIdx.x == 0) atomicOr(a.status, ST_ENGRAM_FULL);
        return;
    }
    int slot = a.start[r] + n0;
    if (slot >= cap) slot -= cap;
    const float* qkv = a.qkv + (size_t)r * 3 * d;
    const size_t row_base = (size_t)r * nh * cap * hs;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const size_t o = row_base + ((size_t)(c / hs) * cap + slot) * hs + c % hs;
        kv_store<BF16>(a.k, o, qkv[d + c]);
        kv_store<BF16>(a.v, o, qkv[2 * d + c]);
    }
}
// n <- n + 1 after an append (the partial kernels read n as the number of keys present)
__global__ void engram_count_kernel(int32_t* n, int M, int cap) {
    pdl_enter();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < M && n[r] < cap) n[r] += 1;
}
// a capped store drops its oldest tokens after the read
__global__ void engram_trim_kernel(int32_t* n, int32_t* start, int M, int cap, int keep) {
    pdl_enter();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= M) return;
    if (n[r] > keep) {
        start[r] = (start[r] + (n[r] - keep)) % cap;
        n[r] = keep;
    }
}

// after the read: the count moves on; a capped store drops its oldest tokens (src/state.rs:526-538)
__global__ void engram_advance_kernel(int32_t* n, int32_t* start, int M, int cap, int keep) {
    pdl_enter();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= M) return;
    int n0 = n[r];
    if (n0 >= cap) n0 = cap - 1;
    const int nn = n0 + 1;
    if (nn > keep) {
        n[r] = keep;
        start[r] = (start[r] + (nn - keep)) % cap;
    } else {
        n[r] = nn;
    }
}

}  // namespace

static int head_group(int nh, int hs);

bool launch_engram(cudaStream_t st, const EngramArgs& a, int n_max) {
    const int nh = a.d / a.hs;
    if (a.hs % 8 != 0) return false;
    // heads per block: as many as give each thread one output channel, dividing the head count
    const int hg = head_group(nh, a.hs);
    const size_t smem = ((size_t)hg * a.hs + 2 * hg + (size_t)hg * n_max) * sizeof(float);
    if (smem > 227 * 1024 - 64) return false;
    const unsigned grid = (unsigned)(a.M * (nh / hg));
    if (a.bf16 && a.hs == 64 && hg == 4) {
        // the streamed form: two tiles of 32 KB beside the scores
        const size_t ssmem = 2 * (size_t)ES_TILE + ((size_t)hg * a.hs + 2 * hg + (size_t)hg * n_max) * sizeof(float);
        if (ssmem <= 227 * 1024 - 64) {
            cudaFuncSetAttribute(engram_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ssmem);
            launch_k(engram_stream_kernel, dim3(grid), dim3(ENG_THREADS), ssmem, st, a);
            launch_k(engram_advance_kernel, dim3((a.M + 127) / 128), dim3(128), 0, st, a.n, a.start, a.M, a.cap, a.keep);
            return true;
        }
    }
    auto go = [&](auto kernel) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(kernel, dim3(grid), dim3(ENG_THREADS), smem, st, a, hg);
    };
    if (a.bf16) {
        if (a.hs == 64) go(engram_kernel<true, 64>);
        else if (a.hs == 32) go(engram_kernel<true, 32>);
        else go(engram_kernel<true, 0>);
    } else {
        if (a.hs == 64) go(engram_kernel<false, 64>);
        else if (a.hs == 32) go(engram_kernel<false, 32>);
        else go(engram_kernel<false, 0>);
    }
    launch_k(engram_advance_kernel, dim3((a.M + 127) / 128), dim3(128), 0, st, a.n, a.start, a.M, a.cap, a.keep);
    return true;
}

static int head_group(int nh, int hs) {
    int hg = ENG_THREADS / hs;
    if (hg < 1) hg = 1;
    if (hg > nh) hg = nh;
    while (nh % hg != 0) --hg;
    return hg;
}

void launch_engram_append(cudaStream_t st, const EngramArgs& a) {
    if (a.bf16) launch_k(engram_append_kernel<true>, dim3(a.M), dim3(256), 0, st, a); else launch_k(engram_append_kernel<false>, dim3(a.M), dim3(256), 0, st, a);
    launch_k(engram_count_kernel, dim3((a.M + 127) / 128), dim3(128), 0, st, a.n, a.M, a.cap);
}

void launch_engram_trim(cudaStream_t st, const EngramArgs& a) {
    launch_k(engram_trim_kernel, dim3((a.M + 127) / 128), dim3(128), 0, st, a.n, a.start, a.M, a.cap, a.keep);
}

bool engram_fits_one_block(int d, int hs, int n_max) {
    const int hg = head_group(d / hs, hs);
    return ((size_t)hg * hs + 2 * hg + (size_t)hg * n_max) * sizeof(float) <= 227 * 1024 - 64;
}

int engram_segments(int n_max, int seg_len) { return (n_max + seg_len - 1) / seg_len; }

bool launch_engram_partial(cudaStream_t st, const EngramArgs& a, int seg_len, int n_seg, float* partial) {
    const int nh = a.d / a.hs;
    if (a.hs % 8 != 0 || n_seg <= 0) return false;
    const int hg = head_group(nh, a.hs);
    const size_t smem = ((size_t)hg * a.hs + hg + (size_t)hg * seg_len) * sizeof(float);
    if (smem > 227 * 1024 - 64) return false;
    const unsigned grid = (unsigned)((size_t)a.M * (nh / hg) * n_seg);
    if (a.bf16) {
        cudaFuncSetAttribute(engram_partial_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(engram_partial_kernel<true>, dim3(grid), dim3(ENG_THREADS), smem, st, a, hg, seg_len, n_seg, partial);
    } else {
        cudaFuncSetAttribute(engram_partial_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(engram_partial_kernel<false>, dim3(grid), dim3(ENG_THREADS), smem, st, a, hg, seg_len, n_seg, partial);
    }
    return true;
}

void launch_engram_combine(cudaStream_t st, const float* partial, int M, int nh, int hs, int n_part, float* o, int n_groups) {
    const int n = M * nh * hs;
    launch_k(engram_combine_kernel, dim3((n + 127) / 128), dim3(128), 0, st, partial, M, nh, hs, n_part, n_groups, o);
}

}  // namespace ava

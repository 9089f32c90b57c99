// Ordered sums over a row held in shared memory, shared by the per-row kernels and by the products for a few rows that
// take a row's norm in their prologue.  "One value after another from 0" (design-tests/nn/gpu/src/model/fstep.rs:12-14):
// one thread takes the sum in that order; the loads run ahead of the chain.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "ava_math.h"

namespace ava {
namespace {

constexpr float NORM_EPS = 1e-5f;  // src/model.rs:36

// Shared-memory loads that stay where they are written: the compiler otherwise sinks a prefetch down to its use and the
// ordered chains below then wait for every load in turn.
__device__ __forceinline__ float lds1(const float* p) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
}
__device__ __forceinline__ float4 lds4(const float* p) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
}

// sum of x[i]^2 one after another from 0; x in shared memory, 16-byte aligned.  Eight values are fetched ahead of the
// chain so that the loads overlap; the order of the additions is the reference's.
__device__ __forceinline__ float sumsq_seq(const float* x, int n) {
    float s = 0.0f;
    int i = 0;
    if (n >= 8) {
        float4 a = lds4(x), b = lds4(x + 4);
        for (; i + 16 <= n; i += 8) {
            const float4 na = lds4(x + i + 8), nb = lds4(x + i + 12);
            const float p[8] = {mul(a.x, a.x), mul(a.y, a.y), mul(a.z, a.z), mul(a.w, a.w), mul(b.x, b.x), mul(b.y, b.y), mul(b.z, b.z), mul(b.w, b.w)};
#pragma unroll
            for (int k = 0; k < 8; ++k) s = add(s, p[k]);
            a = na;
            b = nb;
        }
        const float p[8] = {mul(a.x, a.x), mul(a.y, a.y), mul(a.z, a.z), mul(a.w, a.w), mul(b.x, b.x), mul(b.y, b.y), mul(b.z, b.z), mul(b.w, b.w)};
#pragma unroll
        for (int k = 0; k < 8; ++k) s = add(s, p[k]);
        i += 8;
    }
    for (; i < n; ++i) s = add(s, mul(x[i], x[i]));
    return s;
}

// sum of a[i] * b[i] one after another from 0 (shared memory, 16-byte aligned); the next eight products are formed
// while the chain adds the eight before
__device__ __forceinline__ float dot_seq(const float* a, const float* b, int n) {
    float s = 0.0f;
    int i = 0;
    if (n >= 8) {
        auto prods = [&](int at, float* p) {
            const float4 a0 = lds4(a + at), a1 = lds4(a + at + 4), b0 = lds4(b + at), b1 = lds4(b + at + 4);
            p[0] = mul(a0.x, b0.x); p[1] = mul(a0.y, b0.y); p[2] = mul(a0.z, b0.z); p[3] = mul(a0.w, b0.w);
            p[4] = mul(a1.x, b1.x); p[5] = mul(a1.y, b1.y); p[6] = mul(a1.z, b1.z); p[7] = mul(a1.w, b1.w);
        };
        float p[8];
        prods(0, p);
        for (; i + 16 <= n; i += 8) {
            float np[8];
            prods(i + 8, np);
#pragma unroll
            for (int k = 0; k < 8; ++k) s = add(s, p[k]);
#pragma unroll
            for (int k = 0; k < 8; ++k) p[k] = np[k];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) s = add(s, p[k]);
        i += 8;
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

// One weight byte from shared memory as a float: load and conversion in one statement, so that the conversion stays
// with the load ahead of the chain that uses it.  (The conversion by bit tricks instead, three ALU instructions and no
// conversion instruction, measured slower: the chains are short of issue slots, not of the conversion unit.)
__device__ __forceinline__ float lds_s8f(const int8_t* p) {
    float f;
    asm volatile("{\n\t.reg .s32 t;\n\tld.shared.s8 t, [%1];\n\tcvt.rn.f32.s32 %0, t;\n\t}" : "=f"(f) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return f;
}

// acc = fma(x[k], w[k], acc) for k = 0 .. K-1 in order: x [K] f32 and the column's weight bytes w[k] at wp[k * STRIDE],
// both in shared memory (x 16-byte aligned).  Sixteen terms are fetched and converted while the sixteen before them
// join the chain (a shared-memory load and a conversion take longer than four dependent multiply-adds, so a shorter
// look-ahead leaves the chain waiting).  The order of the multiply-adds is k's.
template <int STRIDE>
__device__ __forceinline__ float chain_s8(const float* x, const int8_t* wp, int K, float acc) {
    // two register sets of sixteen terms take turns (no copies between them: one warp alone is short of issue slots,
    // and every instruction beside the multiply-add lengthens the chain)
    float wa[16], wb[16];
    float4 xa[4], xb[4];
    auto load_a = [&](int g) {
#pragma unroll
        for (int u = 0; u < 16; ++u) wa[u] = lds_s8f(wp + (size_t)(16 * g + u) * STRIDE);
#pragma unroll
        for (int u = 0; u < 4; ++u) xa[u] = lds4(x + 16 * g + 4 * u);
    };
    auto load_b = [&](int g) {
#pragma unroll
        for (int u = 0; u < 16; ++u) wb[u] = lds_s8f(wp + (size_t)(16 * g + u) * STRIDE);
#pragma unroll
        for (int u = 0; u < 4; ++u) xb[u] = lds4(x + 16 * g + 4 * u);
    };
    const int G = K / 16;
    int g = 0;
    if (G > 0) load_a(0);
    while (g + 2 <= G) {
        load_b(g + 1);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            acc = fma(xa[u].x, wa[4 * u], acc);
            acc = fma(xa[u].y, wa[4 * u + 1], acc);
            acc = fma(xa[u].z, wa[4 * u + 2], acc);
            acc = fma(xa[u].w, wa[4 * u + 3], acc);
        }
        if (g + 2 < G) load_a(g + 2);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            acc = fma(xb[u].x, wb[4 * u], acc);
            acc = fma(xb[u].y, wb[4 * u + 1], acc);
            acc = fma(xb[u].z, wb[4 * u + 2], acc);
            acc = fma(xb[u].w, wb[4 * u + 3], acc);
        }
        g += 2;
    }
    if (g < G) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            acc = fma(xa[u].x, wa[4 * u], acc);
            acc = fma(xa[u].y, wa[4 * u + 1], acc);
            acc = fma(xa[u].z, wa[4 * u + 2], acc);
            acc = fma(xa[u].w, wa[4 * u + 3], acc);
        }
    }
    for (int k = 16 * G; k < K; ++k) acc = fma(lds1(x + k), lds_s8f(wp + (size_t)k * STRIDE), acc);
    return acc;
}

// the order-preserving integer key of a float (k-winners-take-all's radix select) and back
__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = f_to_bits(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) { return bits_to_f((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); }

}  // namespace
}  // namespace ava

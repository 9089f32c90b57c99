// exp, ln and x^-1/2 written out in IEEE single-precision operations only (multiply, add, fused multiply-add,
// round-to-integer, square root, divide, integer bit moves), so that the host build and the device build of this file
// return the same bits for the same input.  The engine uses these wherever the reference calls the platform's
// exp / ln / powf(-0.5) (design-tests/nn/gpu/src/model/fstep.rs:212-292); the host versions are exported from the
// library so that a checker can plug the very same functions into its own arithmetic.
//
// Compile the device side with -fmad=false and the host side with -ffp-contract=off: no multiply-add may be fused
// unless it is written fmaf here.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define AVA_HD __host__ __device__ __forceinline__
#else
#define AVA_HD inline
#endif

namespace ava {

AVA_HD float bits_to_f(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}

AVA_HD uint32_t f_to_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}

// separately rounded multiply / add (never contracted), fused multiply-add, correctly rounded divide and root
AVA_HD float mul(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    return a * b;
#endif
}
AVA_HD float add(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}
AVA_HD float sub(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fsub_rn(a, b);
#else
    return a - b;
#endif
}
AVA_HD float fma(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
    return __fmaf_rn(a, b, c);
#else
    return ::fmaf(a, b, c);
#endif
}
AVA_HD float div(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fdiv_rn(a, b);
#else
    return a / b;
#endif
}
AVA_HD float root(float a) {
#if defined(__CUDA_ARCH__)
    return __fsqrt_rn(a);
#else
    return ::sqrtf(a);
#endif
}

// 2^n for n in [-126, 127]
AVA_HD float pow2i(int n) { return bits_to_f((uint32_t)(n + 127) << 23); }

// e^x: x = n ln2 + r, |r| <= ln2/2, a degree-6 polynomial in r, then two exact scalings by powers of two (two, so
// that results in the subnormal range round once, at the last multiply).
AVA_HD float expf_(float x) {
    if (x != x) return bits_to_f(0x7fc00000u);
    if (x > 88.72283935546875f) return bits_to_f(0x7f800000u);
    if (x < -103.972076416015625f) return 0.0f;
    const float n = ::rintf(mul(x, 1.44269504088896341f));
    float r = fma(n, -0.693359375f, x);
    r = fma(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fma(p, r, 1.3981999507e-3f);
    p = fma(p, r, 8.3334519073e-3f);
    p = fma(p, r, 4.1665795894e-2f);
    p = fma(p, r, 1.6666665459e-1f);
    p = fma(p, r, 5.0000001201e-1f);
    const float z = mul(r, r);
    float y = fma(p, z, r);
    y = add(y, 1.0f);
    const int ni = (int)n;
    const int h = ni / 2;
    return mul(mul(y, pow2i(h)), pow2i(ni - h));
}

// ln x for finite x > 0 (else the IEEE special values): x = m 2^e with m in [sqrt(1/2), sqrt 2), a degree-8
// polynomial in m - 1.
AVA_HD float logf_(float x) {
    if (x != x) return bits_to_f(0x7fc00000u);
    if (x < 0.0f) return bits_to_f(0x7fc00000u);
    if (x == 0.0f) return bits_to_f(0xff800000u);
    uint32_t u = f_to_bits(x);
    if (u == 0x7f800000u) return x;
    int e = 0;
    if (u < 0x00800000u) {  // subnormal: scale up by 2^23 first
        x = mul(x, 8388608.0f);
        u = f_to_bits(x);
        e = -23;
    }
    e += (int)(u >> 23) - 126;
    float m = bits_to_f((u & 0x007fffffu) | 0x3f000000u);  // [0.5, 1)
    if (m < 0.707106781186547524f) {
        e -= 1;
        m = sub(add(m, m), 1.0f);
    } else {
        m = sub(m, 1.0f);
    }
    const float z = mul(m, m);
    float p = 7.0376836292e-2f;
    p = fma(p, m, -1.1514610310e-1f);
    p = fma(p, m, 1.1676998740e-1f);
    p = fma(p, m, -1.2420140846e-1f);
    p = fma(p, m, 1.4249322787e-1f);
    p = fma(p, m, -1.6668057665e-1f);
    p = fma(p, m, 2.0000714765e-1f);
    p = fma(p, m, -2.4999993993e-1f);
    p = fma(p, m, 3.3333331174e-1f);
    float y = mul(mul(p, m), z);
    const float fe = (float)e;
    y = fma(fe, -2.12194440e-4f, y);
    y = fma(-0.5f, z, y);
    float r = add(m, y);
    r = fma(fe, 0.693359375f, r);
    return r;
}

// x^-1/2 as 1 / sqrt(x), both correctly rounded
AVA_HD float rsqrtf_(float x) { return div(1.0f, root(x)); }

// the reference's compositions (design-tests/nn/gpu/src/model/fstep.rs:260-268)
AVA_HD float sigmoid(float x) { return div(1.0f, add(mul(expf_(-x), 1.0f), 1.0f)); }
AVA_HD float log_sigmoid(float x) {
    const float soft = logf_(add(mul(expf_(-fabsf(x)), 1.0f), 1.0f));
    return -add(fmaxf(-x, 0.0f), soft);
}

// tanh from the shared exp: (1 - e^(-2|x|)) / (1 + e^(-2|x|)) with the sign of x; x itself below 2^-12 (the cubic term is
// under half an ulp there), +-1 above 9.5.  The gains of the dendrites are 1 + tanh (src/model/fstep/arch_f4.rs:34-37).
AVA_HD float tanhf_(float x) {
    const float ax = fabsf(x);
    if (!(ax == ax)) return bits_to_f(0x7fc00000u);
    if (ax < 2.44140625e-4f) return x;
    if (ax > 9.5f) return x > 0.0f ? 1.0f : -1.0f;
    const float t = expf_(mul(ax, -2.0f));
    const float r = div(sub(1.0f, t), add(1.0f, t));
    return x < 0.0f ? -r : r;
}

// float -> bf16 bits, round to nearest even; NaN stays NaN
AVA_HD uint16_t f_to_bf16(float x) {
    uint32_t u = f_to_bits(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
AVA_HD float bf16_to_f(uint16_t h) { return bits_to_f((uint32_t)h << 16); }

}  // namespace ava

namespace ava {

// sine and cosine of a float, computed in IEEE double operations only (multiply, add, fused multiply-add, round to
// integer) and rounded to float once at the end, so that host and device give the same bits.  --rhythm's phases are
// the one place the step needs them (design-tests/nn/gpu/src/model/fstep/arch_f4.rs:84-89, where the reference calls
// the platform's cosf / sinf).  The argument is reduced by the nearest multiple n of pi/2, pi/2 split into three parts
// whose first two have 33 significant bits (n * part is exact for |n| < 2^20, i.e. |x| below about 1.6e6; beyond that
// the reduction loses accuracy gradually, still the same on both sides); on |r| <= pi/4 the Taylor series to r^19 and
// r^18 (the next terms are below 1e-19).
AVA_HD double dmul(double a, double b) {
#if defined(__CUDA_ARCH__)
    return __dmul_rn(a, b);
#else
    return a * b;
#endif
}
AVA_HD double dadd(double a, double b) {
#if defined(__CUDA_ARCH__)
    return __dadd_rn(a, b);
#else
    return a + b;
#endif
}
AVA_HD double dfma(double a, double b, double c) {
#if defined(__CUDA_ARCH__)
    return __fma_rn(a, b, c);
#else
    return ::fma(a, b, c);
#endif
}

// quadrant (n mod 4) and sin(r), cos(r) of the reduced argument
AVA_HD void sincos_parts(float xf, int* quad, double* s, double* c) {
    const double x = (double)xf;
    const double n = rint(dmul(x, 0.63661977236758134308));  // 2 / pi
    // pi/2 = P1 + P2 + P3 (+ ...), P1 and P2 with 33 significant bits
    const double P1 = 1.57079632673412561417, P2 = 6.07710050630396597660e-11, P3 = 2.02226624879595063154e-21;
    double r = dfma(-n, P1, x);
    r = dfma(-n, P2, r);
    r = dfma(-n, P3, r);
    const double r2 = dmul(r, r);
    // sin r = r (1 - r2/3! + r2^2/5! - ... + r2^9/19!), cos r = 1 - r2/2! + ... + r2^9/18!, by Horner's rule
    double ps = -1.0 / 121645100408832000.0;                  // -1/19!
    ps = dfma(ps, r2, 1.0 / 355687428096000.0);              // 1/17!
    ps = dfma(ps, r2, -1.0 / 1307674368000.0);               // -1/15!
    ps = dfma(ps, r2, 1.0 / 6227020800.0);                   // 1/13!
    ps = dfma(ps, r2, -1.0 / 39916800.0);                    // -1/11!
    ps = dfma(ps, r2, 1.0 / 362880.0);                       // 1/9!
    ps = dfma(ps, r2, -1.0 / 5040.0);                        // -1/7!
    ps = dfma(ps, r2, 1.0 / 120.0);                          // 1/5!
    ps = dfma(ps, r2, -1.0 / 6.0);                           // -1/3!
    ps = dfma(ps, r2, 1.0);
    double pc = -1.0 / 6402373705728000.0;                   // -1/18!
    pc = dfma(pc, r2, 1.0 / 20922789888000.0);               // 1/16!
    pc = dfma(pc, r2, -1.0 / 87178291200.0);                 // -1/14!
    pc = dfma(pc, r2, 1.0 / 479001600.0);                    // 1/12!
    pc = dfma(pc, r2, -1.0 / 3628800.0);                     // -1/10!
    pc = dfma(pc, r2, 1.0 / 40320.0);                        // 1/8!
    pc = dfma(pc, r2, -1.0 / 720.0);                         // -1/6!
    pc = dfma(pc, r2, 1.0 / 24.0);                           // 1/4!
    pc = dfma(pc, r2, -0.5);
    pc = dfma(pc, r2, 1.0);
    *s = dmul(r, ps);
    *c = pc;
    *quad = (int)((long long)n & 3);
}

AVA_HD float sinf_(float x) {
    if (!(fabsf(x) < 3.0e38f)) return bits_to_f(0x7fc00000u);  // infinities and NaN
    int q;
    double s, c;
    sincos_parts(x, &q, &s, &c);
    const double v = q == 0 ? s : q == 1 ? c : q == 2 ? -s : -c;
    return (float)v;
}

AVA_HD float cosf_(float x) {
    if (!(fabsf(x) < 3.0e38f)) return bits_to_f(0x7fc00000u);
    int q;
    double s, c;
    sincos_parts(x, &q, &s, &c);
    const double v = q == 0 ? c : q == 1 ? -s : q == 2 ? -c : s;
    return (float)v;
}

}  // namespace ava

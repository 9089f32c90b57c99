// The fast-weight memory over a chunk of tokens in its chunk-parallel form, the big products on the tensor cores
// (sm_100a).  Optional, for prompt reading in the tolerance mode: it follows the reference's `delta_chunk` /
// `chunk_core` (design-tests/nn/gpu/src/arch.rs:1151-1173, 1243-1327) for per-channel gates without momentum, and like
// it agrees with the token loop to rounding only (the reference's own bound for this form: 1e-4 of max(1, max|ref|),
// src/arch/tests.rs:700-753), not bit for bit.
//
// Per head and chunk of C = 64 tokens (positions i, j inside the chunk; cum = inclusive sums of log alpha per channel,
// cumex = the sums before a position; q, e unit; w = k b the write key, ah = e (b alpha) the erase key):
//     qs = q exp(cum)        es = e exp(cumex)        ws = w exp(-cum)        as = ah exp(-cum)
//     Qw = tril(qs ws^T)     Qa = tril(qs as^T)       Ke = stril(es ws^T)     Ae = stril(es as^T)       one 128x128xhs product
//     T  = (I + Ae)^-1       p1 = T es                r0 = (T Ke) v           qwv = Qw v      (r0 and qwv inside the state read, below)
//     wl = w exp(cum_C - cum)   al = ah exp(cum_C - cum)   gc = exp(cum_C)
// then, chunk after chunk with the state F [key, value]:
//     [rr; yw] = [p1 | T Ke; qs | Qw] [F; v]           128 x (hs + 64) x hs on the tensor cores: rr = p1 F + r0, yw = qs F + qwv
//     y = yw - Qa rr
//     F' = diag(gc) F + wl^T v - al^T rr               hs x hs x 128 on the tensor cores
// The pairwise decays exp(cum_i - cum_j) are formed as products exp(cum_i) exp(-cum_j) so that the Gram matrices are
// plain products; that is safe while the sums stay within the f32 exponent range over one chunk.  The scaling kernel
// raises a flag when a chunk's sum of log rates falls below -60 (forgetting by a factor 1e-26 inside 64 tokens); the
// caller then reads that chunk of tokens with the exact kernels instead.
//
// The state is worked on transposed, Ft [value, key] with its three bf16 limbs beside it, because both big products
// want their operands K-major: the first sums over keys (rows of Ft are K-major as they lie), the second over the
// chunk's 128 token slots.  All f32 operands of the tensor-core products are carried as three bf16 limbs (k_tcb.cu).
#include <cuda_runtime.h>

#include <algorithm>

#include "ava_math.h"
#include "bf16_hw.cuh"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int CC = 64;  // tokens per chunk

__device__ __forceinline__ void limbs3(float x, uint16_t& l0, uint16_t& l1, uint16_t& l2) { limbs3_hw(x, l0, l1, l2); }

// ---- scaling, in three kernels ------------------------------------------------------------------------------------
// (1) the running sums of the log rates: one thread per (chunk, head, channel), the chunk's 64 tokens in order
__global__ void __launch_bounds__(256) chunk_scan_kernel(const ChunkArgs a) {
    pdl_enter();
    const int H = a.hs, ch = blockIdx.x * blockDim.x + threadIdx.x;
    if (ch >= H) return;
    const int u = blockIdx.y, j = u / a.HB, hb = u % a.HB;  // u = j * HB + hb
    const size_t in0 = (size_t)j * CC * a.tok_stride + (size_t)hb * H + ch;
    float cum = 0.0f, mincum = 0.0f;
    for (int i8 = 0; i8 < CC; i8 += 8) {
        float la[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) la[q] = __ldg(a.la + in0 + (size_t)(i8 + q) * a.tok_stride);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            cum += la[q];
            mincum = fminf(mincum, cum);
            a.CUM[((size_t)u * 64 + i8 + q) * H + ch] = cum;
        }
    }
    if (mincum < -60.0f || !(cum == cum)) atomicOr(a.flags, 1u);
    a.gc[(size_t)u * H + ch] = __expf(cum);
}

__device__ __forceinline__ void limbs3x4(const float4 x, uint2& p0, uint2& p1, uint2& p2) {
    uint16_t l[3][4];
    limbs3(x.x, l[0][0], l[1][0], l[2][0]);
    limbs3(x.y, l[0][1], l[1][1], l[2][1]);
    limbs3(x.z, l[0][2], l[1][2], l[2][2]);
    limbs3(x.w, l[0][3], l[1][3], l[2][3]);
    p0 = make_uint2(l[0][0] | ((uint32_t)l[0][1] << 16), l[0][2] | ((uint32_t)l[0][3] << 16));
    p1 = make_uint2(l[1][0] | ((uint32_t)l[1][1] << 16), l[1][2] | ((uint32_t)l[1][3] << 16));
    p2 = make_uint2(l[2][0] | ((uint32_t)l[2][1] << 16), l[2][2] | ((uint32_t)l[2][3] << 16));
}

// (2) the scaled rows, token-major: one thread per (chunk, head, token, four channels)
__global__ void __launch_bounds__(256) chunk_scale_kernel(const ChunkArgs a) {
    pdl_enter();
    const int H = a.hs, H4 = H / 4;
    const size_t n = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= (size_t)a.nC * a.HB * 64 * H4) return;
    const int c4 = (int)(n % H4) * 4, i = (int)((n / H4) % 64), u = (int)(n / ((size_t)H4 * 64)), j = u / a.HB, hb = u % a.HB;
    const size_t at = (size_t)(j * CC + i) * a.tok_stride + (size_t)hb * H + c4;
    const float4 q = *reinterpret_cast<const float4*>(a.qn + at), e = *reinterpret_cast<const float4*>(a.e + at);
    const float4 w = *reinterpret_cast<const float4*>(a.w + at), ah = *reinterpret_cast<const float4*>(a.ah + at);
    const float4 cum = *reinterpret_cast<const float4*>(a.CUM + ((size_t)u * 64 + i) * H + c4);
    const float4 cumex = i > 0 ? *reinterpret_cast<const float4*>(a.CUM + ((size_t)u * 64 + i - 1) * H + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 up = make_float4(__expf(cum.x), __expf(cum.y), __expf(cum.z), __expf(cum.w));
    const float4 upx = make_float4(__expf(cumex.x), __expf(cumex.y), __expf(cumex.z), __expf(cumex.w));
    const float4 dn = make_float4(__expf(-cum.x), __expf(-cum.y), __expf(-cum.z), __expf(-cum.w));
    const float4 qs = make_float4(q.x * up.x, q.y * up.y, q.z * up.z, q.w * up.w), es = make_float4(e.x * upx.x, e.y * upx.y, e.z * upx.z, e.w * upx.w);
    const float4 ws = make_float4(w.x * dn.x, w.y * dn.y, w.z * dn.z, w.w * dn.w), as = make_float4(ah.x * dn.x, ah.y * dn.y, ah.z * dn.z, ah.w * dn.w);
    const size_t P128 = (size_t)a.nC * a.HB * 128 * H;
    const size_t o_top = ((size_t)u * 128 + i) * H + c4, o_bot = ((size_t)u * 128 + 64 + i) * H + c4;
    uint2 p0, p1, p2;
    limbs3x4(qs, p0, p1, p2);
    *reinterpret_cast<uint2*>(a.QE + o_top) = p0; *reinterpret_cast<uint2*>(a.QE + P128 + o_top) = p1; *reinterpret_cast<uint2*>(a.QE + 2 * P128 + o_top) = p2;
    *reinterpret_cast<uint2*>(a.A3 + o_bot) = p0; *reinterpret_cast<uint2*>(a.A3 + P128 + o_bot) = p1; *reinterpret_cast<uint2*>(a.A3 + 2 * P128 + o_bot) = p2;
    limbs3x4(es, p0, p1, p2);
    *reinterpret_cast<uint2*>(a.QE + o_bot) = p0; *reinterpret_cast<uint2*>(a.QE + P128 + o_bot) = p1; *reinterpret_cast<uint2*>(a.QE + 2 * P128 + o_bot) = p2;
    *reinterpret_cast<float4*>(a.ES + ((size_t)u * 64 + i) * H + c4) = es;
    limbs3x4(ws, p0, p1, p2);
    *reinterpret_cast<uint2*>(a.WA + o_top) = p0; *reinterpret_cast<uint2*>(a.WA + P128 + o_top) = p1; *reinterpret_cast<uint2*>(a.WA + 2 * P128 + o_top) = p2;
    limbs3x4(as, p0, p1, p2);
    *reinterpret_cast<uint2*>(a.WA + o_bot) = p0; *reinterpret_cast<uint2*>(a.WA + P128 + o_bot) = p1; *reinterpret_cast<uint2*>(a.WA + 2 * P128 + o_bot) = p2;
}

// (3) the keys decayed to the chunk's end, and the values, channel-major (rows of the 128 token slots): one block per
// (chunk, head, 64 channels), the 64 x 64 pieces turned round in shared memory.  grid (H / 64, nC * HB), 256 threads
__global__ void __launch_bounds__(256) chunk_keys_kernel(const ChunkArgs a) {
    pdl_enter();
    __shared__ float Ws[64][65], As[64][65];
    const int H = a.hs, u = blockIdx.y, j = u / a.HB, hb = u % a.HB, c0 = blockIdx.x * 64, tid = threadIdx.x;
    const int ch = tid >> 2, i0 = (tid & 3) * 16;   // when writing: thread = (channel, sixteen tokens)
    const size_t PT = (size_t)a.nC * a.HB * H * 128;
    const size_t rowT = ((size_t)u * H + c0 + ch) * 128 + i0;
    auto put = [&](const float (*S)[65], uint16_t* dst) {
#pragma unroll
        for (int h8 = 0; h8 < 16; h8 += 8) {
            uint16_t l[3][8];
#pragma unroll
            for (int q = 0; q < 8; ++q) limbs3(S[i0 + h8 + q][ch], l[0][q], l[1][q], l[2][q]);
#pragma unroll
            for (int p = 0; p < 3; ++p)
                *reinterpret_cast<uint4*>(dst + p * PT + h8) =
                    make_uint4(l[p][0] | ((uint32_t)l[p][1] << 16), l[p][2] | ((uint32_t)l[p][3] << 16), l[p][4] | ((uint32_t)l[p][5] << 16), l[p][6] | ((uint32_t)l[p][7] << 16));
        }
    };
    for (int n = tid; n < 64 * 16; n += 256) {
        const int i = n >> 4, c4 = (n & 15) * 4;
        const size_t at = (size_t)(j * CC + i) * a.tok_stride + (size_t)hb * H + c0 + c4;
        const float4 w = *reinterpret_cast<const float4*>(a.w + at), ah = *reinterpret_cast<const float4*>(a.ah + at);
        const float4 cum = *reinterpret_cast<const float4*>(a.CUM + ((size_t)u * 64 + i) * H + c0 + c4);
        const float4 cl = *reinterpret_cast<const float4*>(a.CUM + ((size_t)u * 64 + 63) * H + c0 + c4);
        const float k0 = __expf(cl.x - cum.x), k1 = __expf(cl.y - cum.y), k2 = __expf(cl.z - cum.z), k3 = __expf(cl.w - cum.w);
        Ws[i][c4] = w.x * k0; Ws[i][c4 + 1] = w.y * k1; Ws[i][c4 + 2] = w.z * k2; Ws[i][c4 + 3] = w.w * k3;
        As[i][c4] = ah.x * k0; As[i][c4 + 1] = ah.y * k1; As[i][c4 + 2] = ah.z * k2; As[i][c4 + 3] = ah.w * k3;
    }
    __syncthreads();
    put(Ws, a.B5 + rowT);
    put(As, a.B5 + rowT + 64);
    __syncthreads();
    for (int n = tid; n < 64 * 16; n += 256) {   // the values, through the first square again
        const int i = n >> 4, c4 = (n & 15) * 4;
        const float4 v = *reinterpret_cast<const float4*>(a.v + (size_t)(j * CC + i) * a.tok_stride + (size_t)hb * H + c0 + c4);
        Ws[i][c4] = v.x; Ws[i][c4 + 1] = v.y; Ws[i][c4 + 2] = v.z; Ws[i][c4 + 3] = v.w;
    }
    __syncthreads();
    put(Ws, a.A5 + rowT);
}

// ---- the four 64x64 matrices of a chunk and the inverse: one block of 256 threads per (chunk, head) --------------
__global__ void __launch_bounds__(256) chunk_solve_kernel(const ChunkArgs a) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    float* Ae = sm;               // [64][65]
    float* Ke = Ae + 64 * 65;     // [64][65]
    float* X = Ke + 64 * 65;      // [64][65] the inverse
    const int u = blockIdx.x, tid = threadIdx.x;
    const float* G = a.Gm + (size_t)u * 128 * 128;
    float* Qa = a.Qa + (size_t)u * 4096;
    const size_t PX = (size_t)a.nC * a.HB * 128 * 64;      // plane of XL
    uint16_t* XL = a.XL + (size_t)u * 128 * 64;            // rows 0..63: T Ke, rows 64..127: Qw
    for (int n = tid; n < 4096; n += 256) {
        const int i = n >> 6, jj = n & 63;
        {
            uint16_t l0, l1, l2;
            limbs3(jj <= i ? G[(size_t)i * 128 + jj] : 0.0f, l0, l1, l2);
            XL[4096 + n] = l0; XL[PX + 4096 + n] = l1; XL[2 * PX + 4096 + n] = l2;
        }
        Qa[n] = jj <= i ? G[(size_t)i * 128 + 64 + jj] : 0.0f;
        Ke[i * 65 + jj] = jj < i ? G[(size_t)(64 + i) * 128 + jj] : 0.0f;
        Ae[i * 65 + jj] = jj < i ? G[(size_t)(64 + i) * 128 + 64 + jj] : 0.0f;
    }
    __syncthreads();
    // X = (I + Ae)^-1 by forward substitution, one thread per column: x_i = [i == c] - sum_{k < i} Ae[i][k] x_k
    if (tid < 64) {
        const int c = tid;
        for (int i = 0; i < 64; ++i) {
            float s = i == c ? 1.0f : 0.0f;
            for (int k = c; k < i; ++k) s = fmaf(-Ae[i * 65 + k], X[k * 65 + c], s);  // x_k = 0 for k < c
            X[i * 65 + c] = i < c ? 0.0f : s;
        }
    }
    __syncthreads();
    float* Ti = a.Tinv + (size_t)u * 4096;
    for (int n = tid; n < 4096; n += 256) {
        const int i = n >> 6, c = n & 63;
        Ti[n] = X[i * 65 + c];
        float s = 0.0f;
        for (int k = 0; k <= i; ++k) s = fmaf(X[i * 65 + k], Ke[k * 65 + c], s);  // X is lower triangular
        uint16_t l0, l1, l2;
        limbs3(s, l0, l1, l2);
        XL[n] = l0; XL[PX + n] = l1; XL[2 * PX + n] = l2;
    }
}

// ---- p1 [64 x hs] = T [64 x 64] . es [64 x hs] per (chunk, head), written as limbs into the state read's left operand -----
// grid (H / 128, nC * HB); 128 threads: thread (r8, c8) owns rows r8 * 8 .. + 7 and columns c8 * 8 .. + 7 of the tile
// (an 8 x 8 register tile: four 16-byte reads of shared memory per 64 multiply-adds)
__device__ __forceinline__ void tile_mm_8x8(const float (*Mt)[64], const float (*Xs)[128], int r8, int c8, float (&acc)[8][8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[i][q] = 0.0f;
#pragma unroll 4
    for (int k = 0; k < 64; ++k) {
        const float4 x0 = *reinterpret_cast<const float4*>(&Xs[k][c8 * 8]), x1 = *reinterpret_cast<const float4*>(&Xs[k][c8 * 8 + 4]);
        const float4 m0 = *reinterpret_cast<const float4*>(&Mt[k][r8 * 8]), m1 = *reinterpret_cast<const float4*>(&Mt[k][r8 * 8 + 4]);
        const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        const float mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[i][q] = fmaf(mv[i], xv[q], acc[i][q]);
    }
}

__global__ void __launch_bounds__(128) chunk_small_kernel(const ChunkArgs a) {
    pdl_enter();
    __shared__ __align__(16) float Mt[64][64];  // transposed: [k][row]
    __shared__ __align__(16) float Xs[64][128];
    const int H = a.hs, u = blockIdx.y, c0 = blockIdx.x * 128, tid = threadIdx.x;
    const float* Mx = a.Tinv + (size_t)u * 4096;
    for (int n = tid; n < 4096; n += 128) Mt[n & 63][n >> 6] = Mx[n];
    for (int n = tid; n < 64 * 32; n += 128) {
        const int i = n >> 5, q = (n & 31) * 4;
        *reinterpret_cast<float4*>(&Xs[i][q]) = *reinterpret_cast<const float4*>(a.ES + ((size_t)u * 64 + i) * H + c0 + q);
    }
    __syncthreads();
    const int r8 = tid >> 4, c8 = tid & 15;
    float acc[8][8];
    tile_mm_8x8(Mt, Xs, r8, c8, acc);
    const size_t P128 = (size_t)a.nC * a.HB * 128 * H;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = r8 * 8 + i;
        const size_t o = ((size_t)u * 128 + row) * H + c0 + c8 * 8;
        uint16_t l[3][8];
#pragma unroll
        for (int q = 0; q < 8; ++q) limbs3(acc[i][q], l[0][q], l[1][q], l[2][q]);
#pragma unroll
        for (int p = 0; p < 3; ++p)
            *reinterpret_cast<uint4*>(a.A3 + p * P128 + o) =
                make_uint4(l[p][0] | ((uint32_t)l[p][1] << 16), l[p][2] | ((uint32_t)l[p][3] << 16), l[p][4] | ((uint32_t)l[p][5] << 16), l[p][6] | ((uint32_t)l[p][7] << 16));
    }
}

// ---- one chunk's reads: y = yw - Qa rr (rr and yw come from the state read); -rr^T into the update's left operand ----
// grid (H / 128, HB); 128 threads, the same 8 x 8 register tile
__global__ void __launch_bounds__(128) chunk_read_kernel(const ChunkArgs a, int j) {
    pdl_enter();
    __shared__ __align__(16) float Mt[64][64];  // Qa transposed: [k][row]
    __shared__ __align__(16) float Rs[64][128];
    const int H = a.hs, hb = blockIdx.y, u = j * a.HB + hb, c0 = blockIdx.x * 128, tid = threadIdx.x;
    const float* Qa = a.Qa + (size_t)u * 4096;
    for (int n = tid; n < 4096; n += 128) Mt[n & 63][n >> 6] = Qa[n];
    const float* RY = a.RY + (size_t)hb * 128 * H;
    for (int n = tid; n < 64 * 32; n += 128) {
        const int i = n >> 5, q = (n & 31) * 4;
        *reinterpret_cast<float4*>(&Rs[i][q]) = *reinterpret_cast<const float4*>(RY + (size_t)i * H + c0 + q);
    }
    __syncthreads();
    const int r8 = tid >> 4, c8 = tid & 15;
    float acc[8][8];
    tile_mm_8x8(Mt, Rs, r8, c8, acc);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = r8 * 8 + i;
        const float* yq = RY + (size_t)(64 + row) * H + c0 + c8 * 8;
        float* dst = a.y + (size_t)(j * CC + row) * a.tok_stride + (size_t)hb * H + c0 + c8 * 8;
        const float4 y0 = *reinterpret_cast<const float4*>(yq), y1 = *reinterpret_cast<const float4*>(yq + 4);
        *reinterpret_cast<float4*>(dst) = make_float4(y0.x - acc[i][0], y0.y - acc[i][1], y0.z - acc[i][2], y0.w - acc[i][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(y1.x - acc[i][4], y1.y - acc[i][5], y1.z - acc[i][6], y1.w - acc[i][7]);
    }
    // -rr transposed: row (value) of the update's left operand, token slots 64 .. 127; thread = value
    const size_t PT = (size_t)a.nC * a.HB * H * 128;
    const size_t rowT = ((size_t)u * H + c0 + tid) * 128 + 64;
#pragma unroll 2
    for (int i8 = 0; i8 < 64; i8 += 8) {
        uint16_t l[3][8];
#pragma unroll
        for (int q = 0; q < 8; ++q) limbs3(-Rs[i8 + q][tid], l[0][q], l[1][q], l[2][q]);
#pragma unroll
        for (int p = 0; p < 3; ++p)
            *reinterpret_cast<uint4*>(a.A5 + p * PT + rowT + i8) =
                make_uint4(l[p][0] | ((uint32_t)l[p][1] << 16), l[p][2] | ((uint32_t)l[p][3] << 16), l[p][4] | ((uint32_t)l[p][5] << 16), l[p][6] | ((uint32_t)l[p][7] << 16));
    }
}

// ---- the state between its layouts: slice-major F [hb][hs / cw][key][cw] <-> transposed Ft [hb][value][key] (+ limbs) -----
// grid (H / 32, H / 32, HB), 32 x 8 threads: a 32 x 32 tile through shared memory
__global__ void chunk_state_kernel(const ChunkArgs a, int to_ft) {
    pdl_enter();
    __shared__ float tile[32][33];
    const int H = a.hs, cw = a.cw, hb = blockIdx.z, k0 = blockIdx.x * 32, v0 = blockIdx.y * 32;
    float* F = a.F + (size_t)hb * H * H;
    float* Ft = a.Ft + (size_t)hb * H * H;
    const size_t PF = (size_t)a.HB * H * H;
    auto fidx = [&](int key, int val) { return (size_t)(val / cw) * H * cw + (size_t)key * cw + (val % cw); };
    if (to_ft) {
        for (int r = threadIdx.y; r < 32; r += 8) tile[r][threadIdx.x] = F[fidx(k0 + r, v0 + threadIdx.x)];  // [key][value]
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += 8) {
            const float x = tile[threadIdx.x][r];  // key = k0 + x-thread, value = v0 + r
            const size_t o = (size_t)(v0 + r) * H + k0 + threadIdx.x;
            Ft[o] = x;
            uint16_t l0, l1, l2;
            limbs3(x, l0, l1, l2);
            const size_t ol = (size_t)hb * H * H + o;
            a.Ft_limbs[ol] = l0; a.Ft_limbs[PF + ol] = l1; a.Ft_limbs[2 * PF + ol] = l2;
        }
    } else {
        for (int r = threadIdx.y; r < 32; r += 8) tile[r][threadIdx.x] = Ft[(size_t)(v0 + r) * H + k0 + threadIdx.x];  // [value][key]
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += 8) F[fidx(k0 + r, v0 + threadIdx.x)] = tile[threadIdx.x][r];
    }
}

}  // namespace

size_t mem_chunk_workspace_bytes(int HB, int hs, int nC) {
    const size_t H = hs, U = (size_t)nC * HB;
    size_t b = 0;
    b += 3 * (3 * U * 128 * H * 2);   // QE, WA, A3 limbs
    b += 2 * (3 * U * H * 128 * 2);   // A5, B5 limbs
    b += 2 * (U * 64 * H * 4);        // ES, CUM
    b += 3 * U * 128 * 64 * 2;        // XL
    b += U * H * 4;                   // gc
    b += U * 128 * 128 * 4;           // Gm
    b += 2 * (U * 4096 * 4);          // Qa, Tinv
    b += (size_t)HB * 128 * H * 4;    // RY
    b += (size_t)HB * H * H * 4;      // Ft
    b += 3 * (size_t)HB * H * H * 2;  // Ft limbs
    return b + 4096;
}

void mem_chunk_carve(ChunkArgs& a, void* ws) {
    const size_t H = a.hs, U = (size_t)a.nC * a.HB;
    unsigned char* p = static_cast<unsigned char*>(ws);
    auto take = [&](size_t bytes) { void* q = p; p += (bytes + 255) & ~(size_t)255; return q; };
    a.QE = (uint16_t*)take(3 * U * 128 * H * 2);
    a.WA = (uint16_t*)take(3 * U * 128 * H * 2);
    a.A3 = (uint16_t*)take(3 * U * 128 * H * 2);
    a.A5 = (uint16_t*)take(3 * U * H * 128 * 2);
    a.B5 = (uint16_t*)take(3 * U * H * 128 * 2);
    a.ES = (float*)take(U * 64 * H * 4);
    a.CUM = (float*)take(U * 64 * H * 4);
    a.gc = (float*)take(U * H * 4);
    a.Gm = (float*)take(U * 128 * 128 * 4);
    a.Qa = (float*)take(U * 4096 * 4);
    a.Tinv = (float*)take(U * 4096 * 4);
    a.XL = (uint16_t*)take(3 * U * 128 * 64 * 2);
    a.RY = (float*)take((size_t)a.HB * 128 * H * 4);
    a.Ft = (float*)take((size_t)a.HB * H * H * 4);
    a.Ft_limbs = (uint16_t*)take(3 * (size_t)a.HB * H * H * 2);
}

bool mem_chunk_covers(int hs, int T, float momentum) { return hs % 128 == 0 && T % CC == 0 && T > 0 && !(momentum > 0.0f); }

// Stage 1: scaling (sets *a.flags when a chunk's rates are too strong for this form).  The caller checks the flag
// before stage 2.
bool launch_mem_chunk_scale(cudaStream_t st, const ChunkArgs& a) {
    if (!mem_chunk_covers(a.hs, a.nC * CC, 0.0f)) return false;
    launch_k(chunk_scan_kernel, dim3((a.hs + 255) / 256, a.nC * a.HB), dim3(256), 0, st, a);
    const size_t n = (size_t)a.nC * a.HB * 64 * (a.hs / 4);
    launch_k(chunk_scale_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, a);
    launch_k(chunk_keys_kernel, dim3(a.hs / 64, a.nC * a.HB), dim3(256), 0, st, a);
    return true;
}

// Stage 2: everything else; the state F (slice-major) is read at the start and written back at the end.
bool launch_mem_chunk_rest(cudaStream_t st, const ChunkArgs& a) {
    const int H = a.hs, U = a.nC * a.HB;
    launch_k(chunk_state_kernel, dim3(H / 32, H / 32, a.HB), dim3(32, 8), 0, st, a, 1);
    TcbArgs g{};
    g.a = a.QE; g.b = a.WA; g.rows_a = g.rows_b = (int64_t)U * 128; g.C = a.Gm; g.ldc = 128; g.c_batch_stride = 128 * 128;
    g.M = 128; g.N = 128; g.K = H; g.batch = U; g.status = a.status;
    if (!launch_tc_bgemm(st, g, TCB_STORE)) return false;
    const size_t solve_smem = 3 * 64 * 65 * sizeof(float);
    cudaFuncSetAttribute(chunk_solve_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)solve_smem);
    launch_k(chunk_solve_kernel, dim3(U), dim3(256), solve_smem, st, a);
    launch_k(chunk_small_kernel, dim3(H / 128, U), dim3(128), 0, st, a);
    for (int j = 0; j < a.nC; ++j) {
        TcbArgs s3{};
        s3.a = a.A3; s3.a_row0 = (int64_t)j * a.HB * 128; s3.rows_a = (int64_t)U * 128;
        s3.b = a.Ft_limbs; s3.rows_b = (int64_t)a.HB * H;
        s3.a2 = a.XL; s3.rows_a2 = (int64_t)U * 128; s3.a2_row0 = (int64_t)j * a.HB * 128; s3.lda2 = 64;      // [T Ke; Qw] ...
        s3.b2 = a.A5; s3.rows_b2 = (int64_t)U * H; s3.b2_row0 = (int64_t)j * a.HB * H; s3.ldb2 = 128; s3.K2 = 64;  // ... times the chunk's values
        s3.C = a.RY; s3.ldc = H; s3.c_batch_stride = (int64_t)128 * H; s3.M = 128; s3.N = H; s3.K = H; s3.batch = a.HB; s3.status = a.status;
        if (!launch_tc_bgemm(st, s3, TCB_STORE)) return false;
        launch_k(chunk_read_kernel, dim3(H / 128, a.HB), dim3(128), 0, st, a, j);
        TcbArgs s5{};
        s5.a = a.A5; s5.a_row0 = (int64_t)j * a.HB * H; s5.rows_a = (int64_t)U * H;
        s5.b = a.B5; s5.b_row0 = (int64_t)j * a.HB * H; s5.rows_b = (int64_t)U * H;
        s5.C = a.Ft; s5.ldc = H; s5.c_batch_stride = (int64_t)H * H; s5.M = H; s5.N = H; s5.K = 128; s5.batch = a.HB;
        s5.colscale = a.gc + (size_t)j * a.HB * H; s5.colscale_batch_stride = H;
        s5.c_limbs = a.Ft_limbs; s5.c_limb_plane = (int64_t)a.HB * H * H; s5.status = a.status;
        if (!launch_tc_bgemm(st, s5, TCB_DECAY)) return false;
    }
    launch_k(chunk_state_kernel, dim3(H / 32, H / 32, a.HB), dim3(32, 8), 0, st, a, 0);
    return true;
}

int mem_chunk_launches(int nC) { return 5 + 3 * nC + 3; }

}  // namespace ava

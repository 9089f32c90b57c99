// The per-row kernels of the block step (sm_100a): embedding gather, RMS norm, the memory's gate preparation and
// head norm + output gate, k-winners-take-all, the dense residual mix, greedy argmax.
//
// Sums that the reference takes "one value after another from 0" (design-tests/nn/gpu/src/model/fstep.rs:12-14) are
// taken in that order by one thread, and the small f32 products follow gemm's one-row order (fstep.rs:17-23,222-257):
// out = w0 * x0, then fma(w_j, x_j, out).  The chains are short next to the memory traffic of the step, and keeping
// them makes every value the bits of the reference's arithmetic.
#include <algorithm>

#include "ava_math.h"
#include "bf16_hw.cuh"
#include "kernels.cuh"
#include "row_sums.cuh"

namespace ava {

namespace {

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
// letters: --letters' table [vocab][d] or nullptr; a token's row of it is added to its embedding
__global__ void embed_kernel(const float* __restrict__ tok_emb, const uint32_t* __restrict__ tok, int M, int d, int vocab, float* x, float* stream0,
                             uint32_t* status, const float* __restrict__ letters) {
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
    const float4* let = letters ? reinterpret_cast<const float4*>(letters + (size_t)t * d) : nullptr;
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
        float4 v = src[i];
        if (let) {
            const float4 o = let[i];
            v = make_float4(add(v.x, o.x), add(v.y, o.y), add(v.z, o.z), add(v.w, o.w));
        }
        dst[i] = v;
        if (dst2) dst2[i] = v;
    }
}

// ---------------------------------------------------------------------------------------------------- RMS norm
// three bf16 limbs of v (their sum is v exactly) into planes [3][plane], for the tensor-core products
__device__ __forceinline__ void store_limbs(uint16_t* limbs, int64_t plane, int64_t i, float v) {
    uint16_t hi, mid, lo;
    limbs3_hw(v, hi, mid, lo);
    limbs[i] = hi;
    limbs[plane + i] = mid;
    limbs[2 * plane + i] = lo;
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
    if (limbs) {
        // the tolerance mode (its consumer is a tensor-core product): the squares summed by the whole warp, another order
        float sq = 0.0f;
        for (int i = lane; i < n; i += 32) sq = fmaf(xs[i], xs[i], sq);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        inv = rsqrtf_(sq * (float)(1.0 / (double)n) + NORM_EPS);
    } else {
        if (lane == 0) inv = inv_rms_seq(xs, n);
        inv = __shfl_sync(0xffffffffu, inv, 0);
    }
    float* yr = y + (size_t)r * n;
    for (int i = lane; i < n; i += 32) {
        const float v = mul(mul(xs[i], inv), gain[i]);
        yr[i] = v;
        if (limbs) store_limbs(limbs, (int64_t)M * n, (int64_t)r * n + i, v);
    }
}

// ---------------------------------------------------------------------------------------------------- memory: gates
// src/model/fstep/arch.rs:685-803 for one row per block of threads.
// Stage one of the gates: z [M][ncp] = h . [wa1 | wb1 | wa | wb] in gemm's one-row order (row 0's product, then fma
// down the rows: an fma chain from -0).  One thread per (row, column), a few rows per block so that the block's copy of
// the weights serves them all.  The weights come through a ring of S chunks of CR rows in shared memory (cp.async, every
// thread copies); all S are requested before the first is used, so the chain meets the memory latency once.
__global__ void gate_z_kernel(const float* __restrict__ hin, const float* __restrict__ gate_w, int M, int d, int ncp, int CR, int RB, int S,
                              float* __restrict__ z) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    float* h = sm;                       // [RB][d]
    float* stage = sm + (size_t)RB * d;  // [S][CR * ncp]
    const int tid = threadIdx.x, T = blockDim.x;
    const int row0 = blockIdx.x * RB, rows = min(RB, M - row0);
    const int nchunk = d / CR, per_chunk4 = CR * ncp / 4;
    auto fetch = [&](int c) {  // one commit group per chunk, empty past the end so that the group count stays in step
        if (c < nchunk) {
            float* dst = stage + (size_t)(c % S) * CR * ncp;
            const float* src = gate_w + (size_t)c * CR * ncp;
            for (int i = tid; i < per_chunk4; i += T)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst + 4 * i)), "l"(src + 4 * i) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int c = 0; c < S; ++c) fetch(c);
    for (int i = tid; i < rows * d / 4; i += T)
        reinterpret_cast<float4*>(h)[i] = reinterpret_cast<const float4*>(hin + (size_t)row0 * d)[i];
    const int rb = tid / ncp, col = tid - rb * ncp;
    const bool live = rb < rows;
    float out = -0.0f;  // fma(w, x, -0) is the plain rounded product: the chain's first term
    for (int c = 0; c < nchunk; ++c) {
        // groups are committed in chunk order; at most S - 1 newer ones may still be in flight
        switch (S - 1) {
            case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
            case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
            case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
            case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
            case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
            case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
            case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
            default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
        }
        __syncthreads();
        if (live) {
            const float* wcol = stage + (size_t)(c % S) * CR * ncp + col;
            const float* hx = h + (size_t)rb * d + c * CR;
            float w8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w8[i] = lds1(wcol + (size_t)i * ncp);
            float4 x0 = lds4(hx), x1 = lds4(hx + 4);
            for (int r0 = 0; r0 < CR; r0 += 8) {
                // the next eight rows' weights and inputs are on their way while this eight joins the chain
                float nx[8];
                const int nr = r0 + 8 < CR ? r0 + 8 : r0;
#pragma unroll
                for (int i = 0; i < 8; ++i) nx[i] = lds1(wcol + (size_t)(nr + i) * ncp);
                const float4 y0 = lds4(hx + nr), y1 = lds4(hx + nr + 4);
                const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) out = fma(w8[i], xv[i], out);
#pragma unroll
                for (int i = 0; i < 8; ++i) w8[i] = nx[i];
                x0 = y0;
                x1 = y1;
            }
        }
        __syncthreads();
        fetch(c + S);  // the slot just read takes the chunk S further on
    }
    if (live) z[(size_t)(row0 + rb) * ncp + col] = out;
}

// Stage one for a few rows: with one sequence the kernel above is ONE block that pulls the whole [d][ncp] weight matrix
// through its ring.  Here a block owns four columns: all its threads request the [d][4] strip at once (16 bytes per row),
// and one thread per (row, column) walks the same chain from shared memory, sixteen terms fetched ahead.
constexpr int GZF_ROWS = 8, GZF_THREADS = 128;
__global__ void __launch_bounds__(GZF_THREADS) gate_z_few_kernel(const float* __restrict__ hin, const float* __restrict__ gate_w, int M, int d, int ncp,
                                                                 float* __restrict__ z, const float* __restrict__ norm_gain) {
    extern __shared__ __align__(16) float sm[];
    float* ws = sm;                      // [d][4]
    float* h = sm + (size_t)d * 4;       // [rows][d]
    float* gn = h + (size_t)GZF_ROWS * d;  // [d] the norm's gain, then [GZF_ROWS] the rows' norms (norm_gain only)
    const int tid = threadIdx.x, c0 = blockIdx.x * 4, row0 = blockIdx.y * GZF_ROWS, rows = min(GZF_ROWS, M - row0);
    for (int k = tid; k < d; k += GZF_THREADS)   // the weights depend on nothing before: requested ahead of the wait
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(ws + 4 * k)), "l"(gate_w + (size_t)k * ncp + c0) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
    pdl_enter();
    for (int i = tid; i < rows * d / 4; i += GZF_THREADS)
        reinterpret_cast<float4*>(h)[i] = reinterpret_cast<const float4*>(hin + (size_t)row0 * d)[i];
    if (norm_gain) {
        // the rows came as the block's input: their RMS norm is taken here (rmsnorm_kernel's arithmetic), a row's
        // ordered sum by lane 0 of a warp, the scaling by everyone, while the weights arrive
        for (int i = tid; i < d / 4; i += GZF_THREADS) reinterpret_cast<float4*>(gn)[i] = reinterpret_cast<const float4*>(norm_gain)[i];
        __syncthreads();
        float* inv_sh = gn + d;
        for (int r = tid >> 5; r < rows; r += GZF_THREADS / 32)
            if ((tid & 31) == 0) inv_sh[r] = inv_rms_seq(h + (size_t)r * d, d);
        __syncthreads();
        for (int i = tid; i < rows * d; i += GZF_THREADS) {
            const int r = i / d;
            h[i] = mul(mul(h[i], inv_sh[r]), gn[i - r * d]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const int rb = tid >> 2, col = tid & 3;
    if (rb >= rows) return;
    const float* hx = h + (size_t)rb * d;
    const float* wc = ws + col;
    float out = -0.0f;  // fma(w, x, -0) is the plain rounded product: the chain's first term
    float wa[16], wb[16];
    float4 xa[4], xb[4];
    auto load_a = [&](int g) {
#pragma unroll
        for (int u = 0; u < 16; ++u) wa[u] = lds1(wc + (size_t)(16 * g + u) * 4);
#pragma unroll
        for (int u = 0; u < 4; ++u) xa[u] = lds4(hx + 16 * g + 4 * u);
    };
    auto load_b = [&](int g) {
#pragma unroll
        for (int u = 0; u < 16; ++u) wb[u] = lds1(wc + (size_t)(16 * g + u) * 4);
#pragma unroll
        for (int u = 0; u < 4; ++u) xb[u] = lds4(hx + 16 * g + 4 * u);
    };
    const int G = d / 16;
    int g = 0;
    if (G > 0) load_a(0);
    while (g + 2 <= G) {
        load_b(g + 1);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            out = fma(wa[4 * u], xa[u].x, out);
            out = fma(wa[4 * u + 1], xa[u].y, out);
            out = fma(wa[4 * u + 2], xa[u].z, out);
            out = fma(wa[4 * u + 3], xa[u].w, out);
        }
        if (g + 2 < G) load_a(g + 2);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            out = fma(wb[4 * u], xb[u].x, out);
            out = fma(wb[4 * u + 1], xb[u].y, out);
            out = fma(wb[4 * u + 2], xb[u].z, out);
            out = fma(wb[4 * u + 3], xb[u].w, out);
        }
        g += 2;
    }
    if (g < G) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            out = fma(wa[4 * u], xa[u].x, out);
            out = fma(wa[4 * u + 1], xa[u].y, out);
            out = fma(wa[4 * u + 2], xa[u].z, out);
            out = fma(wa[4 * u + 3], xa[u].w, out);
        }
    }
    for (int k = 16 * G; k < d; ++k) out = fma(lds1(wc + (size_t)k * 4), lds1(hx + k), out);
    z[(size_t)(row0 + rb) * ncp + c0 + col] = out;
}

// gemm's one-row product of k terms, the terms given by functions of j (src/model/fstep.rs:222-257)
template <typename W, typename X>
__device__ __forceinline__ float chain_k(int k, W w, X x) {
    if (k == 0) return 0.0f;
    if (k == 1) return mul(w(0), x(0));
    if (k == 2) return add(mul(w(1), x(1)), mul(w(0), x(0)));
    float out = mul(w(0), x(0));
    for (int j = 1; j < k; ++j) out = fma(w(j), x(j), out);
    return out;
}

// Stage two: lra [M][d] = z1a . wa2, lrb = z1b . wb2 (rank-long chains).  A block owns 16 columns of both matrices:
// each thread keeps its column's weights in registers (RK > 0: the rank, known at compile time) and walks the rows,
// sixteen threads side by side on different rows; the z1 values of the block's tile of rows sit in shared memory.
constexpr int LR_COLS = 16, LR_LANES = 16, LR_ROWS = 256;
template <int RK>
__global__ void __launch_bounds__(LR_COLS* LR_LANES) lowrank_kernel(const float* __restrict__ z, int ncp, int za_col, int zb_col, int rk_rt,
                                                                     const float* __restrict__ wa2, const float* __restrict__ wb2, int M_all, int d,
                                                                     float* __restrict__ lra, float* __restrict__ lrb) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int rk = RK ? RK : rk_rt;
    // this block's tile of rows
    const int row0 = blockIdx.y * LR_ROWS, M = min(LR_ROWS, M_all - row0);
    z += (size_t)row0 * ncp;
    lra += (size_t)row0 * d;
    lrb += (size_t)row0 * d;
    float* zs = sm;  // [M][2 rk]: z1a | z1b of every row of the tile
    const int tid = threadIdx.x, col = tid % LR_COLS, lane_r = tid / LR_COLS;
    const int c = blockIdx.x * LR_COLS + col;
    if ((2 * rk) % 4 == 0 && za_col == 0 && zb_col == rk) {
        // z1a | z1b are the first 2 rk values of each row of z (rows are 16-byte aligned): every copy in flight at once
        const int per_row4 = 2 * rk / 4;
        for (int i = tid; i < M * per_row4; i += blockDim.x) {
            const int r = i / per_row4, j4 = i - r * per_row4;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(zs + 4 * i)), "l"(z + (size_t)r * ncp + 4 * j4)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        for (int i = tid; i < M * 2 * rk; i += blockDim.x) {
            const int r = i / (2 * rk), j = i - r * 2 * rk;
            zs[i] = z[(size_t)r * ncp + (j < rk ? za_col + j : zb_col + j - rk)];
        }
    }
    __syncthreads();
    if (c >= d) return;
    if (RK >= 4 && RK % 4 == 0) {
        float wa[RK ? RK : 1], wb[RK ? RK : 1];
#pragma unroll
        for (int j = 0; j < RK; ++j) {
            wa[j] = __ldg(wa2 + (size_t)j * d + c);
            wb[j] = __ldg(wb2 + (size_t)j * d + c);
        }
        for (int r = lane_r; r < M; r += 2 * LR_LANES) {
            // two rows and both gates at once: four independent chains
            const int r2 = r + LR_LANES;
            const float* z0 = zs + (size_t)r * 2 * RK;
            const float* z1 = zs + (size_t)(r2 < M ? r2 : r) * 2 * RK;
            float a0 = -0.0f, b0 = -0.0f, a1 = -0.0f, b1 = -0.0f;  // fma from -0: the chain's first term is the plain product
#pragma unroll
            for (int j = 0; j < RK; j += 4) {
                const float4 za0 = lds4(z0 + j), zb0 = lds4(z0 + RK + j), za1 = lds4(z1 + j), zb1 = lds4(z1 + RK + j);
                const float xa0[4] = {za0.x, za0.y, za0.z, za0.w}, xb0[4] = {zb0.x, zb0.y, zb0.z, zb0.w};
                const float xa1[4] = {za1.x, za1.y, za1.z, za1.w}, xb1[4] = {zb1.x, zb1.y, zb1.z, zb1.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    a0 = fma(wa[j + u], xa0[u], a0);
                    b0 = fma(wb[j + u], xb0[u], b0);
                    a1 = fma(wa[j + u], xa1[u], a1);
                    b1 = fma(wb[j + u], xb1[u], b1);
                }
            }
            lra[(size_t)r * d + c] = a0;
            lrb[(size_t)r * d + c] = b0;
            if (r2 < M) {
                lra[(size_t)r2 * d + c] = a1;
                lrb[(size_t)r2 * d + c] = b1;
            }
        }
    } else {
        for (int r = lane_r; r < M; r += LR_LANES) {
            const float* zr = zs + (size_t)r * 2 * rk;
            lra[(size_t)r * d + c] = chain_k(rk, [&](int j) { return __ldg(wa2 + (size_t)j * d + c); }, [&](int j) { return zr[j]; });
            lrb[(size_t)r * d + c] = chain_k(rk, [&](int j) { return __ldg(wb2 + (size_t)j * d + c); }, [&](int j) { return zr[rk + j]; });
        }
    }
}

// --dendrite: act [M][H] *= 1 + tanh(z1 . B) (src/model/fstep/arch_f4.rs:120-141).  Laid out like the stage above: a block
// owns 16 units (columns of B, in registers per thread when the rank is known), the z1 values of its tile of rows sit
// in shared memory, sixteen threads side by side on different rows.
template <int RK>
__global__ void __launch_bounds__(LR_COLS* LR_LANES) dend_gain_kernel(const float* __restrict__ z1, int rk_rt, const float* __restrict__ B, int M_all, int H,
                                                                       float* act) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int rk = RK ? RK : rk_rt;
    const int row0 = blockIdx.y * LR_ROWS, M = min(LR_ROWS, M_all - row0);
    const int tid = threadIdx.x, col = tid % LR_COLS, lane_r = tid / LR_COLS;
    const int c = blockIdx.x * LR_COLS + col;
    for (int i = tid; i < M * rk; i += blockDim.x) sm[i] = z1[(size_t)row0 * rk + i];
    __syncthreads();
    if (c >= H) return;
    float w[RK ? RK : 1];
    if (RK) {
#pragma unroll
        for (int j = 0; j < RK; ++j) w[j] = __ldg(B + (size_t)j * H + c);
    }
    for (int r = lane_r; r < M; r += LR_LANES) {
        const float* zr = sm + (size_t)r * rk;
        float z;
        if (RK >= 3) {
            z = mul(w[0], zr[0]);
#pragma unroll
            for (int j = 1; j < RK; ++j) z = fma(w[j], zr[j], z);
        } else {
            z = chain_k(rk, [&](int j) { return __ldg(B + (size_t)j * H + c); }, [&](int j) { return zr[j]; });
        }
        float* ap = act + (size_t)(row0 + r) * H + c;
        *ap = mul(*ap, add(mul(tanhf_(z), 1.0f), 1.0f));
    }
}

// --neuromod: the nucleus's signals 2 sigmoid(z + b) (src/model/fstep/arch.rs:1108-1119); z and sig are [M][4], k <= 4 used
__global__ void nucleus_kernel(const float* __restrict__ z, const float* __restrict__ bias, int k, int M, float* __restrict__ sig) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * 4) return;
    const int j = i & 3;
    sig[i] = j < k ? add(mul(sigmoid(add(z[i], bias[j])), 2.0f), 0.0f) : 1.0f;
}

// x += y, or with a row gain x += y * gain[row * NM_STRIDE] (rows of d, d % 4 == 0)
__global__ void add_into_kernel(float* x, const float* __restrict__ y, int64_t n, const float* __restrict__ gain, int d) {
    pdl_enter();
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 4 <= n) {
        const float4 a = *reinterpret_cast<const float4*>(x + i);
        float4 b = *reinterpret_cast<const float4*>(y + i);
        if (gain) {
            const float g = gain[(i / d) * NM_STRIDE];
            b = make_float4(mul(b.x, g), mul(b.y, g), mul(b.z, g), mul(b.w, g));
        }
        *reinterpret_cast<float4*>(x + i) = make_float4(add(a.x, b.x), add(a.y, b.y), add(a.z, b.z), add(a.w, b.w));
    } else {
        for (int64_t k = i; k < n; ++k) x[k] = add(x[k], gain ? mul(y[k], gain[(k / d) * NM_STRIDE]) : y[k]);
    }
}

// --thalamus, one thread per token-row (src/model/fstep/arch_f2.rs:93-118, src/v51b.rs:312-321): the relay's sum takes
// this read (thr [M][16]; the first read starts the sum), then the next block's gates are
// 2 sigmoid(tanh(acc * (1 / sqrt(reads)) + 0) G + c) with the 16-term product as an ordered chain from G[0] f[0].
// g is [M][NM_STRIDE]: [0] the residual's gate, [1] the memory read's.
__global__ void relay_kernel(const float* __restrict__ thr, float* __restrict__ acc, int first, float mulf, const float* __restrict__ G,
                             const float* __restrict__ bias, int M, float* __restrict__ g) {
    pdl_enter();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= M) return;
    float z0 = -0.0f, z1 = -0.0f;
#pragma unroll
    for (int k4 = 0; k4 < 16; k4 += 4) {
        const float4 t = *reinterpret_cast<const float4*>(thr + (size_t)r * 16 + k4);
        float4 a = t;
        if (!first) {
            const float4 o = *reinterpret_cast<const float4*>(acc + (size_t)r * 16 + k4);
            a = make_float4(add(o.x, t.x), add(o.y, t.y), add(o.z, t.z), add(o.w, t.w));
        }
        *reinterpret_cast<float4*>(acc + (size_t)r * 16 + k4) = a;
        const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float f = tanhf_(add(mul(av[u], mulf), 0.0f));
            const int k = k4 + u;
            if (k == 0) {
                z0 = mul(G[0], f);
                z1 = mul(G[1], f);
            } else {
                z0 = fma(G[k * 2], f, z0);
                z1 = fma(G[k * 2 + 1], f, z1);
            }
        }
    }
    g[(size_t)r * NM_STRIDE] = add(mul(sigmoid(add(z0, bias[0])), 2.0f), 0.0f);
    g[(size_t)r * NM_STRIDE + 1] = add(mul(sigmoid(add(z1, bias[1])), 2.0f), 0.0f);
    g[(size_t)r * NM_STRIDE + 2] = 1.0f;
    g[(size_t)r * NM_STRIDE + 3] = 1.0f;
}

// --thalamus: the residual rule x + (x - x_in)(g * 1 + -1) on a block's whole change (src/v51b.rs:323-325)
__global__ void relay_res_kernel(float* x, const float* __restrict__ x_in, const float* __restrict__ g, int64_t n, int d) {
    pdl_enter();
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    const float gm1 = add(mul(g[(i / d) * NM_STRIDE], 1.0f), -1.0f);
    const float4 a = *reinterpret_cast<const float4*>(x + i), b = *reinterpret_cast<const float4*>(x_in + i);
    *reinterpret_cast<float4*>(x + i) = make_float4(add(a.x, mul(sub(a.x, b.x), gm1)), add(a.y, mul(sub(a.y, b.y), gm1)),
                                                    add(a.z, mul(sub(a.z, b.z), gm1)), add(a.w, mul(sub(a.w, b.w), gm1)));
}

// ---------------------------------------------------------------------------------------------------- memory: gates
// src/model/fstep/arch.rs:685-803 for one row per block of threads, after the two stages of the gate projections.
// FAST (the tolerance mode): the sums of squares and the two dot products are summed by a warp each (another order) and
// the gates use the CUDA library's exp and log; everything else is the same.
template <bool FAST>
__global__ void mem_prep_kernel(const MemPrepArgs a) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int d = a.d, hs = a.hs, nh = d / hs;
    const int r = blockIdx.x, tid = threadIdx.x, T = blockDim.x;
    float* q = sm;            // [d] raw, then unit
    float* kr = q + d;        // [d] raw key
    float* ek = kr + d;       // [d] raw erase key, then unit
    float* wv = ek + d;       // [d] w = k b
    float* ahv = wv + d;      // [d] ah = e (b alpha)
    float* inv_q = ahv + d;   // [nh]
    float* inv_k = inv_q + nh;
    float* inv_e = inv_k + nh;

    const float* pr = a.proj + (size_t)r * a.ldp;
    // (all of a thread's loads before its first store: the compiler cannot move a load above a store it cannot tell apart)
    constexpr int LD = 4;
    for (int c0 = tid; c0 < d; c0 += T * LD) {
        float lq[LD], lk[LD], le[LD];
#pragma unroll
        for (int u = 0; u < LD; ++u) {
            const int c = c0 + u * T;
            const bool in = c < d;
            lq[u] = in ? pr[c] : 0.0f;
            lk[u] = in ? pr[d + c] : 0.0f;
            le[u] = in ? pr[3 * d + c] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < LD; ++u) {
            const int c = c0 + u * T;
            if (c < d) {
                q[c] = lq[u];
                kr[c] = lk[u];
                ek[c] = add(lk[u], le[u]);
            }
        }
    }
    __syncthreads();
    // the gate phase's inputs for this thread's first channels are requested now, so that their latency passes while the
    // sums of squares run
    constexpr int PRE = 3;
    float p_lra[PRE], p_lrb[PRE], p_off[PRE], p_v[PRE], p_v0[PRE], p_za[PRE], p_zb[PRE];
    const float* zr = a.z + (size_t)r * a.gate_cols;
    const float vres0 = a.vres ? a.vres[0] : 0.0f, vres1 = a.vres ? a.vres[1] : 0.0f;
#pragma unroll
    for (int u = 0; u < PRE; ++u) {
        const int c = tid + u * T;
        const bool in = c < d;
        const size_t o = (size_t)r * d + (in ? c : 0);
        const int e = (in ? c : 0) / hs;
        p_za[u] = add(zr[2 * a.rank + e], a.ba[e]);
        p_zb[u] = add(zr[2 * a.rank + nh + e], a.bb[e]);
        p_lra[u] = in ? __ldg(a.lra + o) : 0.0f;
        p_lrb[u] = in ? __ldg(a.lrb + o) : 0.0f;
        p_off[u] = in ? __ldg(a.off + c) : 0.0f;
        p_v[u] = in ? pr[2 * d + c] : 0.0f;
        p_v0[u] = (in && !a.first && a.vres) ? a.v_first[o] : 0.0f;
    }
    // the three sums of squares per head, each in order by one thread; spread over the warps
    if (FAST) {
        for (int it = tid >> 5; it < 3 * nh; it += T >> 5) {
            const int which = it / nh, e = it % nh;
            const float* src = (which == 0 ? q : which == 1 ? kr : ek) + e * hs;
            float s = 0.0f;
            for (int i = tid & 31; i < hs; i += 32) s = fmaf(src[i], src[i], s);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if ((tid & 31) == 0) (which == 0 ? inv_q : which == 1 ? inv_k : inv_e)[e] = rsqrtf_(s + (float)1e-6);
        }
    } else {
    for (int it = tid; it < 3 * nh * 32; it += T) {
        if (it & 31) continue;
        const int which = (it >> 5) / nh, e = (it >> 5) % nh;
        const float* src = (which == 0 ? q : which == 1 ? kr : ek) + e * hs;
        (which == 0 ? inv_q : which == 1 ? inv_k : inv_e)[e] = inv_l2_seq(src, hs);
    }
    }
    __syncthreads();
    bool bad = false;
    const float ach = a.ach ? a.ach[(size_t)r * a.ach_stride] : 1.0f;
    auto gates = [&](int c, float in_lra, float in_lrb, float in_off, float v, float v0, float za, float zb) {
        const int e = c / hs;
        const size_t o = (size_t)r * d + c;
        float la, be;
        if (FAST) {
            const float xa = (za + in_off) + in_lra, xb = zb + in_lrb;
            la = -(fmaxf(-xa, 0.0f) + ::log1pf(::expf(-fabsf(xa))));
            be = 2.0f / (1.0f + ::expf(-xb));
        } else {
            la = log_sigmoid(add(add(za, in_off), in_lra));
            be = add(mul(sigmoid(add(zb, in_lrb)), 2.0f), 0.0f);
        }
        if (a.rh_w) be = mul(be, a.rh_w[(size_t)r * nh + e]);  // --rhythm: the write gate, before ACh's clamp
        if (a.ach) {  // --neuromod ACh: times its signal, kept in [0, 2] (maximum, then minimum: src/model/fstep/arch.rs:1121-1129)
            be = mul(be, ach);
            be = be < 0.0f ? 0.0f : be;
            be = be > 2.0f ? 2.0f : be;
        }
        const float ex = FAST ? ::expf(la) : expf_(la);
        const float qn = mul(q[c], inv_q[e]);
        const float kn = mul(kr[c], inv_k[e]);
        const float en = mul(ek[c], inv_e[e]);
        if (a.first) {
            a.v_first[o] = v;
        } else if (a.vres) {
            // (1 + p0) v + p1 v0 (src/model/fstep/arch.rs:697-702)
            const float p0 = add(mul(vres0, 1.0f), 1.0f);
            v = add(mul(v, p0), mul(v0, vres1));
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
        if (a.be_out) a.be_out[o] = be;
        if (a.qn_out) {
            a.qn_out[o] = qn;
            a.la_out[o] = la;
        }
        if (a.qs) a.qs[o] = mul(qn, add(mul(1.0f, a.mom), 0.0f));  // q * (1 * M + 0) (src/model/fstep/arch.rs:784)
        q[c] = qn;
        wv[c] = w;
        ahv[c] = ah;
    };
#pragma unroll
    for (int u = 0; u < PRE; ++u) {
        const int c = tid + u * T;
        if (c < d) gates(c, p_lra[u], p_lrb[u], p_off[u], p_v[u], p_v0[u], p_za[u], p_zb[u]);
    }
    for (int c = tid + PRE * T; c < d; c += T) {
        const size_t o = (size_t)r * d + c;
        const int e = c / hs;
        gates(c, a.lra[o], a.lrb[o], a.off[c], pr[2 * d + c], (!a.first && a.vres) ? a.v_first[o] : 0.0f, add(zr[2 * a.rank + e], a.ba[e]),
              add(zr[2 * a.rank + nh + e], a.bb[e]));
    }
    if (bad) atomicOr(a.status, ST_NONFINITE);
    __syncthreads();
    // q.w and q.ah, each summed in order from 0 (src/model/fstep/arch.rs:789-797); one thread per sum, in separate warps
    if (FAST) {
        for (int role = tid >> 5; role < 2 * nh; role += T >> 5) {
            const int e = role % nh;
            const float *av = q + e * hs, *bvec = (role < nh ? wv : ahv) + e * hs;
            float s = 0.0f;
            for (int i = tid & 31; i < hs; i += 32) s = fmaf(av[i], bvec[i], s);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if ((tid & 31) == 0) (role < nh ? a.qw : a.qa)[(size_t)r * nh + e] = s;
        }
        return;
    }
    for (int it = tid; it < 2 * nh * 32; it += T) {
        if (it & 31) continue;
        const int role = it >> 5, e = role % nh;
        const float* bvec = role < nh ? wv : ahv;
        (role < nh ? a.qw : a.qa)[(size_t)r * nh + e] = dot_seq(q + e * hs, bvec + e * hs, hs);
    }
}


// ---------------------------------------------------------------------------------------------------- memory: output
// head norm, then the silu output gate (src/model/fstep/arch.rs:842-852)
__global__ void mem_post_kernel(const float* __restrict__ y_raw, const float* __restrict__ gate, int ldg, int M, int d, int hs, float* __restrict__ y,
                                uint16_t* __restrict__ limbs, const float* __restrict__ rh_r) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const int nh = d / hs, r = blockIdx.x, tid = threadIdx.x, T = blockDim.x;
    float* ys = sm;
    float* inv = sm + d;
    for (int c = tid; c < d; c += T) ys[c] = y_raw[(size_t)r * d + c];
    __syncthreads();
    if (limbs) {  // the tolerance mode: a warp sums a head's squares (another order)
        for (int e = tid >> 5; e < nh; e += T >> 5) {
            float sq = 0.0f;
            for (int i = tid & 31; i < hs; i += 32) sq = fmaf(ys[e * hs + i], ys[e * hs + i], sq);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if ((tid & 31) == 0) inv[e] = rsqrtf_(sq * (float)(1.0 / (double)hs) + NORM_EPS);
        }
    } else {
        for (int e = tid; e < nh; e += T) inv[e] = inv_rms_seq(ys + e * hs, hs);
    }
    __syncthreads();
    for (int c = tid; c < d; c += T) {
        float v = mul(ys[c], inv[c / hs]);
        if (rh_r) v = mul(v, rh_r[(size_t)r * nh + c / hs]);
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
__global__ void kwta_kernel(const float* __restrict__ u, int M, int n, int k, int relu2, float* __restrict__ out, uint16_t* __restrict__ limbs) {
    pdl_enter();
    extern __shared__ uint32_t keys[];  // [n] keys
    const int r = blockIdx.x, tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5;
    const float* ur = u + (size_t)r * n;
    float* orow = out + (size_t)r * n;
    if (k >= n) {
        for (int i = tid; i < n; i += T) {
            float v = fmaxf(mul(ur[i], 1.0f), 0.0f);
            v = relu2 ? mul(v, v) : v;
            orow[i] = v;
            if (limbs) store_limbs(limbs, (int64_t)M * n, (int64_t)r * n + i, v);
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
        const float ov = relu2 ? mul(o, o) : o;
        orow[i] = ov;
        if (limbs) store_limbs(limbs, (int64_t)M * n, (int64_t)r * n + i, ov);
    }
}

// ---------------------------------------------------------------------------------------------------- dense mix
// src/model/fstep/arch.rs:1014-1024: the block's output joins the streams, then x <- x + sum_j stream_j w_j in order.
__global__ void dense_mix_kernel(float* x, float* streams, const float* __restrict__ w, int n_streams, int64_t MD) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= MD) return;
    const float xv = x[i];
    float mix = xv;
    for (int j = 0; j < n_streams - 1; ++j) mix = add(mix, mul(streams[(int64_t)j * MD + i], w[j]));  // every load before the first store
    mix = add(mix, mul(xv, w[n_streams - 1]));
    streams[(int64_t)(n_streams - 1) * MD + i] = xv;
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

void launch_embed(cudaStream_t st, const float* tok_emb, const uint32_t* tok, int M, int d, int vocab, float* x, float* stream0, uint32_t* status,
                  const float* letters) {
    launch_k(embed_kernel, dim3(M), dim3(128), 0, st, tok_emb, tok, M, d, vocab, x, stream0, status, letters);
}

void launch_rmsnorm(cudaStream_t st, const float* x, const float* gain, int M, int n, float* y, uint16_t* limbs) {
    const int warps = 4;
    const size_t smem = (size_t)warps * n * sizeof(float);
    opt_in_smem(rmsnorm_kernel, smem);
    launch_k(rmsnorm_kernel, dim3((M + warps - 1) / warps), dim3(warps * 32), smem, st, x, gain, M, n, y, limbs);
}

bool gate_z_few_covers(const float* x, const float* W, int M, int d, int n) {
    const size_t sm = ((size_t)d * 4 + (size_t)GZF_ROWS * d + d + GZF_ROWS) * sizeof(float);
    return M <= 2 * GZF_ROWS && n % 4 == 0 && d % 4 == 0 && !((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x)) & 15) && sm <= 200 * 1024;
}

// norm_gain (a few rows only: ask gate_z_few_covers first): x is not normed yet, the kernel takes its RMS norm with this gain
void launch_chain_gemv(cudaStream_t st, const float* x, const float* W, int M, int d, int n, int chunk_rows, float* out, const float* norm_gain) {
    // a few rows: the columns spread over blocks of four
    if (gate_z_few_covers(x, W, M, d, n) && !(reinterpret_cast<uintptr_t>(norm_gain) & 15)) {
        const size_t sm = ((size_t)d * 4 + (size_t)GZF_ROWS * d + d + GZF_ROWS) * sizeof(float);
        opt_in_smem(gate_z_few_kernel, sm);
        launch_k(gate_z_few_kernel, dim3(n / 4, (M + GZF_ROWS - 1) / GZF_ROWS), dim3(GZF_THREADS), sm, st, x, W, M, d, n, out, norm_gain);
        return;
    }
    if (norm_gain) {   // never: the caller asked first
        if (g_launch_error == cudaSuccess) g_launch_error = cudaErrorInvalidValue;
        return;
    }
    // a few rows per block share the staged weights
    // rows per block: one thread per (row, column), the rows' inputs within about 96 KB of shared memory
    const int RB = std::max(1, std::min(256 / n, (int)((96 * 1024) / ((size_t)d * sizeof(float))))), threads = ((RB * n + 31) / 32) * 32;
    // as many chunks of the weights in flight as shared memory holds (all of them at d = 768)
    const size_t chunk = (size_t)chunk_rows * n * sizeof(float), rows_b = (size_t)RB * d * sizeof(float);
    const int S = (int)std::max<size_t>(1, std::min<size_t>({(size_t)(d / chunk_rows), (size_t)8, (220 * 1024 - rows_b) / chunk}));
    const size_t smem = rows_b + S * chunk;
    opt_in_smem(gate_z_kernel, smem);
    launch_k(gate_z_kernel, dim3((M + RB - 1) / RB), dim3(threads), smem, st, x, W, M, d, n, chunk_rows, RB, S, out);
}

void launch_dend_gain(cudaStream_t st, const float* z1, int rank, const float* B, int M, int H, float* act) {
    const size_t smem = (size_t)std::min(M, LR_ROWS) * rank * sizeof(float);
    const dim3 grid((H + LR_COLS - 1) / LR_COLS, (M + LR_ROWS - 1) / LR_ROWS), block(LR_COLS * LR_LANES);
    if (rank == 32) {
        opt_in_smem(dend_gain_kernel<32>, smem);
        launch_k(dend_gain_kernel<32>, grid, block, smem, st, z1, rank, B, M, H, act);
    } else {
        opt_in_smem(dend_gain_kernel<0>, smem);
        launch_k(dend_gain_kernel<0>, grid, block, smem, st, z1, rank, B, M, H, act);
    }
}

void launch_nucleus(cudaStream_t st, const float* z, const float* bias, int k, int M, float* sig) {
    launch_k(nucleus_kernel, dim3((M * 4 + 255) / 256), dim3(256), 0, st, z, bias, k, M, sig);
}

void launch_add_into(cudaStream_t st, float* x, const float* y, int64_t n, const float* row_gain, int d) {
    launch_k(add_into_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, st, x, y, n, row_gain, d);
}

void launch_relay(cudaStream_t st, const float* thr, float* acc, bool first, int reads, const float* G, const float* bias, int M, float* g) {
    const float mulf = (float)(1.0 / std::sqrt((double)reads));
    launch_k(relay_kernel, dim3((M + 127) / 128), dim3(128), 0, st, thr, acc, first ? 1 : 0, mulf, G, bias, M, g);
}

void launch_relay_res(cudaStream_t st, float* x, const float* x_in, const float* g, int M, int d) {
    const int64_t n = (int64_t)M * d;
    launch_k(relay_res_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, st, x, x_in, g, n, d);
}

void launch_mem_prep(cudaStream_t st, const MemPrepArgs& a) {
    launch_mem_gates(st, a);
    launch_mem_prep_rows(st, a);
}

// the gates' two projection stages (they read the normed input only, so they can run beside the q|k|v|e|g product)
void launch_mem_gates(cudaStream_t st, const MemPrepArgs& a) {
    // stage one
    launch_chain_gemv(st, a.h, a.gate_w, a.M, a.d, a.gate_cols, a.gate_chunk, a.z, a.h_gain);
    launch_mem_gates_low(st, a);
}

// stage two alone (stage one's products a.z exist already)
void launch_mem_gates_low(cudaStream_t st, const MemPrepArgs& a) {
    {
        const size_t smem = (size_t)std::min(a.M, LR_ROWS) * 2 * a.rank * sizeof(float);
        const dim3 grid((a.d + LR_COLS - 1) / LR_COLS, (a.M + LR_ROWS - 1) / LR_ROWS), block(LR_COLS * LR_LANES);
        if (a.rank == 32) {
            opt_in_smem(lowrank_kernel<32>, smem);
            launch_k(lowrank_kernel<32>, grid, block, smem, st, a.z, a.gate_cols, 0, a.rank, a.rank, a.wa2, a.wb2, a.M, a.d, a.lra, a.lrb);
        } else {
            opt_in_smem(lowrank_kernel<0>, smem);
            launch_k(lowrank_kernel<0>, grid, block, smem, st, a.z, a.gate_cols, 0, a.rank, a.rank, a.wa2, a.wb2, a.M, a.d, a.lra, a.lrb);
        }
    }
}

// everything per row once the projections and the gates' stages exist
void launch_mem_prep_rows(cudaStream_t st, const MemPrepArgs& a) {
    const int nh = a.d / a.hs;
    const size_t smem = ((size_t)5 * a.d + 3 * nh + 4) * sizeof(float);
    if (a.fast) {
        opt_in_smem(mem_prep_kernel<true>, smem);
        launch_k(mem_prep_kernel<true>, dim3(a.M), dim3(256), smem, st, a);
    } else {
        opt_in_smem(mem_prep_kernel<false>, smem);
        launch_k(mem_prep_kernel<false>, dim3(a.M), dim3(256), smem, st, a);
    }
}

void launch_mem_post(cudaStream_t st, const float* y_raw, const float* gate, int ldg, int M, int d, int hs, float* y, uint16_t* limbs,
                     const float* rh_r) {
    const size_t smem = ((size_t)d + d / hs) * sizeof(float);
    opt_in_smem(mem_post_kernel, smem);
    launch_k(mem_post_kernel, dim3(M), dim3(256), smem, st, y_raw, gate, ldg, M, d, hs, y, limbs, rh_r);
}

void launch_kwta(cudaStream_t st, const float* u, int M, int n, int k, int relu2, float* a, uint16_t* limbs) {
    const size_t smem = (size_t)n * sizeof(uint32_t);
    opt_in_smem(kwta_kernel, smem);
    launch_k(kwta_kernel, dim3(M), dim3(256), smem, st, u, M, n, k, relu2, a, limbs);
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

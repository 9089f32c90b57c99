// The engram's causal read over a whole prompt chunk on the tensor cores (sm_100a: TMA + tcgen05.mma + tensor memory).
//
// The reference reads the store once per token (design-tests/nn/gpu/src/model/fstep.rs:303-356,
// src/model/fstep/arch.rs:909-974): the token's key and value join the store, then per head softmax(K q / sqrt(hs)) V
// over every key so far.  Token by token that re-reads the whole store for every token of a prompt.  This kernel is
// the tolerance mode's form for a chunk of T tokens: all T keys and values are appended first, then one block per
// (row, head, 128 queries) walks the store in tiles of 64 keys, each tile read once for its 128 queries, with the causal
// limit (query t sees keys 0 .. n0 + t, n0 the count before the chunk) applied as a mask.  It agrees with the one-token
// read to rounding (another summation order, exp2-based exponentials), not bit for bit.
//
// Arithmetic: the store is bf16 (exact operands); the query, times 1/sqrt(64) (a power of two), is carried as three
// bf16 limbs, so a score is the f32 product to about 2^-24.  Two passes over the keys: the first leaves each query's
// maximum and sum of exponentials, the second forms p = exp(s - max) / sum as two bf16 limbs (2^-17 of p) and
// accumulates O += p V in tensor memory; nothing is ever rescaled.  The value tile arrives [key][channel]; the product
// wants it K-major in the keys, so three warps transpose it in shared memory into the swizzled layout (and write
// zeros for slots beyond the last key present, whose bytes may be anything).
//
// Roles in a block of 256 threads: warps 0-3 own one query each (tensor-memory lane = query), warp 4's first lane
// issues the copies and the multiply-adds, warps 5-7 transpose values.  Every wait is bounded; a thread whose wait
// runs out raises ST_WAIT_TIMEOUT, stops waiting, and the block stores nothing.
#include <cuda.h>
#include <cuda_runtime.h>

#include "ava_math.h"
#include "bf16_hw.cuh"
#include "kernels.cuh"
#include "tc_common.cuh"

namespace ava {

namespace {

using namespace tcc;

constexpr int EA_THREADS = 256, EA_Q = 128, EA_KEYS = 64, EA_HS = 64;
constexpr uint32_t EA_TILE_Q = EA_Q * EA_HS * 2;       // 16 KB: 128 rows of 64 bf16
constexpr uint32_t EA_TILE_K = EA_KEYS * EA_HS * 2;    // 8 KB
constexpr uint32_t EA_OFF_P = 3 * EA_TILE_Q, EA_OFF_K = EA_OFF_P + 2 * EA_TILE_Q, EA_OFF_VT = EA_OFF_K + EA_TILE_K, EA_OFF_V = EA_OFF_VT + EA_TILE_K,
                   EA_OFF_BAR = EA_OFF_V + EA_TILE_K, EA_SMEM = EA_OFF_BAR + 64 + 1024;

__device__ __forceinline__ void limbs3(float x, uint16_t& l0, uint16_t& l1, uint16_t& l2) { limbs3_hw(x, l0, l1, l2); }
__device__ __forceinline__ uint32_t pack2(uint16_t a, uint16_t b) { return a | ((uint32_t)b << 16); }
__device__ __forceinline__ void bar_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory"); }
__device__ __forceinline__ void fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate ? 1u : 0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}

// this chunk's keys and values join the store: token t of row r at slot start + n + t (the host has checked that the
// ring does not wrap inside the chunk); grid (rows, T)
__global__ void engram_append_chunk_kernel(const EngramChunkArgs a) {
    pdl_enter();
    const int r = blockIdx.x, t = blockIdx.y, d = a.d, nh = d / EA_HS;
    const int slot = a.start[r] + a.n[r] + t;
    if (slot >= a.cap) {
        if (threadIdx.x == 0) atomicOr(a.status, ST_ENGRAM_FULL);
        return;
    }
    const float* qkv = a.qkv + ((size_t)t * a.M + r) * 3 * d;
    uint16_t* kk = reinterpret_cast<uint16_t*>(a.k);
    uint16_t* vv = reinterpret_cast<uint16_t*>(a.v);
    const size_t row_base = (size_t)r * nh * a.cap * EA_HS;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const size_t o = row_base + ((size_t)(c / EA_HS) * a.cap + slot) * EA_HS + c % EA_HS;
        kk[o] = f_to_bf16(qkv[d + c]);
        vv[o] = f_to_bf16(qkv[2 * d + c]);
    }
}

__global__ void engram_count_add_kernel(int32_t* n, int M, int T, int cap) {
    pdl_enter();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < M) n[r] = min(n[r] + T, cap);
}

__global__ void __launch_bounds__(EA_THREADS) engram_chunk_attn_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                                                      const EngramChunkArgs a) {
    pdl_enter();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (s32(smem_raw) & 1023u)) & 1023u);
    unsigned char* sQ = smem;              // three limb tiles [128 queries][64 channels]
    unsigned char* sP = smem + EA_OFF_P;   // two limb tiles [128 queries][64 keys]
    unsigned char* sK = smem + EA_OFF_K;   // [64 keys][64 channels], as the copy leaves it (swizzled)
    unsigned char* sVt = smem + EA_OFF_VT; // [64 channels][64 keys], swizzled, written by the transposing warps
    unsigned char* sV = smem + EA_OFF_V;   // [64 keys][64 channels], plain rows of 128 bytes
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + EA_OFF_BAR);
    uint64_t *full = bars, *s_ready = bars + 1, *s_free = bars + 2, *p_ready = bars + 3, *vt_ready = bars + 4, *pv_done = bars + 5, *full_v = bars + 6;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = blockIdx.x * EA_Q, h = blockIdx.y, r = blockIdx.z, nh = a.d / EA_HS;
    const int n0 = a.n[r], start = a.start[r];
    const int n_valid = min(n0 + a.T, a.cap - start);          // keys present once the chunk has joined
    const int hi = min(n0 + min(t0 + EA_Q, a.T), n_valid);     // keys some query of this tile may see
    const int n_tiles = (hi + EA_KEYS - 1) / EA_KEYS;
    const int kv_row0 = (r * nh + h) * a.cap + start;

    if (tid == 0) {
        bar_init(full, 1);
        bar_init(s_ready, 1);
        bar_init(s_free, EA_Q);
        bar_init(p_ready, EA_Q);
        bar_init(vt_ready, 96);
        bar_init(pv_done, 1);
        bar_init(full_v, 1);   // the value tiles have a barrier of their own: its phases count the second pass's tiles only
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the queries, scaled and split into limbs, into the swizzled operand layout: thread = query
    const int t = t0 + tid;
    const bool q_valid = tid < EA_Q && t < a.T;
    if (tid < EA_Q) {
        const float* q = a.qkv + ((size_t)(q_valid ? t : 0) * a.M + r) * 3 * a.d + h * EA_HS;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            float x[8];
            if (q_valid) {
                const float4 u = *reinterpret_cast<const float4*>(q + ch * 8), v = *reinterpret_cast<const float4*>(q + ch * 8 + 4);
                x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w; x[4] = v.x; x[5] = v.y; x[6] = v.z; x[7] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = 0.0f;
            }
            uint16_t l[3][8];
#pragma unroll
            for (int i = 0; i < 8; ++i) limbs3(x[i] * 0.125f, l[0][i], l[1][i], l[2][i]);
            const uint32_t off = swz128(tid, ch * 8);
#pragma unroll
            for (int p = 0; p < 3; ++p)
                *reinterpret_cast<uint4*>(sQ + p * EA_TILE_Q + off) = make_uint4(pack2(l[p][0], l[p][1]), pack2(l[p][2], l[p][3]), pack2(l[p][4], l[p][5]), pack2(l[p][6], l[p][7]));
        }
        fence_async();
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = *tmem_slot, tmem_s = tmem, tmem_o = tmem + 64;
    constexpr uint32_t idesc = instr_desc(64);
    bool ok = true;

    if (tid < EA_Q) {
        // ---- the queries' side: statistics in the first pass, weights in the second
        const int lim = q_valid ? n0 + t + 1 : 0;   // keys [0, lim) are visible
        const uint32_t lane_base = ((uint32_t)(warp * 32) << 16);
        float m = -INFINITY, l = 0.0f;
        uint32_t s[64];
        for (int kt = 0; kt < n_tiles && ok; ++kt) {
            ok = __all_sync(0xffffffffu, bar_wait(s_ready, (uint32_t)(kt & 1)));   // the same answer for the whole warp: the reads below are warp-wide
            if (!ok) break;
            tc_after();
            tmem_ld32(tmem_s + lane_base, s);
            tmem_ld32(tmem_s + lane_base + 32, s + 32);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            tc_before();
            bar_arrive(s_free);
            const int k0 = kt * EA_KEYS;
            float tm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 64; ++j)
                if (k0 + j < lim) tm = fmaxf(tm, __uint_as_float(s[j]));
            if (tm > -INFINITY) {
                const float mn = fmaxf(m, tm);
                float sum = 0.0f;
#pragma unroll
                for (int j = 0; j < 64; ++j)
                    if (k0 + j < lim) sum += __expf(__uint_as_float(s[j]) - mn);
                l = l * __expf(m - mn) + sum;   // exp(-inf) = 0 the first time
                m = mn;
            }
        }
        const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
        for (int kt = 0; kt < n_tiles && ok; ++kt) {
            ok = __all_sync(0xffffffffu, bar_wait(s_ready, (uint32_t)((n_tiles + kt) & 1)));
            if (!ok) break;
            tc_after();
            tmem_ld32(tmem_s + lane_base, s);
            tmem_ld32(tmem_s + lane_base + 32, s + 32);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int k0 = kt * EA_KEYS;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                uint16_t p0[8], p1[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int j = ch * 8 + i;
                    const float p = (k0 + j < lim) ? __expf(__uint_as_float(s[j]) - m) * inv_l : 0.0f;
                    p0[i] = bf16_rn_hw(p);
                    p1[i] = bf16_rn_hw(p - bf16_widen(p0[i]));
                }
                const uint32_t off = swz128(tid, ch * 8);
                *reinterpret_cast<uint4*>(sP + off) = make_uint4(pack2(p0[0], p0[1]), pack2(p0[2], p0[3]), pack2(p0[4], p0[5]), pack2(p0[6], p0[7]));
                *reinterpret_cast<uint4*>(sP + EA_TILE_Q + off) = make_uint4(pack2(p1[0], p1[1]), pack2(p1[2], p1[3]), pack2(p1[4], p1[5]), pack2(p1[6], p1[7]));
            }
            fence_async();
            tc_before();
            bar_arrive(p_ready);
        }
        // ---- the mix, once the last multiply-add has landed
        if (n_tiles > 0) ok = __all_sync(0xffffffffu, ok && bar_wait(pv_done, (uint32_t)((n_tiles - 1) & 1)));
        if (ok && n_tiles > 0) {
            tc_after();
            tmem_ld32(tmem_o + lane_base, s);
            tmem_ld32(tmem_o + lane_base + 32, s + 32);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (q_valid) {
                float* o = a.o + ((size_t)t * a.M + r) * a.d + h * EA_HS;
#pragma unroll
                for (int j = 0; j < 64; j += 4)
                    *reinterpret_cast<float4*>(o + j) = make_float4(__uint_as_float(s[j]), __uint_as_float(s[j + 1]), __uint_as_float(s[j + 2]), __uint_as_float(s[j + 3]));
            }
        }
    } else if (tid == EA_Q) {
        // ---- copies and multiply-adds, one thread
        auto scores = [&]() {
            bool first = true;
#pragma unroll
            for (int p = 0; p < 3; ++p) {
                const uint64_t da = operand_desc(sQ + p * EA_TILE_Q), db = operand_desc(sK);
#pragma unroll
                for (int k16 = 0; k16 < EA_HS / 16; ++k16) {
                    mma_f16(tmem_s, da + 2u * k16, db + 2u * k16, idesc, !first);
                    first = false;
                }
            }
        };
        for (int kt = 0; kt < n_tiles && ok; ++kt) {   // pass one: scores only
            if (kt > 0) ok = bar_wait(s_free, (uint32_t)((kt - 1) & 1));
            if (!ok) break;
            bar_expect(full, EA_TILE_K);
            tma_load(sK, &map_k, 0, kv_row0 + kt * EA_KEYS, full);
            ok = bar_wait(full, (uint32_t)(kt & 1));
            if (!ok) break;
            tc_after();
            scores();
            mma_commit(s_ready);
        }
        for (int kt = 0; kt < n_tiles && ok; ++kt) {   // pass two: scores, then the weighted values
            ok = kt > 0 ? bar_wait(pv_done, (uint32_t)((kt - 1) & 1)) : bar_wait(s_free, (uint32_t)((n_tiles - 1) & 1));
            if (!ok) break;
            bar_expect(full, EA_TILE_K);
            tma_load(sK, &map_k, 0, kv_row0 + kt * EA_KEYS, full);
            bar_expect(full_v, EA_TILE_K);
            tma_load(sV, &map_v, 0, kv_row0 + kt * EA_KEYS, full_v);
            ok = bar_wait(full, (uint32_t)((n_tiles + kt) & 1));
            if (!ok) break;
            tc_after();
            scores();
            mma_commit(s_ready);
            ok = bar_wait(p_ready, (uint32_t)(kt & 1)) && bar_wait(vt_ready, (uint32_t)(kt & 1));
            if (!ok) break;
            tc_after();
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const uint64_t da = operand_desc(sP + p * EA_TILE_Q), db = operand_desc(sVt);
#pragma unroll
                for (int k16 = 0; k16 < EA_KEYS / 16; ++k16) mma_f16(tmem_o, da + 2u * k16, db + 2u * k16, idesc, !(kt == 0 && p == 0 && k16 == 0));
            }
            mma_commit(pv_done);
        }
    } else if (warp >= 5) {
        // ---- the value tile, transposed into the operand layout: 2 x 2 pieces, 96 threads
        const int w = tid - 160;
        for (int kt = 0; kt < n_tiles && ok; ++kt) {
            if (kt > 0) ok = bar_wait(pv_done, (uint32_t)((kt - 1) & 1));   // the product before has read the tile
            if (ok) ok = bar_wait(full_v, (uint32_t)(kt & 1));
            if (!ok) break;
            const int k0 = kt * EA_KEYS;
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(sV);
            for (int b = w; b < 1024; b += 96) {
                const int jb = b >> 5, cb = b & 31;
                uint32_t x0 = raw[(2 * jb) * 32 + cb], x1 = raw[(2 * jb + 1) * 32 + cb];
                if (k0 + 2 * jb >= n_valid) x0 = 0u;       // a slot past the last key: its bytes may be anything
                if (k0 + 2 * jb + 1 >= n_valid) x1 = 0u;
                *reinterpret_cast<uint32_t*>(sVt + swz128(2 * cb, 2 * jb)) = (x0 & 0xffffu) | (x1 << 16);
                *reinterpret_cast<uint32_t*>(sVt + swz128(2 * cb + 1, 2 * jb)) = (x0 >> 16) | (x1 & 0xffff0000u);
            }
            fence_async();
            bar_arrive(vt_ready);
        }
    }
    if (!ok) atomicOr(a.status, ST_WAIT_TIMEOUT);
    tc_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
}

}  // namespace

// The chunk's keys and values join the store, the causal read of all T tokens, and the counts move on by T.
// false: not this kernel's case (head size 64 and a bf16 store only) or no tensor-map encoder.
bool launch_engram_chunk(cudaStream_t st, const EngramChunkArgs& a) {
    if (a.hs != EA_HS || !a.bf16 || a.d % EA_HS || a.T < 1 || a.M < 1) return false;
    const int nh = a.d / EA_HS;
    const uint64_t rows = (uint64_t)a.M * nh * a.cap;
    if (rows > 0x7fffffffull) return false;
    CUtensorMap mk, mv;
    if (!make_map(&mk, a.k, rows, EA_HS, EA_KEYS, true) || !make_map(&mv, a.v, rows, EA_HS, EA_KEYS, false)) return false;
    launch_k(engram_append_chunk_kernel, dim3(a.M, a.T), dim3(256), 0, st, a);
    cudaFuncSetAttribute(engram_chunk_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)EA_SMEM);
    prefer_max_shared(reinterpret_cast<const void*>(engram_chunk_attn_kernel), 100);
    launch_k(engram_chunk_attn_kernel, dim3((a.T + EA_Q - 1) / EA_Q, nh, a.M), dim3(EA_THREADS), EA_SMEM, st, mk, mv, a);
    launch_k(engram_count_add_kernel, dim3((a.M + 127) / 128), dim3(128), 0, st, a.n, a.M, a.T, a.cap);
    return true;
}

}  // namespace ava

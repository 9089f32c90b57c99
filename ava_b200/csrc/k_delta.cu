// The fast-weight memory's update + read with a block's slice of the state resident in shared memory (sm_100a): the form for
// a chunk of T tokens (prompt reading) and for the memory with momentum.  One token of the plain memory takes the streaming
// pass of k_stream.cu.
//
// Per head, F [hs, hs] f32 (row = key dimension, column = value dimension), as the reference's `head_rows`
// (design-tests/nn/gpu/src/model/fstep/arch.rs:256-337) without momentum:
//     rr  = e^T F                      (each column summed over the rows in order: row 0's product, then fma)
//     t1  = (q alpha)^T F
//     y   = (t1 + (q.w) v) - (q.ah) rr
//     F'  = (F * alpha_row + w v^T) - ah rr^T
// Columns are independent, so one block of threads owns a slice of CW columns of one head.  The state is kept
// SLICE-MAJOR in HBM: [row][head][slice][hs][CW], so a block's slice is one contiguous run of hs * CW * 4 bytes.  It
// comes into shared memory as a few large bulk copies (cp.async.bulk, one mbarrier per chunk of rows), the column sums
// run down the rows, the slice is updated in place in shared memory token after token, and it goes back with bulk stores
// once the chunk's last token is done: the state is read once and written once per CHUNK.
#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int MAX_CHUNKS = 16;
constexpr int THREADS = 256;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // polls (most back off ~64 ns) before a wait gives up: about a quarter second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// false when the wait ran out
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (i > 256) __nanosleep(64);
    }
    return false;
}
// the same with the caller's limit (a testing aid shortens it)
__device__ __forceinline__ bool mbar_wait_lim(uint64_t* bar, uint32_t parity, uint32_t limit) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (i > 256) __nanosleep(64);
    }
    return false;
}
// global -> shared, completion counted in bytes on the mbarrier; addresses and size multiples of 16
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// shared-memory loads as volatile asm: they keep their place ahead of the chains that use them
__device__ __forceinline__ float lds_f(const float* p) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ float4 lds_f4(const float* p) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ void bulk_store(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}

// The update + read for T tokens in a row (chunked prompt reading, and the memory with momentum): one block owns row m, head e,
// slice s; the block's slice comes into shared memory
// once, every token of the chunk updates it there in order, and it goes back to HBM once: the state traffic of a chunk
// is that of one token.  Per token the block needs the head's vectors (time-major [T][M][nh * hs]), all brought by
// bulk copies that overlap the other pass: alpha, w and ah of token t land while its column sums run; e, q*alpha of
// token t + 1 land while token t's update runs (the value slice is double-buffered: both passes read it).
// MOM: the memory's momentum (second matrix S, src/model/fstep/arch.rs:281-323): rr gains p2 S (an exact zero kept for
// the sign of zero), y gains (q M) S, F' = ((F alpha + w v^T) - ah rr^T) + S M, S' = ((S M + 0) + w v^T) - ah rr^T.
// DBG: the testing form, whose waits take the caller's poll limit and whose byte count for one chunk can be over-stated
// so that the wait on it runs out; the production form keeps the limit a compile-time constant.
template <int CW, bool MOM, bool DBG>
__global__ void __launch_bounds__(THREADS) mem_heads_seq_kernel(const MemHeadsArgs a, int T) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int hs = a.hs, cr = a.chunk_rows, nchunk = hs / cr, d = a.nh * hs;
    float* tile = reinterpret_cast<float*>(smem_raw);
    float* ve = tile + (size_t)hs * CW;
    float* vqg = ve + hs;
    float* vex = vqg + hs;
    float* vw = vex + hs;
    float* vah = vw + hs;
    float* vqs = vah + hs;                          // [hs] q * M (momentum only)
    float* vvb = vqs + (MOM ? hs : 0);              // [2][CW]
    float* rr = vvb + 2 * CW;
    float* t1 = rr + CW;
    float* tqv = t1 + CW;                           // [CW] (q M) S (momentum only)
    float* tileS = tqv + CW;                        // [hs][CW] the momentum matrix's slice (momentum only)
    uint64_t* bars = reinterpret_cast<uint64_t*>(tileS + (MOM ? (size_t)hs * CW : 0));  // slice chunks, then A, B
    uint64_t* barA = &bars[nchunk];
    uint64_t* barB = &bars[nchunk + 1];

    const int tid = threadIdx.x;
    const int slices = hs / CW;
    const int slice = blockIdx.x % slices;
    const int head = (blockIdx.x / slices) % a.nh;
    const int m = blockIdx.x / (slices * a.nh);
    const int c0 = slice * CW;
    const size_t ho = (size_t)head * hs;
    const size_t goff = (((size_t)m * a.nh + head) * hs * hs) + (size_t)slice * hs * CW;
    float* gslice = a.f + goff;
    float* gsliceS = MOM ? a.s + goff : nullptr;
    const uint32_t chunk_bytes = (uint32_t)(cr * CW * sizeof(float));
    const uint32_t vb = (uint32_t)(hs * sizeof(float));
    const size_t Md = (size_t)a.M * d;
    auto row_off = [&](int t) { return (size_t)t * Md + (size_t)m * d + ho; };

    auto fetch_a = [&](int t) {  // thread 0: what the column sums of token t read (+ its value slice)
        const size_t o = row_off(t);
        mbar_expect_tx(barA, (MOM ? 3 : 2) * vb + (uint32_t)(CW * sizeof(float)));
        bulk_load(ve, a.e + o, vb, barA);
        bulk_load(vqg, a.qg + o, vb, barA);
        if (MOM) bulk_load(vqs, a.qs + o, vb, barA);
        bulk_load(vvb + (t & 1) * CW, a.v + o + c0, (uint32_t)(CW * sizeof(float)), barA);
    };
    auto fetch_b = [&](int t) {  // thread 0: what the update of token t reads
        const size_t o = row_off(t);
        mbar_expect_tx(barB, 3 * vb);
        bulk_load(vex, a.ex + o, vb, barB);
        bulk_load(vw, a.w + o, vb, barB);
        bulk_load(vah, a.ah + o, vb, barB);
    };

    if (tid == 0) {
        for (int c = 0; c < nchunk + 2; ++c) mbar_init(&bars[c], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
        fetch_a(0);
        for (int c = 0; c < nchunk; ++c) {
            mbar_expect_tx(&bars[c], (MOM ? 2 : 1) * chunk_bytes + ((DBG && a.fault_chunk_plus1 == c + 1) ? 16u : 0u));
            bulk_load(tile + (size_t)c * cr * CW, gslice + (size_t)c * cr * CW, chunk_bytes, &bars[c]);
            if (MOM) bulk_load(tileS + (size_t)c * cr * CW, gsliceS + (size_t)c * cr * CW, chunk_bytes, &bars[c]);
        }
    }
    bool ok = true;
    auto wait = [&](uint64_t* bar, uint32_t par) { return DBG ? mbar_wait_lim(bar, par, a.wait_limit ? a.wait_limit : WAIT_LIMIT) : mbar_wait(bar, par); };
    const float mf = a.mom;
    const float gsx = add(mul(0.0f, mf), 0.0f);  // the factor of the recall's zero row p2 = e * (0 * M + 0)
    for (int c = 0; c < nchunk; ++c) ok = wait(&bars[c], 0) && ok;  // the slice is resident from here on
    if (__syncthreads_or(!ok)) {  // not even the slice arrived: nothing is computed, nothing stored
        if (tid == 0) atomicOr(a.status, ST_WAIT_TIMEOUT);
        return;
    }
    constexpr int QW = CW / 4, RPP = THREADS / QW;
    const int q4 = tid % QW, rg = tid / QW;
    for (int t = 0; t < T; ++t) {
        const uint32_t par = (uint32_t)(t & 1);
        // alpha, w, ah of this token: their buffers were last read by the update of token t - 1 (barrier at its end)
        if (tid == 0) fetch_b(t);
        ok = wait(barA, par) && ok;
        const float* vv = vvb + (t & 1) * CW;
        if (tid < CW) {
            // the column sums, eight rows fetched one batch ahead of the two chains (chains start from -0: see above)
            float r = -0.0f, s1 = -0.0f, z = -0.0f, tq = -0.0f;
            const float* p = tile + tid;
            const float* ps = tileS + tid;
            float f[8], ev[8], gv[8];
            // loads as volatile asm: here the slice is resident and the chains are the whole critical path, so the eight
            // rows fetched ahead must really be ahead (the compiler otherwise sinks them down to the multiply-adds)
            auto load8 = [&](int row, float* ff, float* ee, float* gg) {
#pragma unroll
                for (int i = 0; i < 8; ++i) ff[i] = lds_f(p + (size_t)(row + i) * CW);
                const float4 e0 = lds_f4(ve + row), e1 = lds_f4(ve + row + 4), g0 = lds_f4(vqg + row), g1 = lds_f4(vqg + row + 4);
                ee[0] = e0.x; ee[1] = e0.y; ee[2] = e0.z; ee[3] = e0.w; ee[4] = e1.x; ee[5] = e1.y; ee[6] = e1.z; ee[7] = e1.w;
                gg[0] = g0.x; gg[1] = g0.y; gg[2] = g0.z; gg[3] = g0.w; gg[4] = g1.x; gg[5] = g1.y; gg[6] = g1.z; gg[7] = g1.w;
            };
            load8(0, f, ev, gv);
            for (int row = 0; row < hs; row += 8) {
                float nf[8], ne[8], ng[8];
                if (row + 8 < hs) load8(row + 8, nf, ne, ng);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    r = fma(f[i], ev[i], r);
                    s1 = fma(f[i], gv[i], s1);
                }
                if (MOM) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float sv = ps[(size_t)(row + i) * CW];
                        z = fma(sv, mul(ev[i], gsx), z);
                        tq = fma(sv, vqs[row + i], tq);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    f[i] = nf[i];
                    ev[i] = ne[i];
                    gv[i] = ng[i];
                }
            }
            r = add(r, mul(1.0f, mul(0.0f, vv[tid])));
            if (MOM) {
                r = add(r, z);
                tqv[tid] = tq;
            }
            rr[tid] = r;
            t1[tid] = s1;
        }
        __syncthreads();
        // e, q*alpha of the next token: the sums above were their last readers
        if (tid == 0 && t + 1 < T) fetch_a(t + 1);
        const size_t ro = row_off(t);
        if (tid < CW) {
            const size_t qo = ((size_t)t * a.M + m) * a.nh + head;
            float yv = sub(add(t1[tid], mul(a.qw[qo], vv[tid])), mul(a.qa[qo], rr[tid]));
            if (MOM) yv = add(yv, tqv[tid]);
            a.y[ro + c0 + tid] = yv;
        }
        ok = wait(barB, par) && ok;
        {
            const float4 vb4 = *reinterpret_cast<const float4*>(vv + 4 * q4), rb4 = *reinterpret_cast<const float4*>(rr + 4 * q4);
#pragma unroll 4
            for (int row = rg; row < hs; row += RPP) {
                float4* p = reinterpret_cast<float4*>(tile + (size_t)row * CW) + q4;
                float4 f = *p;
                const float x = vex[row], w = vw[row], ah = vah[row];
                if (!MOM) {
                    f.x = sub(add(mul(f.x, x), mul(w, vb4.x)), mul(ah, rb4.x));
                    f.y = sub(add(mul(f.y, x), mul(w, vb4.y)), mul(ah, rb4.y));
                    f.z = sub(add(mul(f.z, x), mul(w, vb4.z)), mul(ah, rb4.z));
                    f.w = sub(add(mul(f.w, x), mul(w, vb4.w)), mul(ah, rb4.w));
                } else {
                    float4* q = reinterpret_cast<float4*>(tileS + (size_t)row * CW) + q4;
                    float4 sv = *q;
                    const float fv[4] = {f.x, f.y, f.z, f.w}, s4[4] = {sv.x, sv.y, sv.z, sv.w};
                    const float v4[4] = {vb4.x, vb4.y, vb4.z, vb4.w}, r4[4] = {rb4.x, rb4.y, rb4.z, rb4.w};
                    float fo[4], so[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float wv = mul(w, v4[k]), ar = mul(ah, r4[k]), sm = mul(s4[k], mf);
                        fo[k] = add(sub(add(mul(fv[k], x), wv), ar), sm);
                        so[k] = sub(add(add(sm, 0.0f), wv), ar);
                    }
                    f = make_float4(fo[0], fo[1], fo[2], fo[3]);
                    *q = make_float4(so[0], so[1], so[2], so[3]);
                }
                *p = f;
            }
        }
        __syncthreads();
    }
    // a wait ran out somewhere in the block: flag it and store nothing (the state keeps what it held before the chunk)
    if (__syncthreads_or(!ok)) {
        if (tid == 0) atomicOr(a.status, ST_WAIT_TIMEOUT);
        return;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        for (int c = 0; c < nchunk; ++c) {
            bulk_store(gslice + (size_t)c * cr * CW, tile + (size_t)c * cr * CW, chunk_bytes);
            if (MOM) bulk_store(gsliceS + (size_t)c * cr * CW, tileS + (size_t)c * cr * CW, chunk_bytes);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
}

size_t smem_bytes_seq(int hs, int cw, bool mom = false) {
    return ((size_t)hs * cw * (mom ? 2 : 1) + (mom ? 6 : 5) * (size_t)hs + 5 * (size_t)cw) * sizeof(float) + (MAX_CHUNKS + 2) * sizeof(uint64_t);
}

size_t smem_bytes(int hs, int cw) { return ((size_t)hs * cw + 5 * (size_t)hs + 3 * (size_t)cw) * sizeof(float) + (MAX_CHUNKS + 1) * sizeof(uint64_t); }  // (the two-blocks-per-SM rule of the tiling below)

}  // namespace

bool mem_heads_tiling(int hs, int* cw, int* chunk_rows, bool momentum) {
    if (hs % 16 != 0) return false;
    // the widest slice (128-byte rows) that leaves room for two blocks per SM, else 64-byte rows; with momentum two
    // matrices' slices share the block and the slice only has to fit
    int w = 32;
    if (momentum) {
        if (hs % w != 0 || smem_bytes_seq(hs, w, true) > 227 * 1024) w = 16;
        if (hs % w != 0 || smem_bytes_seq(hs, w, true) > 227 * 1024) return false;
    } else {
        if (hs % w != 0 || smem_bytes(hs, w) > 113 * 1024) w = 16;
        if (hs % w != 0 || smem_bytes(hs, w) > 227 * 1024) return false;
    }
    // chunks of at least 64 rows, at most MAX_CHUNKS of them, dividing the head
    int cr = hs <= 128 ? hs : 128;
    while (hs / cr > MAX_CHUNKS) cr *= 2;
    if (hs % cr != 0) return false;
    *cw = w;
    *chunk_rows = cr;
    return true;
}

template <int CW, bool MOM>
void launch_seq(cudaStream_t st, const MemHeadsArgs& a, int T, size_t smem, unsigned grid) {
    if (a.wait_limit != 0 || a.fault_chunk_plus1 != 0) {
        cudaFuncSetAttribute(mem_heads_seq_kernel<CW, MOM, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(mem_heads_seq_kernel<CW, MOM, true>, dim3(grid), dim3(THREADS), smem, st, a, T);
        return;
    }
    cudaFuncSetAttribute(mem_heads_seq_kernel<CW, MOM, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_k(mem_heads_seq_kernel<CW, MOM, false>, dim3(grid), dim3(THREADS), smem, st, a, T);
}

void launch_mem_heads_seq(cudaStream_t st, const MemHeadsArgs& a, int T) {
    const bool mom = a.s != nullptr;
    const size_t smem = smem_bytes_seq(a.hs, a.cw, mom);
    const unsigned grid = (unsigned)((size_t)a.M * a.nh * (a.hs / a.cw));
    if (a.cw == 32) {
        if (mom) launch_seq<32, true>(st, a, T, smem, grid); else launch_seq<32, false>(st, a, T, smem, grid);
    } else {
        if (mom) launch_seq<16, true>(st, a, T, smem, grid); else launch_seq<16, false>(st, a, T, smem, grid);
    }
}

// natural [heads_total][hs][hs] <-> slice-major [heads_total][hs / cw][hs][cw]
__global__ void retile_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t heads, int hs, int cw, int to_slices) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // index in the natural layout
    if (i >= heads * hs * hs) return;
    const int b = (int)(i % hs), a = (int)((i / hs) % hs);
    const int64_t h = i / ((int64_t)hs * hs);
    const int64_t j = (h * (hs / cw) + b / cw) * (int64_t)hs * cw + (int64_t)a * cw + b % cw;
    if (to_slices)
        dst[j] = src[i];
    else
        dst[i] = src[j];
}

void launch_retile(cudaStream_t st, const float* src, float* dst, int64_t heads, int hs, int cw, int to_slices) {
    const int64_t n = heads * hs * hs;
    launch_k(retile_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, src, dst, heads, hs, cw, to_slices);
}

}  // namespace ava

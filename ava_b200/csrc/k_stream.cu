// The fast-weight memory's update + read for one token as ONE streaming pass over the state (sm_100a).
//
// `head_rows` (design-tests/nn/gpu/src/model/fstep/arch.rs:256-337, without momentum) reads the whole head twice: the
// column sums rr = e^T F and t1 = (q alpha)^T F need every row before any row can be updated with rr.  Kept resident in
// shared memory between the two passes (k_delta.cu) that costs 96 KB per block and two block-wide phases.  This kernel
// instead DEFERS a token's update to the next token's pass: the state in HBM after token t holds F as token t found it,
// together with what token t would have written (its alpha, w, ah per row and its value and rr per column, 5 vectors of
// the model width per block and row of the batch, kept in the carried state).  The pass for token t + 1 then does, row
// by row as the rows stream by,
//     f  = (f * alpha_t[row] + w_t[row] v_t[col]) - ah_t[row] rr_t[col]      token t's update, the same three roundings
//     store f                                                                   (the state is written once per token)
//     rr += f * e[row],   t1 += f * (q alpha)[row]                              token t + 1's ordered column sums
// and ends with token t + 1's read y = (t1 + (q.w) v) - (q.ah) rr.  Every element goes through exactly the operations
// of the two-pass form in the same order, so the bits are the same; the traffic is the same one read and one write of
// the state per token; what changes is that nothing has to stay resident: a lane owns four columns, takes its rows
// straight from HBM into registers sixteen rows ahead (coalesced 128-bit loads, 512 contiguous bytes per warp and
// row), and writes them straight back.  No shared-memory tile, no bulk copies, no barriers to wait on, eight
// independent chains per lane to cover the multiply-add latency, and an SM keeps most of its shared memory, registers
// and issue slots for whatever else runs beside it.  A state that is read by anything else (export, select, a chunked
// prompt pass, a save) is first brought up to date by `launch_mem_flush`, which applies the pending update alone.
#include <algorithm>
#include <cstdlib>

#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {


// loads through the default path, stores that stay out of L1 (st.global.cg): measured best of the pairings of cache
// hints tried (0.92 of the copy bandwidth against 0.86 with streaming hints on both)
__device__ __forceinline__ float4 ldg_stream(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void stg_stream(float* p, float4 v) { __stcg(reinterpret_cast<float4*>(p), v); }

__device__ __forceinline__ float4 pending_update(float4 f, float x, float w, float ah, float4 pv, float4 prr) {
    f.x = sub(add(mul(f.x, x), mul(w, pv.x)), mul(ah, prr.x));
    f.y = sub(add(mul(f.y, x), mul(w, pv.y)), mul(ah, prr.y));
    f.z = sub(add(mul(f.z, x), mul(w, pv.z)), mul(ah, prr.z));
    f.w = sub(add(mul(f.w, x), mul(w, pv.w)), mul(ah, prr.w));
    return f;
}

// One block per (row of the batch, head, part of the head's columns); a warp owns 128 columns, a lane four of them.
// Shared memory: e, q*alpha and (PEND) the pending alpha, w, ah of the head, [hs] each.  Small blocks on purpose: every
// warp of the launch is resident from the start (registers are the limit, and they hold the rows in flight), so all
// slices stream side by side at the pace of HBM and end together, whatever the count of (row, head) pairs against SMs.
// SD: rows a lane keeps in flight (16, or 32 when the launch has too few warps to keep HBM busy with 16)
// ALT: the updated state goes to a.f_out (a state that commits at the end) instead of back in place
template <bool PEND, int SD, bool ALT = false>
__global__ void __launch_bounds__(256) mem_stream_kernel(const MemStreamArgs a) {
    pdl_enter();
    extern __shared__ __align__(16) float vs[];
    const int hs = a.hs, cw = a.cw;
    float* ve = vs;
    float* vqg = ve + hs;
    float* vpx = vqg + hs;
    float* vpw = vpx + (PEND ? hs : 0);
    float* vpa = vpw + (PEND ? hs : 0);
    const int parts = a.parts, part = blockIdx.x % parts;
    const int head = (blockIdx.x / parts) % a.nh, m = blockIdx.x / (parts * a.nh);
    const size_t vo = ((size_t)m * a.nh + head) * hs;
    for (int i = threadIdx.x * 4; i < hs; i += blockDim.x * 4) {
        // the five loads before the first store (the compiler cannot move a load above a store it cannot tell apart,
        // and five latencies one after another at the start of every block are not nothing)
        const float4 le = *reinterpret_cast<const float4*>(a.e + vo + i), lq = *reinterpret_cast<const float4*>(a.qg + vo + i);
        float4 lx = le, lw = le, la = le;
        if (PEND) {
            lx = *reinterpret_cast<const float4*>(a.px + vo + i);
            lw = *reinterpret_cast<const float4*>(a.pw + vo + i);
            la = *reinterpret_cast<const float4*>(a.pah + vo + i);
        }
        *reinterpret_cast<float4*>(ve + i) = le;
        *reinterpret_cast<float4*>(vqg + i) = lq;
        if (PEND) {
            *reinterpret_cast<float4*>(vpx + i) = lx;
            *reinterpret_cast<float4*>(vpw + i) = lw;
            *reinterpret_cast<float4*>(vpa + i) = la;
        }
    }
    __syncthreads();
    const int c = part * (int)blockDim.x * 4 + (threadIdx.x >> 5) * 128 + (threadIdx.x & 31) * 4;  // first of this lane's four columns
    if (c >= hs) return;
    // slice-major state: [slice][row][cw]; four neighbouring columns lie in one slice
    const size_t fo = vo * hs + (size_t)(c / cw) * hs * cw + (c % cw);
    float* fp = a.f + fo;
    float* fq = ALT ? a.f_out + fo : fp;   // where the updated state goes: in place, or the state's second copy
    float4 pv = make_float4(0.f, 0.f, 0.f, 0.f), prr = pv;
    if (PEND) {
        pv = *reinterpret_cast<const float4*>(a.pv + vo + c);
        prr = *reinterpret_cast<const float4*>(a.prr + vo + c);
    }
    // the chains start from -0: fma(f, e, -0) is the rounded product with its own sign, i.e. row 0's plain product
    float4 r = make_float4(-0.0f, -0.0f, -0.0f, -0.0f), t = r;
    float4 buf[SD];
#pragma unroll
    for (int i = 0; i < SD; ++i) buf[i] = ldg_stream(fp + (size_t)i * cw);
    for (int row = 0; row < hs; row += SD) {
        float* rp = fp + (size_t)row * cw;
        float* wp = fq + (size_t)row * cw;
#pragma unroll
        for (int i4 = 0; i4 < SD; i4 += 4) {
            const float4 e4 = *reinterpret_cast<const float4*>(ve + row + i4), g4 = *reinterpret_cast<const float4*>(vqg + row + i4);
            float4 x4 = e4, w4 = e4, h4 = e4;
            if (PEND) {
                x4 = *reinterpret_cast<const float4*>(vpx + row + i4);
                w4 = *reinterpret_cast<const float4*>(vpw + row + i4);
                h4 = *reinterpret_cast<const float4*>(vpa + row + i4);
            }
            const float ee[4] = {e4.x, e4.y, e4.z, e4.w}, gg[4] = {g4.x, g4.y, g4.z, g4.w};
            const float xx[4] = {x4.x, x4.y, x4.z, x4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w}, hh[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i4 + j;
                float4 f = buf[i];
                if (row + SD < hs) buf[i] = ldg_stream(rp + (size_t)(SD + i) * cw);  // the row sixteen ahead takes the freed register
                if (PEND) {
                    f = pending_update(f, xx[j], ww[j], hh[j], pv, prr);
                    stg_stream(wp + (size_t)i * cw, f);
                }
                r.x = fma(f.x, ee[j], r.x); r.y = fma(f.y, ee[j], r.y); r.z = fma(f.z, ee[j], r.z); r.w = fma(f.w, ee[j], r.w);
                t.x = fma(f.x, gg[j], t.x); t.y = fma(f.y, gg[j], t.y); t.z = fma(f.z, gg[j], t.z); t.w = fma(f.w, gg[j], t.w);
            }
        }
    }
    // this token's read; its rr stays behind (with its alpha, w, ah and values) as the update the next pass applies
    const float4 v = *reinterpret_cast<const float4*>(a.v + vo + c);
    const float qw = a.qw[(size_t)m * a.nh + head], qa = a.qa[(size_t)m * a.nh + head];
    // the recall's term from inside the one-token chunk is an exact zero (arch.rs:277-280): kept for the sign of zero
    float4 rr;
    rr.x = add(r.x, mul(1.0f, mul(0.0f, v.x))); rr.y = add(r.y, mul(1.0f, mul(0.0f, v.y)));
    rr.z = add(r.z, mul(1.0f, mul(0.0f, v.z))); rr.w = add(r.w, mul(1.0f, mul(0.0f, v.w)));
    float4 y;
    y.x = sub(add(t.x, mul(qw, v.x)), mul(qa, rr.x)); y.y = sub(add(t.y, mul(qw, v.y)), mul(qa, rr.y));
    y.z = sub(add(t.z, mul(qw, v.z)), mul(qa, rr.z)); y.w = sub(add(t.w, mul(qw, v.w)), mul(qa, rr.w));
    *reinterpret_cast<float4*>(a.y + vo + c) = y;
    *reinterpret_cast<float4*>(a.rr_out + vo + c) = rr;
}

// The same pass for a FEW sequences (one talking, or a handful): the streaming kernel above keeps a lane's rows in
// registers, which needs thousands of warps to keep HBM busy; with one sequence it has a few warps and a lane waits a
// memory latency per 32 rows of its 768.  Here a block owns a strip of eight columns of one head: all its threads bring
// the strip [hs][8] into shared memory at once (one latency), all of them apply the pending update element by element
// (the same three roundings) and write the state back, and then sixteen lanes run the sixteen ordered column sums
// (eight columns times rr and t1) over the rows from shared memory, one multiply-add per row each.  Same operations
// per element in the same order, so the same bits.
constexpr int MS_COLS = 8, MS_THREADS = 256;

template <bool PEND, bool ALT>
__global__ void __launch_bounds__(MS_THREADS) mem_stream_small_kernel(const MemStreamArgs a) {
    extern __shared__ __align__(16) float ss[];
    const int hs = a.hs, cw = a.cw;
    float* fs = ss;                       // [hs][8]
    float* ve = fs + (size_t)hs * MS_COLS;
    float* vqg = ve + hs;
    float* vpx = vqg + hs;
    float* vpw = vpx + (PEND ? hs : 0);
    float* vpa = vpw + (PEND ? hs : 0);
    const int strips = hs / MS_COLS, strip = blockIdx.x % strips;
    const int head = (blockIdx.x / strips) % a.nh, m = blockIdx.x / (strips * a.nh);
    const size_t vo = ((size_t)m * a.nh + head) * hs;
    const int c = strip * MS_COLS;
    const size_t fo = vo * hs + (size_t)(c / cw) * hs * cw + (c % cw);   // slice-major: row r of the strip at fo + r * cw
    const float* fp = a.f + fo;
    float* fq = ALT ? a.f_out + fo : a.f + fo;
    const int tid = threadIdx.x;
    // In a decode step the state was last written a whole step ago (by this block's pass of the token before), and the
    // kernel just before this one does not touch it: the strip is then requested before the wait for that kernel.
    if (!a.early_state) pdl_enter();
    for (int i = tid; i < hs * 2; i += MS_THREADS) {
        const int r = i >> 1, q = i & 1;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(fs + (size_t)r * MS_COLS + q * 4)),
                     "l"(fp + (size_t)r * cw + q * 4)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (a.early_state) pdl_enter();
    for (int i = tid * 4; i < hs; i += MS_THREADS * 4) {
        // the five loads before the first store
        const float4 le = *reinterpret_cast<const float4*>(a.e + vo + i), lq = *reinterpret_cast<const float4*>(a.qg + vo + i);
        float4 lx = le, lw = le, la = le;
        if (PEND) {
            lx = *reinterpret_cast<const float4*>(a.px + vo + i);
            lw = *reinterpret_cast<const float4*>(a.pw + vo + i);
            la = *reinterpret_cast<const float4*>(a.pah + vo + i);
        }
        *reinterpret_cast<float4*>(ve + i) = le;
        *reinterpret_cast<float4*>(vqg + i) = lq;
        if (PEND) {
            *reinterpret_cast<float4*>(vpx + i) = lx;
            *reinterpret_cast<float4*>(vpw + i) = lw;
            *reinterpret_cast<float4*>(vpa + i) = la;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (PEND) {
        // every thread the same half row (four columns) of every 128th row: its value and rr columns stay in registers
        const int q = tid & 1;
        const float4 pv = *reinterpret_cast<const float4*>(a.pv + vo + c + q * 4), prr = *reinterpret_cast<const float4*>(a.prr + vo + c + q * 4);
        for (int r = tid >> 1; r < hs; r += MS_THREADS / 2) {
            float4* sp = reinterpret_cast<float4*>(fs + (size_t)r * MS_COLS + q * 4);
            const float4 f = pending_update(*sp, vpx[r], vpw[r], vpa[r], pv, prr);
            *sp = f;
            stg_stream(fq + (size_t)r * cw + q * 4, f);
        }
        __syncthreads();
    }
    if (tid >= 2 * MS_COLS) return;
    // lane j < 8: rr of column j (the rows times e); lane 8 + j: t1 of column j (the rows times q alpha)
    const int j = tid & (MS_COLS - 1);
    const float* vec = tid < MS_COLS ? ve : vqg;
    // what the read's tail takes from global memory is requested before the chains
    const float v = a.v[vo + c + j];
    const float qw = a.qw[(size_t)m * a.nh + head], qa = a.qa[(size_t)m * a.nh + head];
    // the chains start from -0: fma(f, e, -0) is the rounded product with its own sign, i.e. row 0's plain product
    float sum = -0.0f;
    const float* col = fs + j;
#pragma unroll 8
    for (int r = 0; r < hs; ++r) sum = fma(col[(size_t)r * MS_COLS], vec[r], sum);
    const float t1 = __shfl_down_sync(0x0000ffffu, sum, MS_COLS, 16);
    if (tid >= MS_COLS) return;
    // the recall's term from inside the one-token chunk is an exact zero (arch.rs:277-280): kept for the sign of zero
    const float rr = add(sum, mul(1.0f, mul(0.0f, v)));
    a.y[vo + c + j] = sub(add(t1, mul(qw, v)), mul(qa, rr));
    a.rr_out[vo + c + j] = rr;
}

// The pending update alone: f = (f * alpha[row] + w[row] v[col]) - ah[row] rr[col] over the whole slice-major state of
// one block of the model.  One thread per four neighbouring columns of a row.
__global__ void mem_flush_kernel(float* f, const float* __restrict__ px, const float* __restrict__ pw, const float* __restrict__ pah,
                                 const float* __restrict__ pv, const float* __restrict__ prr, int64_t heads, int hs, int cw) {
    pdl_enter();
    const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // index of a group of four columns, in slice-major order
    const int64_t per_head = (int64_t)hs * hs / 4;
    if (q >= heads * per_head) return;
    const int64_t h = q / per_head, w = q % per_head;
    const int cq = cw / 4;
    const int slice = (int)(w / ((int64_t)hs * cq)), row = (int)((w / cq) % hs), c = slice * cw + (int)(w % cq) * 4;
    float4* p = reinterpret_cast<float4*>(f) + q;
    const float4 v = *reinterpret_cast<const float4*>(pv + h * hs + c), rr = *reinterpret_cast<const float4*>(prr + h * hs + c);
    *p = pending_update(*p, px[h * hs + row], pw[h * hs + row], pah[h * hs + row], v, rr);
}

}  // namespace

long g_mem_stream_small_max = 8 * 768;  // up to this many (sequence, head, row) triples the strip kernel takes the pass

// false: head size not covered (a multiple of 16; the head's five vectors must fit shared memory)
bool launch_mem_stream(cudaStream_t st, const MemStreamArgs& a) {
    const bool pend = a.px != nullptr;
    // a few sequences: strips of eight columns staged in shared memory (the register-streaming kernel would have a handful of warps)
    if ((long)a.M * a.nh * a.hs <= g_mem_stream_small_max && a.hs % 16 == 0 && a.cw % MS_COLS == 0) {
        const size_t sm = (size_t)(MS_COLS + (pend ? 5 : 2)) * a.hs * sizeof(float);
        if (sm <= 200 * 1024) {
            const unsigned grid = (unsigned)((size_t)a.M * a.nh * (a.hs / MS_COLS));
            auto go = [&](auto kernel) {
                if (sm > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
                launch_k(kernel, dim3(grid), dim3(MS_THREADS), sm, st, a);
            };
            if (!pend) go(mem_stream_small_kernel<false, false>);
            else if (a.f_out) go(mem_stream_small_kernel<true, true>);
            else go(mem_stream_small_kernel<true, false>);
            return true;
        }
    }
    const size_t smem = (size_t)(pend ? 5 : 2) * a.hs * sizeof(float);
    const int wpb = 2;  // warps per block: small blocks, so that every warp of the launch is resident from the start
    const int warps_head = (a.hs + 127) / 128, warps = std::min(wpb, warps_head);
    if (a.hs % 16 || a.cw % 4 || smem > 64 * 1024) return false;
    MemStreamArgs b = a;
    b.parts = (warps_head + warps - 1) / warps;
    const unsigned grid = (unsigned)((size_t)a.M * a.nh * b.parts);
    auto go = [&](auto kernel) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_k(kernel, dim3(grid), dim3(warps * 32), smem, st, b);
    };
    // rows in flight per lane: sixteen, or thirty-two when the launch has too few warps to keep HBM busy with sixteen (about 10 MB
    // in flight over the whole GPU are needed)
    const int deep_below = 1200;  // warps
    const bool deep = (long)a.M * a.nh * warps_head < deep_below;
    if (!pend) { go(mem_stream_kernel<false, 16>); return true; }
    if (a.f_out) {
        if (deep) go(mem_stream_kernel<true, 32, true>); else go(mem_stream_kernel<true, 16, true>);
        return true;
    }
    if (deep) go(mem_stream_kernel<true, 32>); else go(mem_stream_kernel<true, 16>);
    return true;
}

void launch_mem_flush(cudaStream_t st, float* f, const float* px, const float* pw, const float* pah, const float* pv, const float* prr, int64_t heads,
                      int hs, int cw) {
    const int64_t n = heads * hs * hs / 4;
    launch_k(mem_flush_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, f, px, pw, pah, pv, prr, heads, hs, cw);
}

}  // namespace ava

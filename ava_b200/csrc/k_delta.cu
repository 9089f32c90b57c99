// The fast-weight memory's update + read for one token (sm_100a): the kernel that streams the carried state.
//
// Per head, F [hs, hs] f32 (row = key dimension, column = value dimension), as the reference's `head_rows`
// (design-tests/nn/gpu/src/model/fstep/arch.rs:256-337) without momentum:
//     rr  = e^T F                      (each column summed over the rows in order: row 0's product, then fma)
//     t1  = (q alpha)^T F
//     y   = (t1 + (q.w) v) - (q.ah) rr
//     F'  = (F * alpha_row + w v^T) - ah rr^T
// Columns are independent, so one block of threads owns a slice of CW columns of one head: the [hs, CW] slice is
// brought into shared memory once by TMA (2-D tiled bulk copies, one mbarrier per box of rows), the column sums run
// down the rows as the boxes land, the slice is updated in place in shared memory and written back once by TMA.  Per
// token the state is read once and written once: 8 bytes per state element, the kernel's whole DRAM traffic apart
// from the per-head vectors.
#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int MAX_BOXES = 8;
constexpr int THREADS = 256;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // polls (each backs off ~64 ns) before a wait gives up: about a quarter second

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
        if (i > 64) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y), "r"(smem_u32(src))
                 : "memory");
}

// One block: row m, head e, columns [c0, c0 + CW).  Shared memory: the slice [hs][CW], then e, qg, ex, w, ah [hs]
// each, then v, rr, t1 [CW] each, then the barriers.
template <int CW>
__global__ void __launch_bounds__(THREADS) mem_heads_kernel(const __grid_constant__ MemHeadsArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int hs = a.hs, rb = a.rb, nbox = hs / rb;
    float* tile = reinterpret_cast<float*>(smem_raw);
    float* ve = tile + (size_t)hs * CW;
    float* vqg = ve + hs;
    float* vex = vqg + hs;
    float* vw = vex + hs;
    float* vah = vw + hs;
    float* vv = vah + hs;
    float* rr = vv + CW;
    float* t1 = rr + CW;
    uint64_t* bars = reinterpret_cast<uint64_t*>(t1 + CW);

    const int tid = threadIdx.x;
    const int slices = hs / CW;
    const int slice = blockIdx.x % slices;
    const int head = (blockIdx.x / slices) % a.nh;
    const int m = blockIdx.x / (slices * a.nh);
    const int c0 = slice * CW;
    const int64_t trow = a.row0 + ((int64_t)m * a.nh + head) * hs;  // first tensor row of this head
    const size_t vo = ((size_t)m * a.nh + head) * hs;                // offset of this head's vectors

    if (tid == 0) {
        for (int b = 0; b < nbox; ++b) mbar_init(&bars[b], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
        for (int b = 0; b < nbox; ++b) {
            mbar_expect_tx(&bars[b], (uint32_t)(rb * CW * sizeof(float)));
            tma_load_2d(tile + (size_t)b * rb * CW, &a.tmap, c0, (int)(trow + (int64_t)b * rb), &bars[b]);
        }
    }
    for (int i = tid; i < hs; i += THREADS) {
        ve[i] = a.e[vo + i];
        vqg[i] = a.qg[vo + i];
        vex[i] = a.ex[vo + i];
        vw[i] = a.w[vo + i];
        vah[i] = a.ah[vo + i];
    }
    if (tid < CW) vv[tid] = a.v[vo + c0 + tid];
    __syncthreads();

    // pass 1: the column sums, rows in order as their boxes land (the first CW threads, one column each)
    bool ok = true;
    if (tid < CW) {
        float r = 0.0f, t = 0.0f;
        for (int b = 0; b < nbox; ++b) {
            ok = ok && mbar_wait(&bars[b], 0);
            const float* p = tile + (size_t)b * rb * CW + tid;
            int row = b * rb;
            if (b == 0) {
                const float f = p[0];
                r = mul(f, ve[0]);
                t = mul(f, vqg[0]);
                p += CW;
                row = 1;
            }
#pragma unroll 8
            for (; row < (b + 1) * rb; ++row, p += CW) {
                const float f = *p;
                r = fma(f, ve[row], r);
                t = fma(f, vqg[row], t);
            }
        }
        // the recall's term from inside the one-token chunk is an exact zero (arch.rs:277-280): kept for the sign of zero
        r = add(r, mul(1.0f, mul(0.0f, vv[tid])));
        rr[tid] = r;
        t1[tid] = t;
    }
    if (!ok) atomicOr(a.status, ST_WAIT_TIMEOUT);
    __syncthreads();
    // every thread must see the boxes' bytes: a wait that succeeded makes them visible to its thread only
    bool ok2 = true;
    if (tid >= CW)
        for (int b = 0; b < nbox; ++b) ok2 = ok2 && mbar_wait(&bars[b], 0);
    if (!ok2) atomicOr(a.status, ST_WAIT_TIMEOUT);

    // the read
    if (tid < CW) {
        const float qw = a.qw[(size_t)m * a.nh + head], qa = a.qa[(size_t)m * a.nh + head];
        a.y[vo + c0 + tid] = sub(add(t1[tid], mul(qw, vv[tid])), mul(qa, rr[tid]));
    }
    // pass 2: the update, in place; thread -> (row group, column) so that a warp covers whole rows
    {
        const int col = tid % CW, rg = tid / CW, rgs = THREADS / CW;
        const float vb = vv[col], rb_ = rr[col];
        for (int row = rg; row < hs; row += rgs) {
            float* p = tile + (size_t)row * CW + col;
            *p = sub(add(mul(*p, vex[row]), mul(vw[row], vb)), mul(vah[row], rb_));
        }
    }
    // make the generic-proxy writes visible to the TMA engine, then write the slice back
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        for (int b = 0; b < nbox; ++b) tma_store_2d(&a.tmap, c0, (int)(trow + (int64_t)b * rb), tile + (size_t)b * rb * CW);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        // the shared memory must stay until the engine has read it
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
}

size_t smem_bytes(int hs, int cw) { return ((size_t)hs * cw + 5 * (size_t)hs + 3 * (size_t)cw) * sizeof(float) + MAX_BOXES * sizeof(uint64_t); }

}  // namespace

bool mem_heads_tiling(int hs, int* cw, int* rb) {
    // rows per TMA box: at most 256; the head's rows must be whole boxes, at most MAX_BOXES of them
    int r = hs <= 256 ? hs : 256;
    if (hs % r != 0 || hs / r > MAX_BOXES) return false;
    // the widest slice (128-byte rows) that leaves room for two blocks per SM, else 64-byte rows
    int w = 32;
    if (hs % w != 0 || smem_bytes(hs, w) > 113 * 1024) w = 16;
    if (hs % w != 0 || smem_bytes(hs, w) > 227 * 1024) return false;
    *cw = w;
    *rb = r;
    return true;
}

void launch_mem_heads(cudaStream_t st, const MemHeadsArgs& a) {
    const size_t smem = smem_bytes(a.hs, a.cw);
    const unsigned grid = (unsigned)((size_t)a.M * a.nh * (a.hs / a.cw));
    if (a.cw == 32) {
        cudaFuncSetAttribute(mem_heads_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mem_heads_kernel<32><<<grid, THREADS, smem, st>>>(a);
    } else {
        cudaFuncSetAttribute(mem_heads_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mem_heads_kernel<16><<<grid, THREADS, smem, st>>>(a);
    }
}

}  // namespace ava

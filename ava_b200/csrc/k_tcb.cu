// Batched f32-accurate products on the tensor cores (sm_100a: TMA + tcgen05.mma + tensor memory) for the chunk-parallel
// form of the fast-weight memory (k_chunk.cu).
//
//   C[b] (M x N, f32) = A[b] (M x K) . B[b]^T (N x K)          b = 0 .. batch - 1
//
// Both operands are f32 values carried as bf16 LIMBS (hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid): their
// sum is x exactly, and a bf16 x bf16 product is exact in f32), stored K-major as planes [limb][batch * rows][K].  The
// kernel issues the limb products A_i . B_j with i + j below the larger limb count (six for three limbs each: hi.hi,
// hi.mid, mid.hi, hi.lo, mid.mid, lo.hi), all into one f32 accumulator in tensor memory, so the result carries the
// operands to about 2^-24 each: an f32 product with the tensor core's summation order.
//
// One block of 256 threads per 128 x BN tile of one batch item; k-tiles of 64 in a ring of stages.  Thread 0 brings the
// limb tiles in by TMA (2-D tiled, 128-byte swizzle; every block fetches its own tiles), thread 32 issues the multiply-adds and
// commits each stage's "empty" barrier, all eight warps read the accumulator back (tcgen05.ld) for the epilogue:
//   TCB_STORE   C = acc
//   TCB_SCALE_ADD  C = C + acc * colscale[b][n]: the int8-weight product of integer-valued rows (spikes), one limb each side:
//               every product and every partial sum is an integer below 2^24, so the accumulator is exact whatever the
//               order, and the result is the ordered sum's bits
//   TCB_DECAY   C = colscale[b][n] * C + acc, and the three limbs of the new C written beside it (the state update of the
//               chunked memory: the next step multiplies by this state, so its limbs are made where it is produced)
// Every wait is bounded; a wait that runs out sets ST_WAIT_TIMEOUT and the tile is not written.
#include <cuda.h>
#include <cuda_runtime.h>

#include "ava_math.h"
#include "bf16_hw.cuh"
#include "kernels.cuh"
#include "tc_common.cuh"

namespace ava {

namespace {

using namespace tcc;
constexpr int B_THREADS = 256;
template <int BN, int LA, int LB, int STAGES, int EPI>
__global__ void __launch_bounds__(B_THREADS) tc_bgemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                             const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                                                             const TcbArgs a) {
    pdl_enter();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (s32(smem_raw) & 1023u)) & 1023u);  // swizzled tiles want a 1024-byte boundary
    constexpr uint32_t A_BYTES = B_BM * B_BK * 2, B_BYTES = BN * B_BK * 2, STAGE_BYTES = LA * A_BYTES + LB * B_BYTES;
    constexpr int PMAX = (LA > LB ? LA : LB) - 1;  // limb products A_i . B_j with i + j <= PMAX
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accbar = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accbar + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * B_BM, n0 = blockIdx.x * BN, bz = blockIdx.z;
    const int kt1 = a.K / B_BK, kt = kt1 + a.K2 / B_BK;   // k-tiles of the operands proper, then of the second stretch

    if (EPI == TCB_DECAY || EPI == TCB_SCALE_ADD) {
        // the tile of the old C is wanted by the epilogue only: ask for it now, so that it waits in L2 by then
        const float* ctile = a.C + (size_t)bz * a.c_batch_stride + (size_t)m0 * a.ldc + n0;
        for (int n = tid; n < B_BM * (BN / 32); n += B_THREADS) {
            const int r = n / (BN / 32), c = (n % (BN / 32)) * 32;
            if (m0 + r < a.M && n0 + c < a.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(ctile + (size_t)r * a.ldc + c));
        }
    }
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            bar_init(&full[s], 1);
            bar_init(&empty[s], 1);
        }
        bar_init(accbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (tid == 0) {
        bool ok = true;
        const int ya = (int)a.a_row0 + bz * a.M + m0, yb = (int)a.b_row0 + bz * a.N + n0;
        for (int it = 0; it < kt && ok; ++it) {
            const int s = it % STAGES, n = it / STAGES;
            if (n > 0) ok = bar_wait(&empty[s], (uint32_t)((n - 1) & 1));
            if (!ok) break;
            unsigned char* st = smem + (size_t)s * STAGE_BYTES;
            bar_expect(&full[s], STAGE_BYTES);
            if (it < kt1) {
#pragma unroll
                for (int l = 0; l < LA; ++l) tma_load(st + l * A_BYTES, &map_a, it * B_BK, (int)(l * a.rows_a) + ya, &full[s]);
#pragma unroll
                for (int l = 0; l < LB; ++l) tma_load(st + LA * A_BYTES + l * B_BYTES, &map_b, it * B_BK, (int)(l * a.rows_b) + yb, &full[s]);
            } else {
                const int ya2 = (int)a.a2_row0 + bz * a.M + m0, yb2 = (int)a.b2_row0 + bz * a.N + n0;
#pragma unroll
                for (int l = 0; l < LA; ++l) tma_load(st + l * A_BYTES, &map_a2, (it - kt1) * B_BK, (int)(l * a.rows_a2) + ya2, &full[s]);
#pragma unroll
                for (int l = 0; l < LB; ++l) tma_load(st + LA * A_BYTES + l * B_BYTES, &map_b2, (it - kt1) * B_BK, (int)(l * a.rows_b2) + yb2, &full[s]);
            }
        }
        if (!ok) atomicOr(a.status, ST_WAIT_TIMEOUT);
    } else if (tid == 32) {
        bool ok = true;
        constexpr uint32_t idesc = instr_desc(BN);
        for (int it = 0; it < kt && ok; ++it) {
            const int s = it % STAGES, n = it / STAGES;
            ok = bar_wait(&full[s], (uint32_t)(n & 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* st = smem + (size_t)s * STAGE_BYTES;
            bool first = it == 0;
#pragma unroll
            for (int i = 0; i < LA; ++i)
#pragma unroll
                for (int j = 0; j < LB; ++j) {
                    if (i + j > PMAX) continue;
                    const uint64_t da = operand_desc(st + i * A_BYTES), db = operand_desc(st + LA * A_BYTES + j * B_BYTES);
#pragma unroll
                    for (int k16 = 0; k16 < B_BK / 16; ++k16) {
                        const uint32_t acc = first ? 0u : 1u;  // the very first multiply-add of the tile overwrites the accumulator
                        first = false;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t"
                            "setp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                            ::"r"(tmem), "l"(da + 2u * k16), "l"(db + 2u * k16), "r"(idesc), "r"(acc)
                            : "memory");
                    }
                }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&empty[s])) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(accbar)) : "memory");
        if (!ok) atomicOr(a.status, ST_WAIT_TIMEOUT);
    }
    __syncwarp();
    const bool acc_ok = bar_wait(accbar, 0);
    if (!acc_ok && lane == 0) atomicOr(a.status, ST_WAIT_TIMEOUT);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // epilogue: warp w reads lanes 32 (w % 4) .. + 31 of the accumulator (one output row per thread), 32 columns per
    // instruction; warps 0-3 take the left half of the tile's columns, warps 4-7 the right half.  Each 32 x 32 piece
    // goes through a staging square in shared memory (the operand stage is free once the accumulator is complete) so
    // that global memory is touched row-wise: eight lanes cover 128 contiguous bytes of a row, four rows per instruction.
    const int wq = warp & 3, half = warp >> 2;
    float* stage = reinterpret_cast<float*>(smem) + warp * (32 * 33);
    const int sub_r = lane >> 3, sub_c = (lane & 7) * 4;
    float* cbase = a.C + (size_t)bz * a.c_batch_stride;
#pragma unroll 1
    for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem + ((uint32_t)(wq * 32) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
              "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
              "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int c = n0 + c0 + sub_c;           // this lane's four columns
        const bool col_ok = c < a.N && acc_ok;   // N is a multiple of 4
        float4 prev[8], g = make_float4(0.f, 0.f, 0.f, 0.f);
        if (EPI == TCB_DECAY || EPI == TCB_SCALE_ADD) {  // the old values: asked for before the staging, all eight row groups at once
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int row = m0 + wq * 32 + it * 4 + sub_r;
                prev[it] = (col_ok && row < a.M) ? *reinterpret_cast<const float4*>(cbase + (size_t)row * a.ldc + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (col_ok) g = *reinterpret_cast<const float4*>(a.colscale + (size_t)bz * a.colscale_batch_stride + c);
        }
        __syncwarp();  // the lanes' reads of the piece before
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[lane * 33 + j] = __uint_as_float(r[j]);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int lr = it * 4 + sub_r, row = m0 + wq * 32 + lr;
            if (!col_ok || row >= a.M) continue;
            const float* sp = stage + lr * 33 + sub_c;
            float4 o = make_float4(sp[0], sp[1], sp[2], sp[3]);
            if (EPI == TCB_DECAY) {
                const float4 x = prev[it];
                o = make_float4(add(mul(x.x, g.x), o.x), add(mul(x.y, g.y), o.y), add(mul(x.z, g.z), o.z), add(mul(x.w, g.w), o.w));
            }
            if (EPI == TCB_SCALE_ADD) {  // the int8 product's epilogue: the sum times the column's scale, added to what is there
                const float4 x = prev[it];
                o = make_float4(add(x.x, mul(o.x, g.x)), add(x.y, mul(o.y, g.y)), add(x.z, mul(o.z, g.z)), add(x.w, mul(o.w, g.w)));
            }
            *reinterpret_cast<float4*>(cbase + (size_t)row * a.ldc + c) = o;
            if (EPI == TCB_DECAY) {
                // the new value's three limbs, in the operand layout of the product that reads it next: [limb][batch * M][N]
                const float ov[4] = {o.x, o.y, o.z, o.w};
                uint16_t l0[4], l1[4], l2[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) limbs3_hw(ov[q], l0[q], l1[q], l2[q]);
                const size_t at = ((size_t)bz * a.M + row) * a.N + c;
                *reinterpret_cast<uint2*>(a.c_limbs + at) = make_uint2(l0[0] | ((uint32_t)l0[1] << 16), l0[2] | ((uint32_t)l0[3] << 16));
                *reinterpret_cast<uint2*>(a.c_limbs + a.c_limb_plane + at) = make_uint2(l1[0] | ((uint32_t)l1[1] << 16), l1[2] | ((uint32_t)l1[3] << 16));
                *reinterpret_cast<uint2*>(a.c_limbs + 2 * a.c_limb_plane + at) = make_uint2(l2[0] | ((uint32_t)l2[1] << 16), l2[2] | ((uint32_t)l2[3] << 16));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
}

template <int BN, int LA, int LB, int STAGES, int EPI>
bool launch_one(cudaStream_t st, const TcbArgs& a) {
    CUtensorMap ma, mb, ma2, mb2;
    if (!make_map(&ma, a.a, (uint64_t)LA * a.rows_a, a.K, B_BM) || !make_map(&mb, a.b, (uint64_t)LB * a.rows_b, a.K, BN)) return false;
    if (a.K2 > 0) {
        if (!make_map(&ma2, a.a2, (uint64_t)LA * a.rows_a2, a.lda2, B_BM) || !make_map(&mb2, a.b2, (uint64_t)LB * a.rows_b2, a.ldb2, BN)) return false;
    } else {
        ma2 = ma;
        mb2 = mb;
    }
    const size_t smem = (size_t)STAGES * (LA * B_BM * B_BK * 2 + LB * BN * B_BK * 2) + (2 * STAGES + 1) * sizeof(uint64_t) + 16 + 1024;
    cudaFuncSetAttribute(tc_bgemm_kernel<BN, LA, LB, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    prefer_max_shared(reinterpret_cast<const void*>(tc_bgemm_kernel<BN, LA, LB, STAGES, EPI>), 100);
    dim3 grid((a.N + BN - 1) / BN, (a.M + B_BM - 1) / B_BM, a.batch);
    return launch_k(tc_bgemm_kernel<BN, LA, LB, STAGES, EPI>, grid, dim3(B_THREADS), smem, st, ma, mb, ma2, mb2, a) == cudaSuccess;
}

}  // namespace

// false: shape not covered (K a multiple of 64, M a multiple of 128, N a multiple of 4) or no tensor-map encoder
bool launch_tc_bgemm(cudaStream_t st, const TcbArgs& a, int epi) {
    if (a.K % B_BK || a.K2 % B_BK || a.K2 < 0 || a.M % B_BM || a.N % 4 || a.batch < 1) return false;
    if (a.K2 > 0 && (!a.a2 || !a.b2 || a.lda2 < a.K2 || a.ldb2 < a.K2 || a.lda2 % 8 || a.ldb2 % 8)) return false;
    // N 128: two stages of 96 KB, one block per SM (measured a little ahead of one stage with two blocks per SM)
    if (epi == TCB_SCALE_ADD) {
        // one limb each side (operands exact in bf16: spikes and int8 weights), four stages of 32 KB
        if (a.K2 > 0) return false;
        return a.N % 128 == 0 ? launch_one<128, 1, 1, 4, TCB_SCALE_ADD>(st, a) : launch_one<64, 1, 1, 4, TCB_SCALE_ADD>(st, a);
    }
    if (a.N % 128 == 0 && epi == TCB_DECAY && a.K + a.K2 <= 2 * B_BK) return launch_one<128, 3, 3, 1, TCB_DECAY>(st, a);
    if (a.N % 128 == 0) return epi == TCB_DECAY ? launch_one<128, 3, 3, 2, TCB_DECAY>(st, a) : launch_one<128, 3, 3, 2, TCB_STORE>(st, a);
    return epi == TCB_DECAY ? launch_one<64, 3, 3, 3, TCB_DECAY>(st, a) : launch_one<64, 3, 3, 3, TCB_STORE>(st, a);
}

}  // namespace ava

// Tensor-core form of the dense int8-weight products (sm_100a: TMA + tcgen05.mma + tensor memory), the engine's
// optional "fast products" mode.
//
// The reference sums f32 activations times int8 weights in f32 in k order (design-tests/nn/gpu/src/int8.rs:315-331); a
// tensor core sums in its own order, so this path does not reproduce the reference's bits and is off by default.  What
// it keeps exact is every PRODUCT: an f32 activation is split into three bf16 limbs whose sum is the f32 value exactly
// (hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid)), an int8 weight is exact in bf16, and a bf16 x bf16 product
// is exact in f32.  Only the order (and the rounding) of the f32 additions differs from the reference: the result
// agrees with the ordered sum to about 1e-6 of the sum of magnitudes.
//
//   C[M, N] = (A_hi + A_mid + A_lo)[M, K] . W[K, N] * scale[N]      A limbs bf16 [3][M][K], W as bf16 [N][K] (K-major)
//
// One block of 256 threads per 128 x BN output tile, a 3-stage ring of k-tiles.  Thread 0 is the producer: per k-tile
// TMA (2-D tiled, 128-byte swizzle) brings the 128 x 64 tiles of the three A limbs and one BN x 64 tile of W into
// shared memory and signals the stage's "full" mbarrier.  Thread 32 issues the multiply-adds: twelve tcgen05.mma per
// stage (three limbs x four steps of K 16; M 128, N BN, bf16 in, f32 accumulate in tensor memory), then tcgen05.commit
// on the stage's "empty" mbarrier, which the producer waits on before it refills the stage.  After the last commit all
// eight warps read the accumulator back (tcgen05.ld, 32 lanes x 32 columns per warp and instruction), scale it and
// store or add it, row-wise through a staging square in shared memory.  Every wait is bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include "ava_math.h"
#include "kernels.cuh"

namespace ava {

namespace {

constexpr int TC_BM = 128, TC_BK = 64, TC_STAGES = 3, TC_THREADS = 256;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = s32(bar);
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (i > 1024) __nanosleep(32);
    }
    return false;
}
__device__ __forceinline__ void tma_load(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(s32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(s32(bar))
                 : "memory");
}

// Shared-memory operand descriptor of a K-major tile of 64 bf16 (128 bytes) per row, rows 128 bytes apart, 128-byte
// swizzle: start address / 16, stride between 8-row groups 1024 bytes / 16, descriptor version 1 (sm_100), layout 2.
__device__ __forceinline__ uint64_t operand_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((s32(tile) & 0x3FFFFu) >> 4);   // bits [0, 14)
    d |= (uint64_t)(1024u >> 4) << 32;              // stride byte offset, bits [32, 46)
    d |= (uint64_t)1 << 46;                         // version
    d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
    return d;
}

// kind::f16 instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, M 128, N n
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

template <int BN, int EPI>
__global__ void __launch_bounds__(TC_THREADS) tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                                                             const float* __restrict__ scale, float* C, int ldc, int M, int N, int K,
                                                             uint32_t* status) {
    pdl_enter();
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles want a 1024-byte boundary, which the dynamic shared-memory base does not promise
    unsigned char* smem = smem_raw + ((1024u - (s32(smem_raw) & 1023u)) & 1023u);
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2, W_BYTES = BN * TC_BK * 2, STAGE_BYTES = 3 * A_BYTES + W_BYTES;
    // stage s: the three limb tiles [3][128][64] bf16, then the weight tile [BN][64] bf16
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + TC_STAGES * STAGE_BYTES);
    uint64_t* empty = full + TC_STAGES;
    uint64_t* accbar = empty + TC_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accbar + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * BN;
    const int kt = K / TC_BK;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            bar_init(&full[s], 1);
            bar_init(&empty[s], 1);
        }
        bar_init(accbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {  // tensor memory for the accumulator: BN columns of 128 lanes x 32 bits
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"((uint32_t)BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    if (EPI == EPI_ADD) {
        // the tile the products are added to is wanted by the epilogue only: ask for it now, so that it waits in L2 by then
        for (int n = tid; n < TC_BM * (BN / 32); n += TC_THREADS) {
            const int r = n / (BN / 32), c = (n % (BN / 32)) * 32;
            if (m0 + r < M && n0 + c < N) asm volatile("prefetch.global.L2 [%0];" ::"l"(C + (size_t)(m0 + r) * ldc + n0 + c));
        }
    }

    if (tid == 0) {
        // producer: one k-tile per stage, the weight tile shared by the three limbs
        bool ok = true;
        for (int it = 0; it < kt && ok; ++it) {
            const int s = it % TC_STAGES, n = it / TC_STAGES;
            if (n > 0) ok = bar_wait(&empty[s], (uint32_t)((n - 1) & 1));
            if (!ok) break;
            unsigned char* st = smem + (size_t)s * STAGE_BYTES;
            bar_expect(&full[s], STAGE_BYTES);
#pragma unroll
            for (int l = 0; l < 3; ++l) tma_load(st + l * A_BYTES, &map_a, it * TC_BK, l * M + m0, &full[s]);
            tma_load(st + 3 * A_BYTES, &map_w, it * TC_BK, n0, &full[s]);
        }
        if (!ok) atomicOr(status, ST_WAIT_TIMEOUT);
    } else if (tid == 32) {
        // issuer of the multiply-adds
        bool ok = true;
        constexpr uint32_t idesc = instr_desc(BN);
        for (int it = 0; it < kt && ok; ++it) {
            const int s = it % TC_STAGES, n = it / TC_STAGES;
            ok = bar_wait(&full[s], (uint32_t)(n & 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* st = smem + (size_t)s * STAGE_BYTES;
            const uint64_t dw = operand_desc(st + 3 * A_BYTES);
#pragma unroll
            for (int l = 0; l < 3; ++l) {
                const uint64_t da = operand_desc(st + l * A_BYTES);
#pragma unroll
                for (int k16 = 0; k16 < TC_BK / 16; ++k16) {
                    // 16 bf16 further along K inside the 128-byte swizzled row: 32 bytes = 2 in descriptor units
                    const uint32_t acc = (it > 0 || l > 0 || k16 > 0) ? 1u : 0u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem), "l"(da + 2u * k16), "l"(dw + 2u * k16), "r"(idesc), "r"(acc)
                        : "memory");
                }
            }
            // the stage is free again when these multiply-adds have read it
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&empty[s])) : "memory");
        }
        // the accumulator is complete when every multiply-add issued so far is
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(accbar)) : "memory");
        if (!ok) atomicOr(status, ST_WAIT_TIMEOUT);
    }
    __syncwarp();
    const bool acc_ok = bar_wait(accbar, 0);
    if (!acc_ok && lane == 0) atomicOr(status, ST_WAIT_TIMEOUT);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // epilogue: warp w reads lanes 32 (w % 4) .. + 31 of the accumulator (one output row per thread), 32 columns per
    // instruction; warps 0-3 take the left half of the tile's columns, warps 4-7 the right half.  Each 32 x 32 piece
    // goes through a staging square in shared memory (the first stage is free once the accumulator is complete) so
    // that global memory is touched row-wise: eight lanes cover 128 contiguous bytes of a row, four rows per instruction.
    const int wq = warp & 3, half = warp >> 2;
    float* stage = reinterpret_cast<float*>(smem) + warp * (32 * 33);
    const int sub_r = lane >> 3, sub_c = (lane & 7) * 4;
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
        const bool col_ok = c < N && acc_ok;     // N is a multiple of 4
        float4 prev[8], sc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (EPI == EPI_ADD) {  // the values the products are added to: asked for before the staging, all eight row groups at once
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int row = m0 + wq * 32 + it * 4 + sub_r;
                prev[it] = (col_ok && row < M) ? *reinterpret_cast<const float4*>(C + (size_t)row * ldc + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (col_ok) sc = *reinterpret_cast<const float4*>(scale + c);
        __syncwarp();  // the lanes' reads of the piece before
#pragma unroll
        for (int j = 0; j < 32; ++j) stage[lane * 33 + j] = __uint_as_float(r[j]);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int lr = it * 4 + sub_r, row = m0 + wq * 32 + lr;
            if (!col_ok || row >= M) continue;
            const float* sp = stage + lr * 33 + sub_c;
            float4 o = make_float4(mul(sp[0], sc.x), mul(sp[1], sc.y), mul(sp[2], sc.z), mul(sp[3], sc.w));
            if (EPI == EPI_ADD) {
                const float4 x = prev[it];
                o = make_float4(add(x.x, o.x), add(x.y, o.y), add(x.z, o.z), add(x.w, o.w));
            }
            *reinterpret_cast<float4*>(C + (size_t)row * ldc + c) = o;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
}

// x f32 [n] -> three bf16 planes [3][n] whose sum is x exactly
__global__ void split3_kernel(const float* __restrict__ x, int64_t n, uint16_t* __restrict__ out) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    const uint16_t hi = f_to_bf16(v);
    const float r1 = sub(v, bf16_to_f(hi));
    const uint16_t mid = f_to_bf16(r1);
    const float r2 = sub(r1, bf16_to_f(mid));
    out[i] = hi;
    out[n + i] = mid;
    out[2 * n + i] = f_to_bf16(r2);
}

// int8 [K][N] -> bf16 [N][K] (exact)
__global__ void widen_transpose_kernel(const int8_t* __restrict__ q, int K, int N, uint16_t* __restrict__ out) {
    pdl_enter();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)K * N) return;
    const int k = (int)(i % K), n = (int)(i / K);
    out[i] = f_to_bf16((float)q[(size_t)k * N + n]);
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    }
    return fn;
}

// bf16 [rows][cols] row-major, boxes of [64 columns, box_rows rows], 128-byte swizzle, out-of-range filled with zeros
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {TC_BK, box_rows};
    const cuuint32_t es[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
size_t tc_smem() { return (size_t)TC_STAGES * (3 * TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * TC_STAGES + 1) * sizeof(uint64_t) + 16 + 1024; }

template <int BN>
bool launch_bn(cudaStream_t st, const TcGemmArgs& a, GemmEpilogue epi) {
    CUtensorMap ma, mw;
    if (!make_map(&ma, a.a_limbs, (uint64_t)3 * a.M, a.K, TC_BM) || !make_map(&mw, a.w_bf16, a.N, a.K, BN)) return false;
    dim3 grid((a.N + BN - 1) / BN, (a.M + TC_BM - 1) / TC_BM);
    const size_t smem = tc_smem<BN>();
    // the attribute belongs to the function on the current device: set on every launch (a table lookup in the runtime)
    if (epi == EPI_ADD) {
        if (cudaFuncSetAttribute(tc_gemm_kernel<BN, EPI_ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
    } else {
        if (cudaFuncSetAttribute(tc_gemm_kernel<BN, EPI_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
    }
    if (epi == EPI_ADD) {
        launch_k(tc_gemm_kernel<BN, EPI_ADD>, dim3(grid), dim3(TC_THREADS), smem, st, ma, mw, a.scale, a.C, a.ldc, a.M, a.N, a.K, a.status);
    } else {
        launch_k(tc_gemm_kernel<BN, EPI_STORE>, dim3(grid), dim3(TC_THREADS), smem, st, ma, mw, a.scale, a.C, a.ldc, a.M, a.N, a.K, a.status);
    }
    return true;
}

}  // namespace

bool launch_tc_gemm(cudaStream_t st, const TcGemmArgs& a, GemmEpilogue epi) {
    if (a.K % TC_BK != 0 || a.N % 4 != 0 || epi == EPI_LIF) return false;
    // narrower tiles when the product is narrow, so that more SMs take part
    if ((a.N + 127) / 128 * ((a.M + 127) / 128) >= 48) return launch_bn<128>(st, a, epi);
    return launch_bn<64>(st, a, epi);
}

void launch_split3(cudaStream_t st, const float* x, int64_t n, uint16_t* out) {
    launch_k(split3_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, n, out);
}

void launch_widen_transpose(cudaStream_t st, const int8_t* q, int K, int N, uint16_t* out) {
    const int64_t n = (int64_t)K * N;
    launch_k(widen_transpose_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, q, K, N, out);
}

}  // namespace ava

// Helpers shared by the tcgen05 kernels (sm_100a): bounded mbarrier waits, 2-D tiled TMA loads, shared-memory operand
// descriptors for K-major bf16 tiles with the 128-byte swizzle, the kind::f16 instruction descriptor, and the host's
// tensor-map encoder (fetched from the driver at run time, so nothing links against libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace ava {
namespace tcc {

constexpr int B_BM = 128, B_BK = 64;
constexpr uint32_t B_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = s32(bar);
    for (uint32_t i = 0; i < B_WAIT_LIMIT; ++i) {
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
// K-major tile of 64 bf16 (128 bytes) per row, 128-byte swizzle: start address / 16, 1024 bytes between 8-row groups,
// descriptor version 1 (sm_100), layout 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t operand_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((s32(tile) & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16: f32 accumulate, bf16 x bf16, both K-major, M 128, N n
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(B_BM >> 4) << 24);
}


// byte offset of element (row, col) inside a K-major tile of 64 bf16 per row laid out with the 128-byte swizzle (what a
// TMA load with CU_TENSOR_MAP_SWIZZLE_128B leaves, and what operand_desc describes); the tile starts on a 1024-byte boundary
__device__ __forceinline__ uint32_t swz128(int row, int col) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((((col >> 3) ^ (row & 7)) & 7) << 4) + (col & 7) * 2);
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    }
    return fn;
}
// bf16 [rows][cols] row-major, boxes of [64 columns, box_rows rows], with the 128-byte swizzle or without
inline bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, bool swizzle = true) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {B_BK, box_rows};
    const cuuint32_t es[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


}  // namespace tcc
}  // namespace ava

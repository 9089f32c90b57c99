// bf16 limbs of an f32 value with the hardware's conversion (cvt.rn.bf16.f32: round to nearest even, one instruction
// instead of the seven of the portable form in ava_math.h).  For the tolerance mode's kernels only: the exact paths
// (the engram's bf16 store) keep f_to_bf16, whose treatment of NaN payloads is part of the bit contract.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace ava {

__device__ __forceinline__ uint16_t bf16_rn_hw(float x) {
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float bf16_widen(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

// hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid): both differences are exact in f32, the three sum to x to 2^-24
__device__ __forceinline__ void limbs3_hw(float x, uint16_t& l0, uint16_t& l1, uint16_t& l2) {
    l0 = bf16_rn_hw(x);
    const float r1 = __fsub_rn(x, bf16_widen(l0));
    l1 = bf16_rn_hw(r1);
    l2 = bf16_rn_hw(__fsub_rn(r1, bf16_widen(l1)));
}

}  // namespace ava

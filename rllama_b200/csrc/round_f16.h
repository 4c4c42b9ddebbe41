// Rounding an f32 pair to the nearest f16 values (ties to even) and back to f32, the rounding the reference applies to
// the output of every f16 contraction (src/tensor.rs: f16 matrix products are computed in f32 and stored as f16).
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

// a, b <- the f16 values nearest to them, as f32. One packed conversion for the pair and two mixed-precision adds of
// -0 (exact for every f16 value, sign of zero kept, NaN stays NaN) instead of four conversions: the conversion unit
// issues a fraction of what the FMA pipe does, and a tile's epilogue converts every element it stores.
// tests/cuda/round_pair_check.cu compares both steps with __float2half_rn / __half2float bit for bit.
__device__ __forceinline__ void round_pair_f16(float& a, float& b) {
    const __half2 h = __floats2half2_rn(a, b);
    const uint32_t hb = *reinterpret_cast<const uint32_t*>(&h);
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(a) : "h"((unsigned short)(hb & 0xffffu)), "f"(-0.0f));
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(b) : "h"((unsigned short)(hb >> 16)), "f"(-0.0f));
}

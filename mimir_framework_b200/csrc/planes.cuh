// planes.cuh — how an fp32 value becomes the 16-bit operand planes of the tensor-core kernels.
//
// x = hi + lo, hi = rn16(x), lo = rn16(x - hi), in one of two 16-bit formats chosen once per process
// (plane_format(), common.h):
//   PLANES_F16  (default)  hi and lo are IEEE half: 11 + 11 significant bits, |x - (hi + lo)| <= 2^-23 |x| while lo
//                          stays a normal half (|x| >= 2^-3), else <= 2^-25 absolute.  Range: |x| <= 65504, beyond
//                          that hi is +-inf and the result is visibly non-finite.  Weights are multiplied by a power
//                          of two per layer (weight_plane_scale) so that their largest magnitude sits near 2^14; the
//                          GEMM epilogue divides it out again, exactly.
//   PLANES_BF16            hi and lo are bfloat16: 8 + 8 significant bits, error <= 2^-17 |x| whatever the magnitude.
// Measured on B200 (K = 768, normal operands, two MMAs per K step): operand rounding contributes 2.45e-6 of the
// result's rms with bf16 planes and < 2e-7 with half planes; what remains is the tensor core's truncating fp32
// accumulation (gemm_sm100.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace mb {

enum : int { PLANES_BF16 = 0, PLANES_F16 = 1 };

namespace {

// two values -> two packed pairs (element 0 in the low half)
__device__ __forceinline__ void split_pair(float x0, float x1, int f16, uint32_t& hi, uint32_t& lo) {
  if (f16) {
    const __half2 h2 = __floats2half2_rn(x0, x1);
    const float2 hf = __half22float2(h2);
    const __half2 l2 = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h2);
    lo = *reinterpret_cast<const uint32_t*>(&l2);
  } else {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(x0, x1);
    const float2 hf = __bfloat1622float2(h2);
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(x0 - hf.x, x1 - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h2);
    lo = *reinterpret_cast<const uint32_t*>(&l2);
  }
}

__device__ __forceinline__ void split_one(float x, int f16, uint16_t& hi, uint16_t& lo) {
  if (f16) {
    const __half h = __float2half_rn(x);
    const __half l = __float2half_rn(x - __half2float(h));
    hi = *reinterpret_cast<const uint16_t*>(&h);
    lo = *reinterpret_cast<const uint16_t*>(&l);
  } else {
    const __nv_bfloat16 h = __float2bfloat16_rn(x);
    const __nv_bfloat16 l = __float2bfloat16_rn(x - __bfloat162float(h));
    hi = *reinterpret_cast<const uint16_t*>(&h);
    lo = *reinterpret_cast<const uint16_t*>(&l);
  }
}

}  // namespace
}  // namespace mb

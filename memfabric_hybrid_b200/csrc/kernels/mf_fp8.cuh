// fp8 e4m3 block quantisation with power-of-two scales (UE8M0), the activation / weight format of the
// expert GEMMs: a block of 128 values shares one scale s = 2^e, the smallest power of two with
// amax / s <= 448. Such a scale is exactly the byte the block-scaled tensor-core MMA wants (its biased
// fp32 exponent), and multiplying or dividing by it is exact.
#pragma once
#include <cuda_fp8.h>
#include <stdint.h>

namespace mfk {

__device__ __forceinline__ float pow2_scale_e4m3(float amax)
{
    if (!(amax > 0.f)) return 1.f;
    const uint32_t b = __float_as_uint(amax * (1.f / 448.f));
    uint32_t e = b >> 23;                // amax > 0: the sign bit is clear
    if ((b & 0x7FFFFFu) != 0) e += 1;    // round the scale up to the next power of two
    e = e < 1u ? 1u : (e > 254u ? 254u : e);
    return __uint_as_float(e << 23);
}

// The UE8M0 byte of a power-of-two fp32 scale.
__device__ __forceinline__ uint32_t ue8m0_byte(float scale) { return (__float_as_uint(scale) >> 23) & 0xFFu; }

// Four floats -> four e4m3 bytes (saturating), x[i] * mul.
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d, float mul)
{
    return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a * mul, b * mul), __NV_SATFINITE, __NV_E4M3) |
           ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(c * mul, d * mul), __NV_SATFINITE, __NV_E4M3) << 16);
}

}  // namespace mfk

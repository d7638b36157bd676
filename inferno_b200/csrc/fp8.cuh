// FP8 E4M3FN codec of the Laguna KV cache (crates/backend/src/metal/kernels/fp8_attention_kernels.metal:11-54),
// shared by the codec entry points, the FP8 append and the attention kernels that read FP8 pages.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace inf {

// laguna_fp8_e4m3fn_encode (fp8_attention_kernels.metal:29-54), with the exponent taken from the float's bits
// instead of floor(log2()).
__device__ __forceinline__ uint8_t fp8_e4m3fn_encode(float value) {
    if (isnan(value) || value == 0.0f) return 0;
    const uint32_t sign = value < 0.0f ? 0x80u : 0u;
    const float mag = fminf(fabsf(value), 448.0f);
    if (mag < 0.015625f) {  // below 2^-6, the smallest normal value: multiples of 2^-9
        const uint32_t mant = (uint32_t)rintf(mag * 512.0f);
        return (uint8_t)(sign | min(mant, 8u));
    }
    int e = (int)((__float_as_uint(mag) >> 23) & 0xffu) - 127;  // floor(log2(mag)) for a normal float
    uint32_t exponent = (uint32_t)(e + 7);
    const float normalized = mag * __uint_as_float((uint32_t)(127 - e) << 23);  // mag * 2^-e, in [1, 2), exact
    uint32_t mant = (uint32_t)rintf((normalized - 1.0f) * 8.0f);  // ties to even
    if (mant == 8u) {
        mant = 0u;
        exponent += 1u;
    }
    if (exponent > 15u || (exponent == 15u && mant > 6u)) {
        exponent = 15u;
        mant = 6u;
    }
    return (uint8_t)(sign | (exponent << 3) | mant);
}

// laguna_fp8_e4m3fn_decode (fp8_attention_kernels.metal:11-27)
__device__ __forceinline__ float fp8_e4m3fn_decode(uint8_t bits) {
    const uint32_t sign = bits >> 7, exponent = (bits >> 3) & 0x0fu, mant = bits & 0x07u;
    if (exponent == 15u && mant == 7u) return 0.0f;
    const float mag = exponent == 0u ? (float)mant * 0.001953125f
                                     : (1.0f + (float)mant * 0.125f) * __uint_as_float((exponent + 120u) << 23);  // 2^(exponent-7)
    return sign ? -mag : mag;
}

// Two E4M3FN bytes (the low and the high byte of `pair`) to two fp16 values, exact (every E4M3FN value is an fp16
// value).  The two NaN codes 0x7f / 0xff come out as fp16 NaN here, not as the zero the scalar decode gives: the
// encoder above never writes them, and pools are expected to hold encoder output.
__device__ __forceinline__ uint32_t fp8x2_to_f16x2(uint16_t pair) {
    uint32_t out;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(out) : "h"(pair));
    return out;
}
// Four bytes to two fp16 pairs: lo = bytes 0, 1; hi = bytes 2, 3.
__device__ __forceinline__ void fp8x4_to_f16x4(uint32_t four, uint32_t& lo, uint32_t& hi) {
#ifdef INF_FP8_CVT_INT
    // Integer form.  An E4M3FN byte s eeee mmm placed as s 0eeee mmm0000000 is the fp16 value 2^-8 times the byte's
    // value, subnormals included (fp16 subnormals scale the same way); the caller multiplies by 256 once.
    const uint32_t a = __byte_perm(four, 0u, 0x1404), b = __byte_perm(four, 0u, 0x3424);  // bytes into the high byte of each half
    lo = ((a >> 1) & 0x3f803f80u) | (a & 0x80008000u);
    hi = ((b >> 1) & 0x3f803f80u) | (b & 0x80008000u);
#else
    asm("{\n\t.reg .b16 l, h;\n\t"
        "mov.b32 {l, h}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, l;\n\t"
        "cvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
        : "=r"(lo), "=r"(hi)
        : "r"(four));
#endif
}
#ifdef INF_FP8_CVT_INT
constexpr float FP8_CVT_GAIN = 256.0f;  // what fp8x4_to_f16x4 leaves out
#else
constexpr float FP8_CVT_GAIN = 1.0f;
#endif

}  // namespace inf

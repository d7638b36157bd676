// FP8 E4M3FN KV storage of the Laguna cache (crates/backend/src/metal/kernels/fp8_attention_kernels.metal:11-54,
// append kernel :227-263): a cached value is encode(x / scale) with one scale per tensor (key_scale, value_scale),
// and decode(byte) * scale when read.  Built here: the exact codec, and the dequantisation of FP8 pages into the
// fp16 pools the attention kernels read.  Attention directly over FP8 pages is not built.
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>

#include "common.cuh"

namespace {

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

__global__ void fp8_encode_kernel(const float* __restrict__ in, uint8_t* __restrict__ out, long long n, float scale) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = fp8_e4m3fn_encode(__fdiv_rn(in[i], scale));
}

__global__ void fp8_decode_kernel(const uint8_t* __restrict__ in, float* __restrict__ out, long long n, float scale) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = fp8_e4m3fn_decode(in[i]) * scale;
}

// FP8 pages [num_pages][kv_heads][page_size][head_dim] -> the fp16 pool of the same geometry, 16 values per thread
__global__ void fp8_pages_to_f16_kernel(const uint8_t* __restrict__ k8, const uint8_t* __restrict__ v8,
                                        __half* __restrict__ k16, __half* __restrict__ v16, long long n16, float key_scale,
                                        float value_scale) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n16) return;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        const uint4 raw = reinterpret_cast<const uint4*>(which ? v8 : k8)[i];
        const float scale = which ? value_scale : key_scale;
        const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
        __align__(16) __half h[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) h[j] = __float2half_rn(fp8_e4m3fn_decode(b[j]) * scale);
        uint4* dst = reinterpret_cast<uint4*>((which ? v16 : k16) + i * 16);
        dst[0] = reinterpret_cast<const uint4*>(h)[0];
        dst[1] = reinterpret_cast<const uint4*>(h)[1];
    }
}

}  // namespace

extern "C" int32_t inf_fp8_e4m3fn_encode(inf_ctx* ctx, const float* input, int64_t count, float scale, void* output) {
    INF_CHECK_CTX(ctx);
    if (!input || !output) return inf_fail(ctx, INF_E_ARG, "fp8_encode: null pointer");
    if (count <= 0) return inf_fail(ctx, INF_E_SHAPE, "fp8_encode: count must be positive");
    if (!(scale > 0.0f) || !isfinite(scale)) return inf_fail(ctx, INF_E_CONFIG, "fp8_encode: scale must be positive and finite");
    fp8_encode_kernel<<<(unsigned)((count + 255) / 256), 256, 0, ctx->stream>>>(input, (uint8_t*)output, count, scale);
    INF_LAUNCH_CHECK(ctx, "fp8_encode_kernel");
    return INF_OK;
}

extern "C" int32_t inf_fp8_e4m3fn_decode(inf_ctx* ctx, const void* input, int64_t count, float scale, float* output) {
    INF_CHECK_CTX(ctx);
    if (!input || !output) return inf_fail(ctx, INF_E_ARG, "fp8_decode: null pointer");
    if (count <= 0) return inf_fail(ctx, INF_E_SHAPE, "fp8_decode: count must be positive");
    if (!(scale > 0.0f) || !isfinite(scale)) return inf_fail(ctx, INF_E_CONFIG, "fp8_decode: scale must be positive and finite");
    fp8_decode_kernel<<<(unsigned)((count + 255) / 256), 256, 0, ctx->stream>>>((const uint8_t*)input, output, count, scale);
    INF_LAUNCH_CHECK(ctx, "fp8_decode_kernel");
    return INF_OK;
}

extern "C" int32_t inf_kv_pool_from_fp8(inf_ctx* ctx, const void* k_fp8, const void* v_fp8, float key_scale,
                                        float value_scale, const inf_kv_pool* pool) {
    INF_CHECK_CTX(ctx);
    if (!k_fp8 || !v_fp8 || !pool || !pool->k || !pool->v) return inf_fail(ctx, INF_E_ARG, "kv_pool_from_fp8: null pointer");
    if (!(key_scale > 0.0f) || !(value_scale > 0.0f) || !isfinite(key_scale) || !isfinite(value_scale))
        return inf_fail(ctx, INF_E_CONFIG, "kv_pool_from_fp8: scales must be positive and finite");
    const long long n = (long long)pool->num_pages * pool->kv_heads * pool->page_size * pool->head_dim;
    if (n % 16 != 0 || (((uintptr_t)k_fp8 | (uintptr_t)v_fp8) & 15))
        return inf_fail(ctx, INF_E_SHAPE, "kv_pool_from_fp8: pages must be 16-byte aligned multiples of 16 values");
    fp8_pages_to_f16_kernel<<<(unsigned)((n / 16 + 255) / 256), 256, 0, ctx->stream>>>(
        (const uint8_t*)k_fp8, (const uint8_t*)v_fp8, (__half*)pool->k, (__half*)pool->v, n / 16, key_scale, value_scale);
    INF_LAUNCH_CHECK(ctx, "fp8_pages_to_f16_kernel");
    return INF_OK;
}

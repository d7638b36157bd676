// FP8 E4M3FN KV storage of the Laguna cache (crates/backend/src/metal/kernels/fp8_attention_kernels.metal:11-54,
// append kernel :227-263): a cached value is encode(x / scale) with one scale per tensor (key_scale, value_scale),
// and decode(byte) * scale when read.  Built here: the exact codec, and the dequantisation of FP8 pages into the
// fp16 pools.  The FP8 append and the decode attention that reads FP8 pages directly live with their fp16
// counterparts (rope_append.cu, gqa_decode.cu).
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>

#include "common.cuh"
#include "fp8.cuh"

using namespace inf;

namespace {

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

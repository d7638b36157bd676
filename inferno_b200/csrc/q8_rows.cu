// Q8Row cold-store codec of the GLM KV tiers (crates/cache/src/cold_kv.rs:1624-1703; device decode
// crates/backend/src/metal/kernels/cast_kernels.metal:31-56): a row of `dim` f32 values is stored as a
// little-endian f32 scale (max|x| / 127, or 1.0 for an all-zero row) followed by `dim` signed bytes
// round(x / scale) clamped to +-127.  Encode, decode, and the thaw of cold latent / rope rows straight into the
// pages of the MLA pool (dequantise on load).
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float row_scale(const uint8_t* row) {  // the scale sits at any byte alignment
    const uint32_t bits = (uint32_t)row[0] | ((uint32_t)row[1] << 8) | ((uint32_t)row[2] << 16) | ((uint32_t)row[3] << 24);
    return __uint_as_float(bits);
}

// one warp per row
__global__ void q8_rows_encode_kernel(const float* __restrict__ in, uint8_t* __restrict__ payload, long long rows, int dim) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* x = in + row * dim;
    float m = 0.f;
    for (int d = lane; d < dim; d += 32) m = fmaxf(m, fabsf(x[d]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float scale = m == 0.f ? 1.0f : __fdiv_rn(m, 127.0f);
    uint8_t* dst = payload + row * (dim + 4);
    if (lane < 4) dst[lane] = (uint8_t)(__float_as_uint(scale) >> (8 * lane));
    for (int d = lane; d < dim; d += 32) {
        const float qv = fminf(fmaxf(roundf(__fdiv_rn(x[d], scale)), -127.0f), 127.0f);  // round half away from zero
        dst[4 + d] = (uint8_t)(int8_t)(int)qv;
    }
}

__global__ void q8_rows_decode_kernel(const uint8_t* __restrict__ payload, float* __restrict__ out, long long rows, int dim) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const uint8_t* src = payload + row * (dim + 4);
    const float scale = row_scale(src);
    for (int d = lane; d < dim; d += 32) out[row * dim + d] = (float)(int8_t)src[4 + d] * scale;
}

// Cold latent rows [batch][tokens][latent] and rope rows [batch][tokens][rope] (two Q8Row payloads, as the
// reference keeps K and V records) -> fp16 rows of the paged pool at logical positions first_token + t.
__global__ void q8_rows_thaw_mla_kernel(const uint8_t* __restrict__ latent_payload, const uint8_t* __restrict__ rope_payload,
                                        __half* __restrict__ pool, int num_pages, int page_size,
                                        const int* __restrict__ pages, int max_pages, int tokens, int first_token, int L,
                                        int R, long long rows, int* __restrict__ status) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int b = (int)(row / tokens), t = (int)(row % tokens);
    const int position = first_token + t;
    const int slot = position / page_size;
    if (slot >= max_pages) {
        if (lane == 0) atomicOr(status, INF_STATUS_BAD_LEN);
        return;
    }
    const int page = pages[(long long)b * max_pages + slot];
    if (page < 0 || page >= num_pages) {
        if (lane == 0) atomicOr(status, INF_STATUS_BAD_PAGE);
        return;
    }
    __half* dst = pool + ((long long)page * page_size + position % page_size) * (L + R);
    const uint8_t* ls = latent_payload + row * (L + 4);
    const uint8_t* rs = rope_payload + row * (R + 4);
    const float lscale = row_scale(ls), rscale = row_scale(rs);
    for (int d = lane; d < L; d += 32) dst[d] = __float2half_rn((float)(int8_t)ls[4 + d] * lscale);
    for (int d = lane; d < R; d += 32) dst[L + d] = __float2half_rn((float)(int8_t)rs[4 + d] * rscale);
}

}  // namespace

extern "C" int32_t inf_q8_rows_encode(inf_ctx* ctx, const float* input, int64_t rows, int32_t dim, void* payload) {
    INF_CHECK_CTX(ctx);
    if (!input || !payload) return inf_fail(ctx, INF_E_ARG, "q8_rows_encode: null pointer");
    if (rows <= 0 || dim <= 0) return inf_fail(ctx, INF_E_SHAPE, "q8_rows_encode: sizes must be positive");
    q8_rows_encode_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ctx->stream>>>(input, (uint8_t*)payload, rows, dim);
    INF_LAUNCH_CHECK(ctx, "q8_rows_encode_kernel");
    return INF_OK;
}

extern "C" int32_t inf_q8_rows_decode(inf_ctx* ctx, const void* payload, int64_t rows, int32_t dim, float* output) {
    INF_CHECK_CTX(ctx);
    if (!payload || !output) return inf_fail(ctx, INF_E_ARG, "q8_rows_decode: null pointer");
    if (rows <= 0 || dim <= 0) return inf_fail(ctx, INF_E_SHAPE, "q8_rows_decode: sizes must be positive");
    q8_rows_decode_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ctx->stream>>>((const uint8_t*)payload, output, rows, dim);
    INF_LAUNCH_CHECK(ctx, "q8_rows_decode_kernel");
    return INF_OK;
}

extern "C" int32_t inf_mla_pool_thaw_q8_rows(inf_ctx* ctx, const void* latent_payload, const void* rope_payload,
                                             const inf_mla_pool* pool, const inf_page_table* table, int32_t first_token,
                                             int32_t tokens) {
    INF_CHECK_CTX(ctx);
    if (!latent_payload || !rope_payload || !pool || !table) return inf_fail(ctx, INF_E_ARG, "mla_pool_thaw: null pointer");
    if (!pool->rows) return inf_fail(ctx, INF_E_ARG, "mla_pool_thaw: pool has no storage");
    if (first_token < 0 || tokens <= 0) return inf_fail(ctx, INF_E_SHAPE, "mla_pool_thaw: token range must be positive");
    if ((long long)first_token + tokens > (long long)table->max_pages * pool->page_size)
        return inf_fail(ctx, INF_E_CACHE, "mla_pool_thaw: tokens %d..%d exceed the page table", first_token,
                        first_token + tokens - 1);
    const long long rows = (long long)table->batch * tokens;
    q8_rows_thaw_mla_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ctx->stream>>>(
        (const uint8_t*)latent_payload, (const uint8_t*)rope_payload, (__half*)pool->rows, pool->num_pages, pool->page_size,
        table->pages, table->max_pages, tokens, first_token, pool->latent_dim, pool->rope_dim, rows, ctx->status);
    INF_LAUNCH_CHECK(ctx, "q8_rows_thaw_mla_kernel");
    return INF_OK;
}

// laguna_gated_gqa_f16_attention_device (crates/backend/src/backend.rs:1350) as one C-ABI call, and the GLM
// paged MHA decode (paged_decode_attention_resident_device, backend.rs:1966).
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"

int inf_gqa_decode_launch(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                          int q_heads, int max_len, int split_chunk, int sliding_window, const float* gate,
                          float scale, void* out, int out_dtype, void* scratch, size_t scratch_bytes, int len_add,
                          const struct DecodeFp8* fp8);
int inf_gqa_prefill_launch(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                           int tokens, int q_heads, int sliding_window, const float* gate, float scale, void* out,
                           int out_dtype, const struct PrefillPeers* peers);

namespace {

constexpr int GLM_THREADS = 256;
constexpr int GLM_WARPS = GLM_THREADS / 32;
constexpr int GLM_MAX_DIM = 256;
constexpr float NEG_BIG = -3.4028234663852886e+38f;

// attention_kernels.metal:339-457 restated as one online-softmax pass: the eight warps of a CTA stride the
// keys of one (batch, head) row, each lane owns dim/32 consecutive pairs, partial states merge through
// shared memory.  HBM-bound: every cached byte is read once.
__global__ void __launch_bounds__(GLM_THREADS)
glm_paged_decode_kernel(const float* __restrict__ q, const __half* __restrict__ pk, const float* __restrict__ cur_k,
                        const __half* __restrict__ pv, const float* __restrict__ cur_v, float* __restrict__ out,
                        int batch, int heads, int past, int page_size, int dim, int vdim) {
    const int row = blockIdx.x, head = row % heads, b = row / heads;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per_k = dim / 32, per_v = vdim / 32;  // elements per lane, <= 8
    const float scale = 1.0f / sqrtf((float)dim);
    float qr[8], acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        qr[i] = i < per_k ? q[(size_t)row * dim + lane * per_k + i] : 0.f;
        acc[i] = 0.f;
    }
    float m = NEG_BIG, l = 0.f;
    for (int key = warp; key <= past; key += GLM_WARPS) {
        float kv[8], vv[8];
        if (key < past) {
            const int page = key / page_size, off = key - page * page_size;
            const size_t base = ((((size_t)page * batch + b) * heads + head) * page_size + off);
            const __half* kp = pk + base * dim + lane * per_k;
            const __half* vp = pv + base * vdim + lane * per_v;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                kv[i] = i < per_k ? __half2float(kp[i]) : 0.f;
                vv[i] = i < per_v ? __half2float(vp[i]) : 0.f;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                kv[i] = i < per_k ? cur_k[(size_t)row * dim + lane * per_k + i] : 0.f;
                vv[i] = i < per_v ? cur_v[(size_t)row * vdim + lane * per_v + i] : 0.f;
            }
        }
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += qr[i] * kv[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float s = dot * scale;
        const float mn = fmaxf(m, s);
        const float r = l == 0.f ? 0.f : expf(m - mn);
        const float w = expf(s - mn);
        l = l * r + w;
        m = mn;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = acc[i] * r + w * vv[i];
    }
    __shared__ float sm[GLM_WARPS], sl[GLM_WARPS], sacc[GLM_WARPS][GLM_MAX_DIM];
    if (lane == 0) {
        sm[warp] = m;
        sl[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < per_v) sacc[warp][lane * per_v + i] = acc[i];
    __syncthreads();
    float M = NEG_BIG;
    for (int w = 0; w < GLM_WARPS; ++w)
        if (sl[w] > 0.f) M = fmaxf(M, sm[w]);
    float L = 0.f;
    for (int w = 0; w < GLM_WARPS; ++w)
        if (sl[w] > 0.f) L += sl[w] * expf(sm[w] - M);
    for (int d = tid; d < vdim; d += GLM_THREADS) {
        float a = 0.f;
        for (int w = 0; w < GLM_WARPS; ++w)
            if (sl[w] > 0.f) a += sacc[w][d] * expf(sm[w] - M);
        out[(size_t)row * vdim + d] = a / L;
    }
}

}  // namespace

extern "C" {

int32_t inf_laguna_gated_gqa_f16_attention(inf_ctx* ctx, const float* q, const float* k, const float* v,
                                           const float* gate, const inf_kv_pool* pool, const inf_page_table* table,
                                           int32_t tokens, int32_t q_heads, int32_t max_len, int32_t sliding_window,
                                           float* out) {
    INF_CHECK_CTX(ctx);
    if (!q || !k || !v || !pool || !table || !out) return inf_fail(ctx, INF_E_ARG, "laguna_gated_gqa: null pointer");
    if (tokens <= 0 || q_heads <= 0) return inf_fail(ctx, INF_E_SHAPE, "laguna_gated_gqa: sizes must be positive");
    if (pool->head_dim != 128) return inf_fail(ctx, INF_E_SHAPE, "laguna_gated_gqa: head_dim must be 128");
    if (table->batch <= 0) return inf_fail(ctx, INF_E_SHAPE, "laguna_gated_gqa: batch must be positive");
    // scratch: the fp16 queries the attention kernels read, then (decode only) the split-KV partials
    const size_t q_bytes = ((size_t)table->batch * tokens * q_heads * 128 * sizeof(__half) + 255) & ~(size_t)255;
    const int chunk = 512;
    const size_t dec_bytes = tokens == 1 ? inf_gqa_decode_workspace_bytes(table->batch, q_heads, 128, max_len, chunk) : 0;
    if (tokens == 1 && dec_bytes == 0) return inf_fail(ctx, INF_E_SHAPE, "laguna_gated_gqa: max_len must be positive");
    int rc = inf_ensure_workspace(ctx, q_bytes + dec_bytes);
    if (rc != INF_OK) return rc;
    void* q16 = ctx->workspace;
    // append (no rotation: the operator receives q/k already roped, backend.rs:5330-5400) and convert q
    rc = inf_rope_append_gqa(ctx, q, k, v, INF_DTYPE_F32, nullptr, nullptr, 0.f, nullptr, pool, table, tokens, q_heads,
                             q16, nullptr);
    if (rc != INF_OK) return rc;
    if (tokens == 1)
        return inf_gqa_decode_launch(ctx, q16, pool, table, q_heads, max_len, chunk, sliding_window, gate, 0.f, out,
                                     INF_DTYPE_F32, (char*)ctx->workspace + q_bytes, dec_bytes, 1, nullptr);
    return inf_gqa_prefill_launch(ctx, q16, pool, table, tokens, q_heads, sliding_window, gate, 0.f, out,
                                  INF_DTYPE_F32, nullptr);
}

int32_t inf_paged_decode_attention_resident(inf_ctx* ctx, const float* q, const void* paged_k_f16, const float* cur_k,
                                            const void* paged_v_f16, const float* cur_v, int32_t batch, int32_t heads,
                                            int32_t past_tokens, int32_t page_size, int32_t head_dim,
                                            int32_t value_dim, float* out) {
    INF_CHECK_CTX(ctx);
    if (!q || !cur_k || !cur_v || !out) return inf_fail(ctx, INF_E_ARG, "paged_decode_resident: null pointer");
    if (past_tokens > 0 && (!paged_k_f16 || !paged_v_f16))
        return inf_fail(ctx, INF_E_ARG, "paged_decode_resident: null cache with cached tokens");
    if (batch <= 0 || heads <= 0 || past_tokens < 0 || page_size <= 0)
        return inf_fail(ctx, INF_E_SHAPE, "paged_decode_resident: sizes must be positive");
    if (head_dim <= 0 || value_dim <= 0 || head_dim % 32 || value_dim % 32 || head_dim > GLM_MAX_DIM ||
        value_dim > GLM_MAX_DIM)
        return INF_UNSUPPORTED;
    glm_paged_decode_kernel<<<batch * heads, GLM_THREADS, 0, ctx->stream>>>(
        q, (const __half*)paged_k_f16, cur_k, (const __half*)paged_v_f16, cur_v, out, batch, heads, past_tokens,
        page_size, head_dim, value_dim);
    INF_LAUNCH_CHECK(ctx, "glm_paged_decode_kernel");
    return INF_OK;
}

}  // extern "C"

// Attention over a compact, already-selected KV set plus the call's own tokens, expanded heads, f32 at the boundary:
// selected_decode_attention_device (crates/backend/src/backend.rs:2001, kernel fused_selected_decode_attention_f32_kernel,
// crates/backend/src/metal/kernels/attention_kernels.metal:605-721) and selected_sequence_attention_device
// (backend.rs:2015, kernel fused_selected_sequence_attention_f32_kernel, :723-968).  The reference materialises every
// score of a row in threadgroup memory and makes three passes; here a row is one CTA of four warps that take the
// keys round-robin with an online softmax each (a key's K and V row are read once, coalesced, by one warp) and merge
// at the end.  These are the small operators of the DSA path (at most 4096 keys, a handful of query rows); the
// long-context work is done by the absorbed-latent kernels.
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int SA_WARPS = 4;
constexpr int SA_MAX_DIM = 256;
constexpr int SA_PER_LANE = SA_MAX_DIM / 32;
constexpr int SA_MAX_KEYS = 4096;  // FUSED_DECODE_MAX_KEYS (attention_kernels.metal:7)

template <typename T>
__device__ __forceinline__ float sa_load(const T* p);
template <>
__device__ __forceinline__ float sa_load<float>(const float* p) {
    return *p;
}
template <>
__device__ __forceinline__ float sa_load<__half>(const __half* p) {
    return __half2float(*p);
}

// q [B,H,T,D] f32; sel_k [B,H,S,D], sel_v [B,H,S,Dv] (f32 or fp16); cur_k [B,H,T,D], cur_v [B,H,T,Dv] f32;
// out [B,H,T,Dv].  Query row t sees the S selected rows and, when cur_rows > 0, current rows 0..t.
template <typename KV>
__global__ void __launch_bounds__(SA_WARPS * 32)
selected_attention_kernel(const float* __restrict__ q, const KV* __restrict__ sel_k, const KV* __restrict__ sel_v,
                          const float* __restrict__ cur_k, const float* __restrict__ cur_v, float* __restrict__ out,
                          int heads, int S, int T, int D, int Dv, int include_current) {
    __shared__ float s_m[SA_WARPS], s_l[SA_WARPS];
    __shared__ float s_acc[SA_WARPS][SA_MAX_DIM];
    const long long row = blockIdx.x;  // (b * heads + h) * T + t
    const int t = (int)(row % T);
    const long long bh = row / T;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int visible = S + (include_current ? t + 1 : 0);
    const float scale = 1.0f / sqrtf((float)D);
    float qv[SA_PER_LANE], acc[SA_PER_LANE];
#pragma unroll
    for (int i = 0; i < SA_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < D ? q[row * D + d] * scale : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int key = warp; key < visible; key += SA_WARPS) {
        float dot = 0.f;
        float v[SA_PER_LANE];
        if (key < S) {
            const KV* kr = sel_k + (bh * S + key) * D;
            const KV* vr = sel_v + (bh * S + key) * Dv;
#pragma unroll
            for (int i = 0; i < SA_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < D) dot += qv[i] * sa_load(kr + d);
                v[i] = d < Dv ? sa_load(vr + d) : 0.f;
            }
        } else {
            const float* kr = cur_k + (bh * T + (key - S)) * D;
            const float* vr = cur_v + (bh * T + (key - S)) * Dv;
#pragma unroll
            for (int i = 0; i < SA_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < D) dot += qv[i] * kr[d];
                v[i] = d < Dv ? vr[d] : 0.f;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float m_new = fmaxf(m, dot);
        const float alpha = expf(m - m_new), p = expf(dot - m_new);  // m = -inf at the first key: alpha = 0
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < SA_PER_LANE; ++i) acc[i] = acc[i] * alpha + p * v[i];
        m = m_new;
    }
    if (lane == 0) {
        s_m[warp] = m;
        s_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < SA_PER_LANE; ++i) s_acc[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    float M = s_m[0];
#pragma unroll
    for (int w = 1; w < SA_WARPS; ++w) M = fmaxf(M, s_m[w]);
    float L = 0.f;
    float wgt[SA_WARPS];
#pragma unroll
    for (int w = 0; w < SA_WARPS; ++w) {
        wgt[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - M);  // a warp that saw no key
        L += wgt[w] * s_l[w];
    }
    for (int d = threadIdx.x; d < Dv; d += SA_WARPS * 32) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < SA_WARPS; ++w) sum += wgt[w] * s_acc[w][d];
        out[row * Dv + d] = sum / L;
    }
}

int selected_attention_launch(inf_ctx* ctx, const char* what, const float* q, const void* sel_k, const void* sel_v,
                              int sel_dtype, const float* cur_k, const float* cur_v, int batch, int heads, int S, int T,
                              int D, int Dv, int include_current, float* out) {
    if (!q || !out) return inf_fail(ctx, INF_E_ARG, "%s: null pointer", what);
    if (S > 0 && (!sel_k || !sel_v)) return inf_fail(ctx, INF_E_ARG, "%s: null selected K/V", what);
    if (include_current && (!cur_k || !cur_v)) return inf_fail(ctx, INF_E_ARG, "%s: null current K/V", what);
    if (batch <= 0 || heads <= 0 || T <= 0 || D <= 0 || Dv <= 0 || S < 0)
        return inf_fail(ctx, INF_E_SHAPE, "%s: sizes must be positive", what);
    if (D > SA_MAX_DIM || Dv > SA_MAX_DIM) return INF_UNSUPPORTED;
    if (S + (include_current ? T : 0) > SA_MAX_KEYS) return INF_UNSUPPORTED;  // the reference's kernel declines too
    if (S + (include_current ? 1 : 0) <= 0) return inf_fail(ctx, INF_E_BACKEND, "%s: no key is visible", what);
    if (sel_dtype != INF_DTYPE_F32 && sel_dtype != INF_DTYPE_F16)
        return inf_fail(ctx, INF_E_DTYPE, "%s: selected K/V must be f32 or f16", what);
    const long long rows = (long long)batch * heads * T;
    if (rows > 0x7fffffffLL) return inf_fail(ctx, INF_E_SHAPE, "%s: too many query rows", what);
    if (sel_dtype == INF_DTYPE_F16)
        selected_attention_kernel<__half><<<(unsigned)rows, SA_WARPS * 32, 0, ctx->stream>>>(
            q, (const __half*)sel_k, (const __half*)sel_v, cur_k, cur_v, out, heads, S, T, D, Dv, include_current);
    else
        selected_attention_kernel<float><<<(unsigned)rows, SA_WARPS * 32, 0, ctx->stream>>>(
            q, (const float*)sel_k, (const float*)sel_v, cur_k, cur_v, out, heads, S, T, D, Dv, include_current);
    INF_LAUNCH_CHECK(ctx, "selected_attention_kernel");
    return INF_OK;
}

}  // namespace

extern "C" int32_t inf_selected_decode_attention(inf_ctx* ctx, const float* q, const void* selected_k,
                                                 const void* selected_v, int32_t selected_dtype, const float* current_k,
                                                 const float* current_v, int32_t batch, int32_t heads,
                                                 int32_t selected_tokens, int32_t head_dim, int32_t value_dim,
                                                 int32_t include_current_kv, float* out) {
    INF_CHECK_CTX(ctx);
    if (selected_tokens <= 0)  // backend.rs:7864-7868
        return inf_fail(ctx, INF_E_BACKEND, "device selected decode attention requires at least one selected token");
    return selected_attention_launch(ctx, "selected_decode_attention", q, selected_k, selected_v, selected_dtype,
                                     current_k, current_v, batch, heads, selected_tokens, 1, head_dim, value_dim,
                                     include_current_kv != 0, out);
}

extern "C" int32_t inf_selected_sequence_attention(inf_ctx* ctx, const float* q, const float* past_k, const float* past_v,
                                                   const float* current_k, const float* current_v, int32_t batch,
                                                   int32_t heads, int32_t past_tokens, int32_t query_tokens,
                                                   int32_t head_dim, int32_t value_dim, float* out) {
    INF_CHECK_CTX(ctx);
    return selected_attention_launch(ctx, "selected_sequence_attention", q, past_k, past_v, INF_DTYPE_F32, current_k,
                                     current_v, batch, heads, past_tokens, query_tokens, head_dim, value_dim, 1, out);
}

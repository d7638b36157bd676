// RoPE, per-head RMSNorm and KV-append kernels.
//
// Elementwise, HBM-bound work: one warp per head row, lanes stride the row so every
// load and store of a warp is one contiguous segment, and the half-split rotation
// partner (d +- rotary/2) always lives in the same lane.  Frequencies arrive as tables
// computed on the host, so device powf never enters the angle.
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"
#include "fp8.cuh"

namespace {

constexpr int D = 128;  // head_dim of the GQA path

template <typename T>
__device__ __forceinline__ float ld_as_f32(const T* p);
template <>
__device__ __forceinline__ float ld_as_f32<float>(const float* p) {
    return *p;
}
template <>
__device__ __forceinline__ float ld_as_f32<__half>(const __half* p) {
    return __half2float(*p);
}

// rope_kernels.metal:167-229 for one row held as x[j] = row[lane + 32 j].
__device__ __forceinline__ void norm_rope_row(float (&x)[4], int lane, const float* __restrict__ w,
                                              const float* __restrict__ inv_freq, int rotary_dim, float position,
                                              float eps, float factor) {
    if (w) {
        float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        float inv_rms = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = x[j] * w[lane + 32 * j] * inv_rms;
    }
    // rotary 64: pairs (lane, lane+32); rotary 128: pairs (lane, lane+64) and (lane+32, lane+96)
    if (rotary_dim == 64) {
        float angle = position * inv_freq[lane];
        float c = cosf(angle) * factor, s = sinf(angle) * factor;
        float a = x[0], b = x[1];
        x[0] = a * c + (-b) * s;
        x[1] = b * c + a * s;
    } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float angle = position * inv_freq[lane + 32 * j];
            float c = cosf(angle) * factor, s = sinf(angle) * factor;
            float a = x[j], b = x[j + 2];
            x[j] = a * c + (-b) * s;
            x[j + 2] = b * c + a * s;
        }
    }
}

// laguna_qk_rms_norm_rope_pair_device: f32 in, f32 out, Q rows then K rows in one grid.
__global__ void qk_norm_rope_pair_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                         const float* __restrict__ qw, const float* __restrict__ kw,
                                         const float* __restrict__ inv_freq, float* __restrict__ q_out,
                                         float* __restrict__ k_out, long long q_rows, long long k_rows, int tokens,
                                         int q_heads, int kv_heads, int rotary_dim, int position_offset, float eps,
                                         float factor) {
    long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= q_rows + k_rows) return;
    bool is_q = row < q_rows;
    long long r = is_q ? row : row - q_rows;
    int heads = is_q ? q_heads : kv_heads;
    const float* in = (is_q ? q : k) + r * D;
    float* out = (is_q ? q_out : k_out) + r * D;
    int token = (int)((r / heads) % tokens);
    float x[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = in[lane + 32 * j];
    norm_rope_row(x, lane, is_q ? qw : kw, inv_freq, rotary_dim, (float)(position_offset + token), eps, factor);
#pragma unroll
    for (int j = 0; j < 4; ++j) out[lane + 32 * j] = x[j];
}

// Fused RoPE + append.  One CTA per (sequence, token) and slice of its rows (q heads, then k heads, then v heads):
// the token's position, its page and the cos / sin of its angles are found once and shared by all its rows, and a
// row of 128 values is held by 16 threads, eight consecutive values each, so that every load and store is 16 bytes
// per thread and 256 contiguous bytes per row.  The half-split rotation partner (d +- rotary/2) sits rotary/16 lanes
// away in the same 16-lane group.
// eight consecutive input values as they lie in memory (one 16-byte piece for fp16, two for f32) ...
template <typename T>
struct Raw8;
template <>
struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = reinterpret_cast<const float4*>(p)[0];
        b = reinterpret_cast<const float4*>(p)[1];
    }
    __device__ __forceinline__ void to_f32(float (&x)[8]) const {
        x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
    }
};
template <>
struct Raw8<__half> {
    uint4 raw;
    __device__ __forceinline__ void load(const __half* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void to_f32(float (&x)[8]) const {
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            x[2 * j] = f.x, x[2 * j + 1] = f.y;
        }
    }
};
__device__ __forceinline__ void st8_as_f16(__half* p, const float (&x)[8]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(x[2 * j], x[2 * j + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// FP8: the pools hold E4M3FN bytes, stored byte = encode(x / scale) with one scale per tensor
// (fp8_attention_kernels.metal:227-263); the roped keys and the values of the call's tokens are also written out as
// fp16 (cur_k_out / cur_v_out), because attention reads the current tokens at full precision, not through the cache.
template <typename T, bool FP8>
__global__ void __launch_bounds__(256)
rope_append_gqa_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       const float* __restrict__ qw, const float* __restrict__ kw, const float* __restrict__ inv_freq,
                       int rotary_dim, float factor, float eps, void* __restrict__ k_pool, void* __restrict__ v_pool,
                       int num_pages, int page_size, const int* __restrict__ pages, const int* __restrict__ lens,
                       int max_pages, int tokens, int q_heads, int kv_heads, __half* __restrict__ q_out,
                       float* __restrict__ k_f32_out, int* __restrict__ status, float key_scale, float value_scale,
                       __half* __restrict__ cur_k_out, __half* __restrict__ cur_v_out) {
    __shared__ float2 s_cs[64];  // (cos, sin) * factor of the token's angles
    inf_pdl_wait();  // the pages may still be read by the attention kernels of the previous step
    inf_pdl_release();
    const int bt = blockIdx.x, b = bt / tokens, token = bt - b * tokens;
    const int tid = threadIdx.x, sub = tid & 15, slot_id = tid >> 4;
    const int position = lens[b] + token;
    const int half = rotary_dim >> 1;
    if (inv_freq && tid < half) {
        const float angle = (float)position * inv_freq[tid];
        s_cs[tid] = make_float2(cosf(angle) * factor, sinf(angle) * factor);
    }
    long long page_row = -1;  // first row of the token's page slot in the pools, in units of rows of 128
    {
        const int slot = position / page_size;
        if (position < 0 || slot >= max_pages) {
            if (tid == 0 && blockIdx.y == 0) atomicOr(status, INF_STATUS_BAD_LEN);
        } else {
            const int page = pages[(long long)b * max_pages + slot];
            if (page < 0 || page >= num_pages) {
                if (tid == 0 && blockIdx.y == 0) atomicOr(status, INF_STATUS_BAD_PAGE);
            } else {
                page_row = (long long)page * kv_heads * page_size + position % page_size;
            }
        }
    }
    __syncthreads();
    const int rows_per_token = q_heads + 2 * kv_heads;
    const int partner = half >> 3;  // lanes between a value and its rotation partner: 4 or 8
    const int d0 = sub * 8;
    // where row rr of the token lies in its input tensor
    auto row_source = [&](int rr) -> const T* {
        const int kind = rr < q_heads ? 0 : (rr < q_heads + kv_heads ? 1 : 2);
        const int head = kind == 0 ? rr : (kind == 1 ? rr - q_heads : rr - q_heads - kv_heads);
        return (kind == 0 ? q : (kind == 1 ? k : v)) + ((long long)bt * (kind == 0 ? q_heads : kv_heads) + head) * D + d0;
    };
    const int stride = 16 * gridDim.y;
    Raw8<T> ahead{};  // the next trip's values are requested before this trip's are worked on
    if ((int)(blockIdx.y * 16) + slot_id < rows_per_token) ahead.load(row_source(blockIdx.y * 16 + slot_id));
    for (int base = blockIdx.y * 16; base < rows_per_token; base += stride) {  // the same trips for every thread
        const int rr = base + slot_id;
        const bool active = rr < rows_per_token;
        const int kind = rr < q_heads ? 0 : (rr < q_heads + kv_heads ? 1 : 2);
        const int head = kind == 0 ? rr : (kind == 1 ? rr - q_heads : rr - q_heads - kv_heads);
        const long long in_row = (long long)bt * (kind == 0 ? q_heads : kv_heads) + head;
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = 0.f;
        if (active) ahead.to_f32(x);
        if (rr + stride < rows_per_token) ahead.load(row_source(rr + stride));
        if (inv_freq) {  // uniform; the shuffles below are executed by whole warps, rows that are not rotated drop the result
            const float* w = kind == 0 ? qw : kw;
            const bool rotate = active && kind != 2;
            if (qw || kw) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (rotate && w) {
                    const float inv_rms = rsqrtf(ss / (float)D + eps);
                    const float4 w0 = reinterpret_cast<const float4*>(w + d0)[0], w1 = reinterpret_cast<const float4*>(w + d0)[1];
                    const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[j] = x[j] * wv[j] * inv_rms;
                }
            }
            const bool first = d0 < half, second = !first && d0 < rotary_dim;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float other = __shfl_xor_sync(0xffffffffu, x[j], partner);
                if (rotate && (first || second)) {
                    const float2 cs = s_cs[first ? d0 + j : d0 + j - half];
                    const float a = first ? x[j] : other, bb = first ? other : x[j];
                    x[j] = first ? a * cs.x + (-bb) * cs.y : bb * cs.x + a * cs.y;
                }
            }
        }
        if (!active) continue;
        if (kind == 0) {
            st8_as_f16(q_out + in_row * D + d0, x);
            continue;
        }
        if (kind == 1 && k_f32_out) {
            float4* o = reinterpret_cast<float4*>(k_f32_out + in_row * D + d0);
            o[0] = make_float4(x[0], x[1], x[2], x[3]);
            o[1] = make_float4(x[4], x[5], x[6], x[7]);
        }
        if (FP8) {
            __half* cur = kind == 1 ? cur_k_out : cur_v_out;
            if (cur) st8_as_f16(cur + in_row * D + d0, x);
            if (page_row >= 0) {
                const float scale = kind == 1 ? key_scale : value_scale;
                uint32_t w[2] = {0u, 0u};
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j >> 2] |= (uint32_t)inf::fp8_e4m3fn_encode(__fdiv_rn(x[j], scale)) << (8 * (j & 3));
                uint8_t* pool8 = reinterpret_cast<uint8_t*>(kind == 1 ? k_pool : v_pool);
                *reinterpret_cast<uint2*>(pool8 + (page_row + (long long)head * page_size) * D + d0) = make_uint2(w[0], w[1]);
            }
        } else if (page_row >= 0) {
            st8_as_f16(reinterpret_cast<__half*>(kind == 1 ? k_pool : v_pool) + (page_row + (long long)head * page_size) * D + d0, x);
        }
    }
}

struct InvFreq64 {
    float v[64];
};

// rope_kernels.metal:5-40: one thread per (even, odd) pair.
__global__ void rope_slice_kernel(const float* __restrict__ in, float* __restrict__ out, long long pair_total,
                                  int tokens, int heads, int rope_dim, int position_offset, InvFreq64 f) {
    long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= pair_total) return;
    int pair_count = rope_dim / 2;
    int pair = (int)(gid % pair_count);
    int token = (int)((gid / ((long long)pair_count * heads)) % tokens);
    float angle = (float)(position_offset + token) * f.v[pair];
    float c = cosf(angle), s = sinf(angle);
    float2 eo = reinterpret_cast<const float2*>(in)[gid];
    reinterpret_cast<float2*>(out)[gid] = make_float2(eo.x * c - eo.y * s, eo.x * s + eo.y * c);
}

// norm_kernels.metal:52-115 fused with the paged append.  One 128-thread block per token row.
__global__ void __launch_bounds__(128)
mla_postprocess_append_kernel(const float* __restrict__ in, const float* __restrict__ w, float eps, InvFreq64 f,
                              __half* __restrict__ pool, int num_pages, int page_size, const int* __restrict__ pages,
                              const int* __restrict__ lens, int max_pages, int tokens, int L, int R,
                              float* __restrict__ latent_out, float* __restrict__ rope_out, int* __restrict__ status) {
    inf_pdl_wait();  // the pages may still be read by the attention kernels of the previous step
    inf_pdl_release();
    long long row = blockIdx.x;
    int tid = threadIdx.x;
    int b = (int)(row / tokens), token = (int)(row % tokens);
    const float* x = in + row * (L + R);
    __shared__ float warp_sums[4];
    // Everything that does not depend on another load is requested first (the sequence length, up to four latent
    // values and weights per thread, the rope pair), and the page lookup, which does, runs under the reduction: the
    // kernel is one token's worth of work and its time is the length of its chain of loads.
    constexpr int KEEP = 4;
    const bool in_regs = L <= KEEP * 128;
    const int len_b = lens[b];
    float xv[KEEP], wv[KEEP];
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int d = tid + 128 * k;
        xv[k] = (in_regs && d < L) ? x[d] : 0.0f;
        wv[k] = (in_regs && d < L) ? w[d] : 0.0f;
    }
    float rope_value = 0.0f, rope_partner = 0.0f;
    if (tid < R) {
        rope_value = x[L + tid];
        rope_partner = x[L + ((tid & 1) == 0 ? tid + 1 : tid - 1)];
    }
    int position = len_b + token;
    int slot = position / page_size;
    __half* dst = nullptr;
    if (position < 0 || slot >= max_pages) {
        if (tid == 0) atomicOr(status, INF_STATUS_BAD_LEN);
    } else {
        int page = pages[(long long)b * max_pages + slot];
        if (page < 0 || page >= num_pages) {
            if (tid == 0) atomicOr(status, INF_STATUS_BAD_PAGE);
        } else {
            dst = pool + ((long long)page * page_size + position % page_size) * (L + R);
        }
    }
    float ss = 0.0f;
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) ss += xv[k] * xv[k];  // same order as the loop below: d = tid, tid + 128, ...
    } else {
        for (int d = tid; d < L; d += 128) ss += x[d] * x[d];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) warp_sums[tid >> 5] = ss;
    __syncthreads();
    float total = warp_sums[0] + warp_sums[1] + warp_sums[2] + warp_sums[3];
    float norm_scale = rsqrtf(total / (float)L + eps);
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int d = tid + 128 * k;
            if (d < L) {
                float y = xv[k] * norm_scale * wv[k];
                if (latent_out) latent_out[row * L + d] = y;
                if (dst) dst[d] = __float2half_rn(y);
            }
        }
    } else {
        for (int d = tid; d < L; d += 128) {
            float y = x[d] * norm_scale * w[d];
            if (latent_out) latent_out[row * L + d] = y;
            if (dst) dst[d] = __float2half_rn(y);
        }
    }
    for (int d = tid; d < R; d += 128) {
        bool even = (d & 1) == 0;
        float angle = (float)position * f.v[d >> 1];
        float value = d == tid ? rope_value : x[L + d], partner = d == tid ? rope_partner : x[L + (even ? d + 1 : d - 1)];
        float rotated = even ? -partner : partner;
        float y = value * cosf(angle) + rotated * sinf(angle);
        if (rope_out) rope_out[row * R + d] = y;
        if (dst) dst[L + d] = __float2half_rn(y);
    }
}

// layout_kernels.metal:205-232 under a page table: one warp per (b, head, token) row of 128 halves.
__global__ void linearize_paged_kernel(const __half* __restrict__ pool, const int* __restrict__ pages, int max_pages,
                                       int num_pages, int kv_heads, int page_size, int tokens, long long rows,
                                       __half* __restrict__ out, int* __restrict__ status) {
    long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    int t = (int)(row % tokens);
    int h = (int)((row / tokens) % kv_heads);
    int b = (int)(row / ((long long)tokens * kv_heads));
    int page = pages[(long long)b * max_pages + t / page_size];
    if (page < 0 || page >= num_pages) {
        if (lane == 0) atomicOr(status, INF_STATUS_BAD_PAGE);
        return;
    }
    const uint2* src =
        reinterpret_cast<const uint2*>(pool + ((((long long)page * kv_heads + h) * page_size) + t % page_size) * D);
    reinterpret_cast<uint2*>(out + row * D)[lane] = src[lane];
}

void host_inv_freq_glm(float theta, int rope_dim, InvFreq64* f) {
    int pair_count = rope_dim / 2;
    for (int p = 0; p < 64; ++p) f->v[p] = p < pair_count ? 1.0f / powf(theta, (float)p / (float)pair_count) : 0.0f;
}

int check_rope(inf_ctx* ctx, const inf_rope_table* rope) {
    if (!rope->inv_freq) return inf_fail(ctx, INF_E_ARG, "rope table has no device frequencies");
    if (rope->rotary_dim != 64 && rope->rotary_dim != 128)
        return inf_fail(ctx, INF_E_BACKEND, "Laguna rotary dimension must be 64 or 128, got %d", rope->rotary_dim);
    return INF_OK;
}

}  // namespace

extern "C" {

int32_t inf_qk_rms_norm_rope(inf_ctx* ctx, const float* input, const float* norm_weight, float eps,
                             int32_t position_offset, const inf_rope_table* rope, int32_t batch, int32_t tokens,
                             int32_t heads, int32_t head_dim, float* output) {
    INF_CHECK_CTX(ctx);
    if (!input || !rope || !output) return inf_fail(ctx, INF_E_ARG, "qk_rms_norm_rope: null pointer");
    if (head_dim != D) return inf_fail(ctx, INF_E_SHAPE, "qk_rms_norm_rope: head_dim must be 128, got %d", head_dim);
    if (batch <= 0 || tokens <= 0 || heads <= 0) return inf_fail(ctx, INF_E_SHAPE, "qk_rms_norm_rope: sizes must be positive");
    int rc = check_rope(ctx, rope);
    if (rc != INF_OK) return rc;
    // the pair kernel with an empty K side: one warp per head row
    const long long rows = (long long)batch * tokens * heads;
    qk_norm_rope_pair_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, ctx->stream>>>(
        input, nullptr, norm_weight, nullptr, rope->inv_freq, output, nullptr, rows, 0, tokens, heads, 1, rope->rotary_dim,
        position_offset, eps, rope->attention_factor);
    INF_LAUNCH_CHECK(ctx, "qk_norm_rope_pair_kernel");
    return INF_OK;
}

int32_t inf_laguna_qk_rms_norm_rope_pair(inf_ctx* ctx, const float* q, const float* k, const float* qw,
                                         const float* kw, float eps, int32_t position_offset,
                                         const inf_rope_table* rope, int32_t batch, int32_t tokens, int32_t q_heads,
                                         int32_t kv_heads, int32_t head_dim, float* q_out, float* k_out) {
    INF_CHECK_CTX(ctx);
    if (!q || !k || !rope || !q_out || !k_out) return inf_fail(ctx, INF_E_ARG, "qk_norm_rope_pair: null pointer");
    if (head_dim != D) return inf_fail(ctx, INF_E_SHAPE, "qk_norm_rope_pair: head_dim must be 128, got %d", head_dim);
    if (batch <= 0 || tokens <= 0 || q_heads <= 0 || kv_heads <= 0)
        return inf_fail(ctx, INF_E_SHAPE, "qk_norm_rope_pair: sizes must be positive");
    int rc = check_rope(ctx, rope);
    if (rc != INF_OK) return rc;
    long long q_rows = (long long)batch * tokens * q_heads, k_rows = (long long)batch * tokens * kv_heads;
    long long rows = q_rows + k_rows;
    int blocks = (int)((rows + 7) / 8);
    qk_norm_rope_pair_kernel<<<blocks, 256, 0, ctx->stream>>>(q, k, qw, kw, rope->inv_freq, q_out, k_out, q_rows,
                                                              k_rows, tokens, q_heads, kv_heads, rope->rotary_dim,
                                                              position_offset, eps, rope->attention_factor);
    INF_LAUNCH_CHECK(ctx, "qk_norm_rope_pair_kernel");
    return INF_OK;
}

}  // extern "C"

// The fp16 and the FP8 entry points differ only in the pool's element type.
static int rope_append_gqa_any(inf_ctx* ctx, const void* q, const void* k, const void* v, int32_t in_dtype,
                               const float* qw, const float* kw, float eps, const inf_rope_table* rope,
                               const inf_kv_pool* pool, bool fp8, float key_scale, float value_scale,
                               const inf_page_table* table, int32_t tokens, int32_t q_heads, void* q_out_f16,
                               float* k_f32_out, void* cur_k_out, void* cur_v_out) {
    if (!q || !k || !v || !pool || !table || !q_out_f16) return inf_fail(ctx, INF_E_ARG, "rope_append_gqa: null pointer");
    if (!pool->k || !pool->v) return inf_fail(ctx, INF_E_ARG, "rope_append_gqa: pool has no storage");
    if (pool->head_dim != D) return inf_fail(ctx, INF_E_SHAPE, "rope_append_gqa: head_dim must be 128");
    if (fp8 && (!(key_scale > 0.f) || !(value_scale > 0.f) || !isfinite(key_scale) || !isfinite(value_scale)))
        return inf_fail(ctx, INF_E_CONFIG, "rope_append_gqa: FP8 scales must be positive and finite");
    if (tokens <= 0 || q_heads <= 0 || q_heads % pool->kv_heads != 0)
        return inf_fail(ctx, INF_E_SHAPE, "rope_append_gqa: q_heads %d must be a positive multiple of kv_heads %d",
                        q_heads, pool->kv_heads);
    if (in_dtype != INF_DTYPE_F32 && in_dtype != INF_DTYPE_F16)
        return inf_fail(ctx, INF_E_DTYPE, "rope_append_gqa: input dtype must be f32 or f16");
    if (rope) {
        int rc = check_rope(ctx, rope);
        if (rc != INF_OK) return rc;
    }
    int rc = inf_validate_table(ctx, table, pool->num_pages, pool->page_size, tokens, "rope_append_gqa", 0, 1, true);
    if (rc != INF_OK) return rc;
    const long long bt = (long long)table->batch * tokens;
    if (bt > 0x7fffffffLL) return inf_fail(ctx, INF_E_SHAPE, "rope_append_gqa: batch x tokens exceeds the launch grid");
    const int rows_per_token = q_heads + 2 * pool->kv_heads;
    // long prompts: one CTA per token walks its rows; short batches (decode): one CTA per 16 rows
    dim3 grid((unsigned)bt, bt >= 2 * ctx->sm_count ? 1u : (unsigned)((rows_per_token + 15) / 16));
    const float* inv = rope ? rope->inv_freq : nullptr;
    int rd = rope ? rope->rotary_dim : 64;
    float factor = rope ? rope->attention_factor : 1.0f;
    auto launch = [&](auto kernel, auto* tq, auto* tk, auto* tv) {
        return inf_launch_pdl(kernel, grid, dim3(256), 0, ctx->stream, tq, tk, tv, qw, kw, inv, rd, factor, eps, pool->k,
                              pool->v, pool->num_pages, pool->page_size, table->pages, table->lens, table->max_pages,
                              tokens, q_heads, pool->kv_heads, (__half*)q_out_f16, k_f32_out, ctx->status, key_scale,
                              value_scale, (__half*)cur_k_out, (__half*)cur_v_out);
    };
    const float *qf = (const float*)q, *kf = (const float*)k, *vf = (const float*)v;
    const __half *qh = (const __half*)q, *kh = (const __half*)k, *vh = (const __half*)v;
    if (in_dtype == INF_DTYPE_F32 && !fp8) INF_CUDA(ctx, launch(rope_append_gqa_kernel<float, false>, qf, kf, vf));
    if (in_dtype == INF_DTYPE_F32 && fp8) INF_CUDA(ctx, launch(rope_append_gqa_kernel<float, true>, qf, kf, vf));
    if (in_dtype == INF_DTYPE_F16 && !fp8) INF_CUDA(ctx, launch(rope_append_gqa_kernel<__half, false>, qh, kh, vh));
    if (in_dtype == INF_DTYPE_F16 && fp8) INF_CUDA(ctx, launch(rope_append_gqa_kernel<__half, true>, qh, kh, vh));
    return INF_OK;
}

extern "C" {

int32_t inf_rope_append_gqa(inf_ctx* ctx, const void* q, const void* k, const void* v, int32_t in_dtype,
                            const float* qw, const float* kw, float eps, const inf_rope_table* rope,
                            const inf_kv_pool* pool, const inf_page_table* table, int32_t tokens, int32_t q_heads,
                            void* q_out_f16, float* k_f32_out) {
    INF_CHECK_CTX(ctx);
    return rope_append_gqa_any(ctx, q, k, v, in_dtype, qw, kw, eps, rope, pool, false, 1.f, 1.f, table, tokens, q_heads,
                               q_out_f16, k_f32_out, nullptr, nullptr);
}

int32_t inf_rope_append_gqa_fp8(inf_ctx* ctx, const void* q, const void* k, const void* v, int32_t in_dtype,
                                const float* qw, const float* kw, float eps, const inf_rope_table* rope,
                                const inf_kv_pool_fp8* pool, const inf_page_table* table, int32_t tokens,
                                int32_t q_heads, void* q_out_f16, void* cur_k_out_f16, void* cur_v_out_f16) {
    INF_CHECK_CTX(ctx);
    if (!pool) return inf_fail(ctx, INF_E_ARG, "rope_append_gqa_fp8: null pool");
    const inf_kv_pool shape = {pool->k, pool->v, pool->num_pages, pool->page_size, pool->kv_heads, pool->head_dim};
    return rope_append_gqa_any(ctx, q, k, v, in_dtype, qw, kw, eps, rope, &shape, true, pool->key_scale, pool->value_scale,
                               table, tokens, q_heads, q_out_f16, nullptr, cur_k_out_f16, cur_v_out_f16);
}

int32_t inf_rope_slice(inf_ctx* ctx, const float* input, float* output, int32_t batch, int32_t tokens, int32_t heads,
                       int32_t rope_dim, int32_t position_offset, float theta) {
    INF_CHECK_CTX(ctx);
    if (!input || !output) return inf_fail(ctx, INF_E_ARG, "rope_slice: null pointer");
    if (rope_dim <= 0 || (rope_dim & 1)) return inf_fail(ctx, INF_E_SHAPE, "rope_dim must be even, got %d", rope_dim);
    if (rope_dim > 128) return inf_fail(ctx, INF_E_SHAPE, "rope_dim must be at most 128, got %d", rope_dim);
    if (batch <= 0 || tokens <= 0 || heads <= 0) return inf_fail(ctx, INF_E_SHAPE, "rope_slice: sizes must be positive");
    if (!(theta > 0.0f) || !isfinite(theta)) return inf_fail(ctx, INF_E_CONFIG, "rope theta must be positive");
    InvFreq64 f;
    host_inv_freq_glm(theta, rope_dim, &f);
    long long pairs = (long long)batch * tokens * heads * (rope_dim / 2);
    int blocks = (int)((pairs + 255) / 256);
    rope_slice_kernel<<<blocks, 256, 0, ctx->stream>>>(input, output, pairs, tokens, heads, rope_dim, position_offset, f);
    INF_LAUNCH_CHECK(ctx, "rope_slice_kernel");
    return INF_OK;
}

int32_t inf_mla_kv_postprocess_append(inf_ctx* ctx, const float* input, const float* norm_weight, float eps,
                                      float theta, const inf_mla_pool* pool, const inf_page_table* table,
                                      int32_t tokens, float* latent_out, float* rope_out) {
    INF_CHECK_CTX(ctx);
    if (!input || !norm_weight || !pool || !table) return inf_fail(ctx, INF_E_ARG, "mla_kv_postprocess: null pointer");
    if (!pool->rows) return inf_fail(ctx, INF_E_ARG, "mla_kv_postprocess: pool has no storage");
    if (tokens <= 0) return inf_fail(ctx, INF_E_SHAPE, "mla_kv_postprocess: tokens must be positive");
    if (pool->rope_dim > 128 || (pool->rope_dim & 1)) return inf_fail(ctx, INF_E_SHAPE, "rope_dim must be even and <= 128");
    if (!(theta > 0.0f) || !isfinite(theta)) return inf_fail(ctx, INF_E_CONFIG, "rope theta must be positive");
    int rc = inf_validate_table(ctx, table, pool->num_pages, pool->page_size, tokens, "mla_kv_postprocess", 0, 1, true);
    if (rc != INF_OK) return rc;
    InvFreq64 f;
    host_inv_freq_glm(theta, pool->rope_dim, &f);
    long long rows = (long long)table->batch * tokens;
    INF_CUDA(ctx, inf_launch_pdl(mla_postprocess_append_kernel, dim3((unsigned)rows), dim3(128), 0, ctx->stream, input,
                                 norm_weight, eps, f, (__half*)pool->rows, pool->num_pages, pool->page_size, table->pages,
                                 table->lens, table->max_pages, tokens, pool->latent_dim, pool->rope_dim, latent_out,
                                 rope_out, ctx->status));
    return INF_OK;
}

int32_t inf_linearize_paged(inf_ctx* ctx, const void* pool_f16, const inf_kv_pool* shape, const inf_page_table* table,
                            int32_t tokens, void* out_f16) {
    INF_CHECK_CTX(ctx);
    if (!pool_f16 || !shape || !table || !out_f16) return inf_fail(ctx, INF_E_ARG, "linearize_paged: null pointer");
    if (shape->head_dim != D) return inf_fail(ctx, INF_E_SHAPE, "linearize_paged: head_dim must be 128");
    if (tokens <= 0 || tokens > table->max_pages * shape->page_size)
        return inf_fail(ctx, INF_E_CACHE, "linearize_paged: %d tokens exceed the page table", tokens);
    long long rows = (long long)table->batch * shape->kv_heads * tokens;
    int blocks = (int)((rows + 7) / 8);
    linearize_paged_kernel<<<blocks, 256, 0, ctx->stream>>>((const __half*)pool_f16, table->pages, table->max_pages,
                                                            shape->num_pages, shape->kv_heads, shape->page_size, tokens,
                                                            rows, (__half*)out_f16, ctx->status);
    INF_LAUNCH_CHECK(ctx, "linearize_paged_kernel");
    return INF_OK;
}

}  // extern "C"

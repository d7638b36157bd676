// q8_0_absorbed_mla_device (crates/backend/src/backend.rs:1982, 7695) as one C-ABI call, in the order the
// reference encodes it (crates/backend/src/metal/device.rs:3537-3584):
//     q_latent[h] = K_b[h] . q_no_rope[h]                     Q8_0 per-head matvec
//     context     = absorbed MLA attention over the paged latent / rope cache   (mla_decode.cu)
//     out[h]      = V_b[h] . context[h]                       Q8_0 per-head matvec
// plus the per-head matvec itself (kernel q8_0_packed_heads_matvec_f32_kernel,
// crates/backend/src/metal/kernels/q2_kernels.metal:3146).
#include <cuda_fp16.h>

#include "common.cuh"

size_t inf_mla_decode_scratch_bytes(const inf_ctx* ctx, int batch, int tokens, int heads, int max_len);
int inf_mla_decode_launch(inf_ctx* ctx, const void* q_f16, const inf_mla_pool* pool, const inf_page_table* table,
                          int tokens, int heads, int max_len, float scale, void* out, int out_dtype, size_t ws_offset,
                          const int* sel, const int* sel_counts, int sel_stride);

namespace {

constexpr int Q8_BLOCK_VALUES = 32;  // q2_kernels.metal:13
constexpr int Q8_BLOCK_BYTES = 34;   // q2_kernels.metal:14: little-endian f16 scale, then 32 signed quants
constexpr int MV_WARPS = 8;
constexpr int MV_ROWS = 4;  // input rows that share one pass over a weight row

// Weight [heads][out_features][in_features] in Q8_0 row blocks, input f32 [rows][heads][in_features].
// One warp per (head, output feature); lane = value inside a block, as in the reference kernel, so a warp
// reads each 34-byte block with one coalesced request.  HBM-bound: every weight byte is read once per
// MV_ROWS input rows.  out element (row, head, o) goes to out[(row * heads + head) * out_stride + o].
template <typename OutT>
__global__ void __launch_bounds__(MV_WARPS * 32)
q8_0_heads_matvec_kernel(const uint8_t* __restrict__ weights, const float* __restrict__ input, OutT* __restrict__ out,
                         int rows, int heads, int in_features, int out_features, long long out_stride) {
    inf_pdl_wait();
    inf_pdl_release();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o = blockIdx.x * MV_WARPS + warp;
    const int head = blockIdx.y;
    const int row0 = blockIdx.z * MV_ROWS;
    if (o >= out_features) return;
    const int blocks_per_row = in_features / Q8_BLOCK_VALUES;
    const uint8_t* wrow = weights + ((size_t)head * out_features + o) * blocks_per_row * Q8_BLOCK_BYTES;
    float sum[MV_ROWS];
#pragma unroll
    for (int r = 0; r < MV_ROWS; ++r) sum[r] = 0.f;
#pragma unroll 4
    for (int blk = 0; blk < blocks_per_row; ++blk) {
        const uint8_t* bp = wrow + (size_t)blk * Q8_BLOCK_BYTES;
        const float d = __half2float(__ushort_as_half((unsigned short)(bp[0] | (bp[1] << 8))));
        const float w = d * (float)(signed char)bp[2 + lane];
#pragma unroll
        for (int r = 0; r < MV_ROWS; ++r)
            if (row0 + r < rows)
                sum[r] += input[((size_t)(row0 + r) * heads + head) * in_features + blk * Q8_BLOCK_VALUES + lane] * w;
    }
#pragma unroll
    for (int r = 0; r < MV_ROWS; ++r) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], off);
        if (lane == 0 && row0 + r < rows) out[((size_t)(row0 + r) * heads + head) * out_stride + o] = OutT(sum[r]);
    }
}

// The same product for out_features % 32 == 0 (every shape of the absorbed-MLA path): a CTA owns 32 consecutive
// output features of one head (one warp per 32 / G rows at a time: with a single pass per warp and four times as
// many CTAs the operator step measured 47.5 us against 46.8 us).  G lanes share a weight row, each lane taking 16 consecutive quants (half a Q8_0
// block) per step.  Everything in a Q8_0 row is 2-byte aligned and nothing more (a block is 34 bytes), so a lane
// reads its half block as eight 16-bit loads straight from global memory -- the 32 rows of a CTA are one contiguous
// run, prefetched into L2 before the programmatic-launch wait because weights never change -- and pairs them into
// words; int8 -> f32 goes through the 2^23 trick on the integer and FP32 pipes (I2F would run at a quarter of their
// rate), and the lanes of a row meet with log2(G) shuffles.  No shared memory, no CTA barrier.  Optionally the CTAs
// with blockIdx.x == 0 also convert the head's `tail` f32 values per input row into fp16 columns
// [tail_col0, tail_col0 + tail_n) of the output row (the RoPE part of the absorbed query).
constexpr int TILE_ROWS = 32;

__device__ __forceinline__ float q8_byte_to_float(uint32_t biased_word, int byte) {
    // biased_word holds q + 128 in each byte: 0x4B0000uu is 2^23 + u exactly
    const uint32_t bits = __byte_perm(biased_word, 0x4B000000u, 0x7650 + byte);  // bytes {u, 00, 00, 4B}
    return __uint_as_float(bits) - 8388736.0f;
}

template <typename OutT, int G>
__global__ void __launch_bounds__(MV_WARPS * 32)
q8_0_heads_matvec_tile_kernel(const uint8_t* __restrict__ weights, const float* __restrict__ input,
                              OutT* __restrict__ out, int rows, int heads, int in_features, int out_features,
                              long long out_stride, const float* __restrict__ tail, int tail_n, int tail_col0) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int ROWS_PER_PASS = 32 / G;                       // weight rows a warp works on at once
    constexpr int CTA_ROWS = TILE_ROWS;
    constexpr int PASSES = TILE_ROWS / (MV_WARPS * ROWS_PER_PASS);
    const int o0 = blockIdx.x * CTA_ROWS;
    const int head = blockIdx.y;
    const int row0 = blockIdx.z * MV_ROWS;
    const int blocks_per_row = in_features / Q8_BLOCK_VALUES;
    const int row_units = blocks_per_row * (Q8_BLOCK_BYTES / 2);  // 16-bit units per weight row
    const unsigned short* w16 =
        reinterpret_cast<const unsigned short*>(weights) + ((size_t)head * out_features + o0) * row_units;
    {
        // one 128-byte line per thread and step covers the CTA's run of CTA_ROWS * row_units * 2 bytes
        const char* run = reinterpret_cast<const char*>(w16);
        const int run_bytes = CTA_ROWS * row_units * 2;
        for (int off = threadIdx.x * 128; off < run_bytes; off += MV_WARPS * 32 * 128)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(run + off));
    }
    inf_pdl_wait();
    inf_pdl_release();
    if (tail && blockIdx.x == 0) {
        for (int r = 0; r < MV_ROWS && row0 + r < rows; ++r)
            for (int d = threadIdx.x; d < tail_n; d += MV_WARPS * 32)
                out[((size_t)(row0 + r) * heads + head) * out_stride + tail_col0 + d] =
                    OutT(tail[((size_t)(row0 + r) * heads + head) * tail_n + d]);
    }
    const int gl = lane % G, sub = lane / G;
    const int chunks = in_features / 16;                        // 16-quant steps per weight row
    const int n_rows = min(MV_ROWS, rows - row0);
#pragma unroll 1
    for (int pass = 0; pass < PASSES; ++pass) {
        const int lr = (pass * MV_WARPS + warp) * ROWS_PER_PASS + sub;
        const unsigned short* wrow = w16 + (size_t)lr * row_units;
        float sum[MV_ROWS];
#pragma unroll
        for (int r = 0; r < MV_ROWS; ++r) sum[r] = 0.f;
        for (int c = gl; c < chunks; c += G) {
            const unsigned short* bp = wrow + (c >> 1) * (Q8_BLOCK_BYTES / 2);
            const float d = __half2float(__ushort_as_half(__ldg(bp)));
            const unsigned short* qp = bp + 1 + (c & 1) * 8;
            uint32_t qw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                qw[j] = ((uint32_t)__ldg(qp + 2 * j) | ((uint32_t)__ldg(qp + 2 * j + 1) << 16)) ^ 0x80808080u;
            float wf[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) wf[i] = q8_byte_to_float(qw[i >> 2], i & 3);
#pragma unroll
            for (int r = 0; r < MV_ROWS; ++r) {
                if (r < n_rows) {
                    const float4* xp = reinterpret_cast<const float4*>(
                        input + ((size_t)(row0 + r) * heads + head) * in_features + c * 16);
                    float part = 0.f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 x = __ldg(xp + i);
                        part = fmaf(x.x, wf[4 * i], part);
                        part = fmaf(x.y, wf[4 * i + 1], part);
                        part = fmaf(x.z, wf[4 * i + 2], part);
                        part = fmaf(x.w, wf[4 * i + 3], part);
                    }
                    sum[r] = fmaf(part, d, sum[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MV_ROWS; ++r) {
            if (r < n_rows) {  // uniform over the CTA
#pragma unroll
                for (int off = G / 2; off > 0; off >>= 1) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], off);
                if (gl == 0) out[((size_t)(row0 + r) * heads + head) * out_stride + o0 + lr] = OutT(sum[r]);
            }
        }
    }
}

// q_rope f32 [rows*heads][rope] -> fp16 columns [latent, latent+rope) of the absorbed query rows.
__global__ void pack_q_rope_kernel(const float* __restrict__ q_rope, __half* __restrict__ q_abs, long long n, int rope,
                                   int row_width, int col0) {
    inf_pdl_wait();
    inf_pdl_release();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long r = i / rope;
    const int d = (int)(i % rope);
    q_abs[r * row_width + col0 + d] = __float2half_rn(q_rope[i]);
}

// Already post-processed latent / rope rows (the two outputs of mla_kv_postprocess_device) stored RNE-fp16 at
// logical slot lens[b] + t: the device-side form of the reference's row blits into the paged window
// (crates/runtime/src/lib.rs:4963-5045).
__global__ void append_latent_rows_kernel(const float* __restrict__ latent, const float* __restrict__ rope,
                                          __half* __restrict__ pool, int num_pages, int page_size,
                                          const int* __restrict__ pages, const int* __restrict__ lens, int max_pages,
                                          int tokens, int L, int R, int* __restrict__ status) {
    inf_pdl_wait();  // the pages may still be read by the attention kernels of the previous step
    inf_pdl_release();
    const long long row = blockIdx.x;
    const int b = (int)(row / tokens), t = (int)(row % tokens);
    const int position = lens[b] + t;
    const int slot = position / page_size;
    if (position < 0 || slot >= max_pages) {
        if (threadIdx.x == 0) atomicOr(status, INF_STATUS_BAD_LEN);
        return;
    }
    const int page = pages[(long long)b * max_pages + slot];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, INF_STATUS_BAD_PAGE);
        return;
    }
    __half* dst = pool + ((long long)page * page_size + position % page_size) * (L + R);
    for (int d = threadIdx.x; d < L; d += blockDim.x) dst[d] = __float2half_rn(latent[row * L + d]);
    for (int d = threadIdx.x; d < R; d += blockDim.x) dst[L + d] = __float2half_rn(rope[row * R + d]);
}

template <typename OutT>
int launch_matvec(inf_ctx* ctx, const void* weights, const float* input, OutT* out, int rows, int heads, int in_features,
                  int out_features, long long out_stride, const char* name, const float* tail = nullptr, int tail_n = 0,
                  int tail_col0 = 0) {
    const bool tiled = out_features % TILE_ROWS == 0 && ((uintptr_t)weights & 1) == 0 && ((uintptr_t)input & 15) == 0;
    inf_prof_scope prof(ctx, name);
    if (tiled) {
        // lanes that share a weight row: as many as it has 16-quant steps, between 8 and 32
        const int chunks = in_features / 16;
        dim3 grid(out_features / TILE_ROWS, heads, (rows + MV_ROWS - 1) / MV_ROWS);
        auto kernel = chunks > 16 ? q8_0_heads_matvec_tile_kernel<OutT, 32>
                                  : (chunks > 8 ? q8_0_heads_matvec_tile_kernel<OutT, 16> : q8_0_heads_matvec_tile_kernel<OutT, 8>);
        INF_CUDA(ctx, inf_launch_pdl(kernel, grid, dim3(MV_WARPS * 32), 0, ctx->stream,
                                     (const uint8_t*)weights, input, out, rows, heads, in_features, out_features,
                                     out_stride, tail, tail_n, tail_col0));
    } else {
        dim3 grid((out_features + MV_WARPS - 1) / MV_WARPS, heads, (rows + MV_ROWS - 1) / MV_ROWS);
        INF_CUDA(ctx, inf_launch_pdl(q8_0_heads_matvec_kernel<OutT>, grid, dim3(MV_WARPS * 32), 0, ctx->stream,
                                     (const uint8_t*)weights, input, out, rows, heads, in_features, out_features,
                                     out_stride));
        if (tail) {
            const long long n = (long long)rows * heads * tail_n;
            INF_CUDA(ctx, inf_launch_pdl(pack_q_rope_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, ctx->stream,
                                         tail, (__half*)out, n, tail_n, (int)out_stride, tail_col0));
        }
    }
    INF_LAUNCH_CHECK(ctx, name);
    return INF_OK;
}

int check_matvec_dims(inf_ctx* ctx, long long rows, int heads, int in_features, int out_features, const char* what) {
    // crates/backend/src/metal/q2.rs:2668-2677
    if (rows <= 0 || heads <= 0 || in_features <= 0 || out_features <= 0)
        return inf_fail(ctx, INF_E_BACKEND, "%s: packed-head Q8_0 matvec dimensions must be positive", what);
    if (in_features % Q8_BLOCK_VALUES != 0)
        return inf_fail(ctx, INF_E_BACKEND, "%s: packed-head Q8_0 input width %d must be divisible by %d", what,
                        in_features, Q8_BLOCK_VALUES);
    if (heads > 65535 || (rows + MV_ROWS - 1) / MV_ROWS > 65535)
        return inf_fail(ctx, INF_E_SHAPE, "%s: %d heads x %lld rows exceed the launch grid", what, heads, rows);
    return INF_OK;
}

}  // namespace

extern "C" int32_t inf_q8_0_packed_heads_matvec(inf_ctx* ctx, const void* weights, const float* input, int32_t rows,
                                                int32_t heads, int32_t in_features, int32_t out_features,
                                                float* output) {
    INF_CHECK_CTX(ctx);
    if (!weights || !input || !output) return inf_fail(ctx, INF_E_ARG, "q8_0_packed_heads_matvec: null pointer");
    int rc = check_matvec_dims(ctx, rows, heads, in_features, out_features, "q8_0_packed_heads_matvec");
    if (rc != INF_OK) return rc;
    return launch_matvec<float>(ctx, weights, input, output, rows, heads, in_features, out_features, out_features,
                                "q8_0_heads_matvec_kernel");
}

extern "C" int32_t inf_q8_0_absorbed_mla(inf_ctx* ctx, const void* k_b_weights, const void* v_b_weights,
                                         const float* q_no_rope, const float* q_rope, const float* current_latent,
                                         const float* current_rope, const inf_mla_pool* pool,
                                         const inf_page_table* table, int32_t tokens, int32_t heads,
                                         int32_t q_no_rope_dim, int32_t value_dim, int32_t qk_head_dim,
                                         int32_t max_len, float* out) {
    INF_CHECK_CTX(ctx);
    if (!k_b_weights || !v_b_weights || !q_no_rope || !q_rope || !pool || !table || !out)
        return inf_fail(ctx, INF_E_ARG, "q8_0_absorbed_mla: null pointer");
    if ((current_latent == nullptr) != (current_rope == nullptr))
        return inf_fail(ctx, INF_E_ARG, "q8_0_absorbed_mla: current latent and rope rows come together or not at all");
    if (!pool->rows) return inf_fail(ctx, INF_E_ARG, "q8_0_absorbed_mla: pool has no storage");
    if (pool->latent_dim != 512 || pool->rope_dim != 64 || pool->page_size != 64) return INF_UNSUPPORTED;
    const int L = pool->latent_dim, R = pool->rope_dim;
    if (tokens <= 0 || heads <= 0 || max_len <= 0)
        return inf_fail(ctx, INF_E_SHAPE, "q8_0_absorbed_mla: sizes must be positive");
    if (qk_head_dim != q_no_rope_dim + R)  // backend.rs:7767-7771
        return inf_fail(ctx, INF_E_BACKEND, "absorbed MLA qk_head_dim %d must equal no-RoPE %d + RoPE %d", qk_head_dim,
                        q_no_rope_dim, R);
    const long long rows = (long long)table->batch * tokens;
    int rc = check_matvec_dims(ctx, rows, heads, q_no_rope_dim, L, "absorbed MLA K_b");
    if (rc != INF_OK) return rc;
    rc = check_matvec_dims(ctx, rows, heads, L, value_dim, "absorbed MLA V_b");
    if (rc != INF_OK) return rc;
    rc = inf_validate_table(ctx, table, pool->num_pages, pool->page_size, tokens, "q8_0_absorbed_mla");
    if (rc != INF_OK) return rc;
    if (table->host_lens)
        for (int b = 0; b < table->batch; ++b)
            if (table->host_lens[b] + tokens > max_len)
                return inf_fail(ctx, INF_E_SHAPE, "q8_0_absorbed_mla: sequence %d reaches %d rows, beyond max_len %d", b,
                                table->host_lens[b] + tokens, max_len);

    // scratch: absorbed query rows (fp16), attended latent (f32), then the decode kernel's split partials
    const size_t q_bytes = ((size_t)rows * heads * (L + R) * sizeof(__half) + 255) & ~(size_t)255;
    const size_t ctx_bytes = ((size_t)rows * heads * L * sizeof(float) + 255) & ~(size_t)255;
    const size_t total = q_bytes + ctx_bytes + inf_mla_decode_scratch_bytes(ctx, table->batch, tokens, heads, max_len);
    rc = inf_ensure_workspace(ctx, total);
    if (rc != INF_OK) return rc;
    __half* q_abs = (__half*)ctx->workspace;
    float* context = (float*)((char*)ctx->workspace + q_bytes);

    if (current_latent) {
        INF_CUDA(ctx, inf_launch_pdl(append_latent_rows_kernel, dim3((unsigned)rows), dim3(128), 0, ctx->stream,
                                     current_latent, current_rope, (__half*)pool->rows, pool->num_pages, pool->page_size,
                                     table->pages, table->lens, table->max_pages, tokens, L, R, ctx->status));
    }
    rc = launch_matvec<__half>(ctx, k_b_weights, q_no_rope, q_abs, (int)rows, heads, q_no_rope_dim, L, L + R,
                               "q8_0_heads_matvec_kernel(K_b)", q_rope, R, L);
    if (rc != INF_OK) return rc;
    const float scale = 1.0f / sqrtf((float)qk_head_dim);  // attention_kernels.metal:501: scale_dim = qk_head_dim
    rc = inf_mla_decode_launch(ctx, q_abs, pool, table, tokens, heads, max_len, scale, context, INF_DTYPE_F32,
                               q_bytes + ctx_bytes, nullptr, nullptr, 0);
    if (rc != INF_OK) return rc;
    return launch_matvec<float>(ctx, v_b_weights, context, out, (int)rows, heads, L, value_dim, value_dim,
                                "q8_0_heads_matvec_kernel(V_b)");
}

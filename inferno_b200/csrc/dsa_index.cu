// DSA indexer for sparse decode: per-token index scores and the top-k selection that feeds
// inf_mla_decode_absorbed_selected.  Reference: dsa_scores_f32_kernel and dsa_topk_block_sort / dsa_topk_merge
// (crates/backend/src/metal/kernels/dsa_kernels.metal:137-176, 178-393).
#include <cuda_fp16.h>
#include <stdint.h>

#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------- scores
// score[b][t] = sum_h w[b][h] * max(0, q[b][h] . key[b][t] / sqrt(D)), key = past_keys[b][t] for t < past, the
// current key for t == past (dsa_kernels.metal:137-176).  HBM-bound on the f32 index keys.  A CTA stages 128 key
// rows with coalesced 16-byte loads (row pitch D + 4 floats, so the row reads below do not collide on banks) and
// q in shared memory; thread (lane = token within a group of 32, warp = head residue mod 8) keeps a 4 token x 4
// head block of dot products in registers, so every value read from shared memory feeds four multiply-adds.
constexpr int SC_TOKENS = 128;
constexpr int SC_THREADS = 256;
constexpr int SC_TB = SC_TOKENS / 32;  // tokens per thread
constexpr int SC_HB = 4;               // heads per thread and pass
constexpr int SC_HG = SC_THREADS / 32; // head residues

// two fp32 multiply-adds in one instruction (packed pairs in 64-bit registers)
__device__ __forceinline__ unsigned long long ffma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__global__ void __launch_bounds__(SC_THREADS)
dsa_scores_kernel(const float* __restrict__ q, const float* __restrict__ weights, const float* __restrict__ past_keys,
                  const float* __restrict__ current_key, float* __restrict__ scores, int past, int heads, int dim) {
    extern __shared__ __align__(16) float sm[];
    inf_pdl_wait();
    inf_pdl_release();
    const int pitch = dim + 4;
    float* s_keys = sm;                          // [SC_TOKENS][pitch]
    float* s_q = sm + SC_TOKENS * pitch;         // [heads][dim]
    float* s_w = s_q + heads * dim;              // [heads]
    float* s_part = s_w + heads;                 // [SC_HG][SC_TOKENS]
    const int b = blockIdx.y;
    const int t0 = blockIdx.x * SC_TOKENS;
    const int n = past + 1;
    const int tid = threadIdx.x, lane = tid & 31, hg = tid >> 5;
    for (int i = tid; i < heads * dim / 4; i += SC_THREADS)
        reinterpret_cast<float4*>(s_q)[i] = reinterpret_cast<const float4*>(q + (size_t)b * heads * dim)[i];
    for (int i = tid; i < heads; i += SC_THREADS) s_w[i] = weights[(size_t)b * heads + i];
    const int vec_per_row = dim / 4;
    // the key rows go straight from global to shared memory (cp.async): all of a thread's 16-byte pieces are in
    // flight at once instead of one load-store round trip after another
    for (int i = tid; i < SC_TOKENS * vec_per_row; i += SC_THREADS) {
        const int r = i / vec_per_row, c = i % vec_per_row;
        const int t = t0 + r;
        float* dst = s_keys + r * pitch + c * 4;
        if (t < past) {
            const float* src = past_keys + ((size_t)b * past + t) * dim + c * 4;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src)
                         : "memory");
        } else {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t == past) v = reinterpret_cast<const float4*>(current_key + (size_t)b * dim)[c];
            *reinterpret_cast<float4*>(dst) = v;
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const float scale = rsqrtf((float)dim);
    float acc[SC_TB];
#pragma unroll
    for (int tb = 0; tb < SC_TB; ++tb) acc[tb] = 0.f;
    for (int h0 = hg; h0 < heads; h0 += SC_HB * SC_HG) {  // this thread's heads: h0, h0 + 8, h0 + 16, h0 + 24
        // each accumulator holds the (even dims, odd dims) halves of one dot product: a 16-byte shared-memory read
        // is two such pairs, so the inner step is two packed multiply-adds per (token, head) and no data movement
        unsigned long long dot2[SC_TB][SC_HB];
#pragma unroll
        for (int tb = 0; tb < SC_TB; ++tb)
#pragma unroll
            for (int g = 0; g < SC_HB; ++g) dot2[tb][g] = 0ull;
#pragma unroll 2
        for (int d = 0; d < dim; d += 4) {
            ulonglong2 kv[SC_TB], qv[SC_HB];
#pragma unroll
            for (int tb = 0; tb < SC_TB; ++tb)
                kv[tb] = *reinterpret_cast<const ulonglong2*>(s_keys + (lane + 32 * tb) * pitch + d);
#pragma unroll
            for (int g = 0; g < SC_HB; ++g) {
                const int h = min(h0 + g * SC_HG, heads - 1);  // a head past the end repeats the last one and is dropped below
                qv[g] = *reinterpret_cast<const ulonglong2*>(s_q + h * dim + d);  // same address in the warp
            }
#pragma unroll
            for (int tb = 0; tb < SC_TB; ++tb)
#pragma unroll
                for (int g = 0; g < SC_HB; ++g) {
                    dot2[tb][g] = ffma2(kv[tb].x, qv[g].x, dot2[tb][g]);
                    dot2[tb][g] = ffma2(kv[tb].y, qv[g].y, dot2[tb][g]);
                }
        }
        float dot[SC_TB][SC_HB];
#pragma unroll
        for (int tb = 0; tb < SC_TB; ++tb)
#pragma unroll
            for (int g = 0; g < SC_HB; ++g)
                dot[tb][g] = __uint_as_float((unsigned)(dot2[tb][g] & 0xffffffffull)) + __uint_as_float((unsigned)(dot2[tb][g] >> 32));
#pragma unroll
        for (int g = 0; g < SC_HB; ++g) {
            const int h = h0 + g * SC_HG;
            if (h < heads) {
                const float w = s_w[h];
#pragma unroll
                for (int tb = 0; tb < SC_TB; ++tb) acc[tb] = fmaf(w, fmaxf(dot[tb][g] * scale, 0.f), acc[tb]);
            }
        }
    }
#pragma unroll
    for (int tb = 0; tb < SC_TB; ++tb) s_part[hg * SC_TOKENS + lane + 32 * tb] = acc[tb];
    __syncthreads();
    if (tid < SC_TOKENS && t0 + tid < n) {
        float sum = 0.f;
#pragma unroll
        for (int g = 0; g < SC_HG; ++g) sum += s_part[g * SC_TOKENS + tid];
        scores[(size_t)b * n + t0 + tid] = sum;
    }
}

// ---------------------------------------------------------------------------------------------- top-k
// ids of the k best tokens, best first, where a precedes b iff score_a > score_b or (score_a == score_b and
// id_a < id_b) (dsa_precedes, dsa_kernels.metal:182-196); missing entries are 0xffffffff.  The reference sorts
// 256-token blocks and merges runs; here one CTA per sequence finds the k-th largest score with a four-pass radix
// select over the order-preserving integer image of the scores, collects everything above it plus the lowest-id
// ties, and sorts those k entries in shared memory.
constexpr int TK_THREADS = 1024;
constexpr int TK_MAX_K = 2048;
constexpr unsigned TK_INVALID = 0xffffffffu;

__device__ __forceinline__ unsigned ordered_bits(float f) {  // larger float <-> larger unsigned
    unsigned u = __float_as_uint(f);
    if (u == 0x80000000u) u = 0u;  // -0 and +0 compare equal in the reference's ordering
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA per sequence.  The row is turned into ordered integers once and kept in shared memory when it fits
// (up to TK_SMEM_ROWS tokens); the radix passes, the collection sweep and the final sort then never leave the SM.
constexpr int TK_SMEM_ROWS = 49152;  // 192 KB of ordered scores

__global__ void __launch_bounds__(TK_THREADS)
dsa_topk_kernel(const float* __restrict__ scores, unsigned* __restrict__ out_ids, int n, int k, int out_stride,
                int row_in_smem) {
    extern __shared__ __align__(16) unsigned srow[];
    __shared__ unsigned hist[256];
    __shared__ unsigned long long keys[TK_MAX_K];
    __shared__ int w_above[32], w_tie[32], w_base[32], w_quota[32];
    __shared__ unsigned sh_prefix, sh_mask;
    __shared__ int sh_remaining;
    inf_pdl_wait();
    inf_pdl_release();
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = scores + (size_t)b * n;
    unsigned* out = out_ids + (size_t)b * out_stride;
    const int want = min(k, n);
    auto value = [&](int i) -> unsigned { return row_in_smem ? srow[i] : ordered_bits(row[i]); };
    if (row_in_smem)
        for (int i = tid; i < n; i += TK_THREADS) srow[i] = ordered_bits(row[i]);
    // ---- the want-th largest value, eight bits at a time
    if (tid == 0) {
        sh_prefix = 0u;
        sh_mask = 0u;
        sh_remaining = want;
    }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < 256; i += TK_THREADS) hist[i] = 0u;
        __syncthreads();
        const unsigned prefix = sh_prefix, mask = sh_mask;
        // whole warps walk the row together so that lanes with the same digit can add once (the leading digits
        // of real scores are nearly all equal, and same-address shared atomics would serialise)
        for (int base = 0; base < n; base += TK_THREADS) {
            const int i = base + tid;
            unsigned digit = 0x100u;  // no candidate
            if (i < n) {
                const unsigned u = value(i);
                if ((u & mask) == prefix) digit = (u >> shift) & 255u;
            }
            // lanes that share lane 0's digit add once through lane 0; the others add on their own
            const unsigned first = __shfl_sync(0xffffffffu, digit, 0);
            const unsigned same = __ballot_sync(0xffffffffu, digit == first);
            if (digit == first) {
                if (lane == 0 && digit < 256u) atomicAdd(&hist[digit], (unsigned)__popc(same));
            } else if (digit < 256u) {
                atomicAdd(&hist[digit], 1u);
            }
        }
        __syncthreads();
        if (warp == 0) {
            // the bin that holds the remaining-th largest candidate: lane l owns bins 8l .. 8l+7; counts of the bins
            // above a lane come from a suffix sum across the warp, the owner then walks its eight bins
            const int remaining = sh_remaining;
            int mine[8], sum = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                mine[i] = (int)hist[lane * 8 + i];
                sum += mine[i];
            }
            int above = sum;  // inclusive suffix sum over lanes >= this one
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_down_sync(0xffffffffu, above, o);
                if (lane + o < 32) above += y;
            }
            above -= sum;  // candidates in bins owned by higher lanes
            if (above < remaining && remaining <= above + sum) {
                int left = remaining - above, bin = 7;
                for (; bin > 0; --bin) {
                    if (mine[bin] >= left) break;
                    left -= mine[bin];
                }
                sh_prefix = prefix | ((unsigned)(lane * 8 + bin) << shift);
                sh_mask = mask | (255u << shift);
                sh_remaining = left;  // how many entries equal to the final value are taken
            }
        }
        __syncthreads();
    }
    const unsigned threshold = sh_prefix;
    const int ties_wanted = sh_remaining;
    // ---- collect everything above the threshold and the ties with the lowest ids.  Warp w owns the contiguous
    //      token range [w * seg, (w + 1) * seg): a counting sweep, a prefix over the 32 warps, a writing sweep.
    for (int i = tid; i < TK_MAX_K; i += TK_THREADS) keys[i] = ~0ull;
    const int seg = ((n + 32 * 32 - 1) / (32 * 32)) * 32;  // multiple of 32, so a warp's chunks stay in id order
    const int s0 = min(n, warp * seg), s1 = min(n, s0 + seg);
    int c_above = 0, c_tie = 0;
    for (int i = s0 + lane; i < s1; i += 32) {
        const unsigned u = value(i);
        c_above += u > threshold;
        c_tie += u == threshold;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        c_above += __shfl_xor_sync(0xffffffffu, c_above, o);
        c_tie += __shfl_xor_sync(0xffffffffu, c_tie, o);
    }
    if (lane == 0) {
        w_above[warp] = c_above;
        w_tie[warp] = c_tie;
    }
    __syncthreads();
    if (warp == 0) {  // exclusive prefixes over the 32 warps' counts
        const int t_w = w_tie[lane];
        int ties_incl = t_w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, ties_incl, o);
            if (lane >= o) ties_incl += y;
        }
        const int quota = max(0, min(t_w, ties_wanted - (ties_incl - t_w)));
        const int out_w = w_above[lane] + quota;
        int out_incl = out_w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, out_incl, o);
            if (lane >= o) out_incl += y;
        }
        w_base[lane] = out_incl - out_w;
        w_quota[lane] = quota;
    }
    __syncthreads();
    {
        int pos = w_base[warp], ties_taken = 0;
        const int quota = w_quota[warp];
        for (int c0 = s0; c0 < s1; c0 += 32) {
            const int i = c0 + lane;
            unsigned u = 0u;
            bool above = false, tie = false;
            if (i < s1) {
                u = value(i);
                above = u > threshold;
                tie = u == threshold;
            }
            const unsigned tie_mask = __ballot_sync(0xffffffffu, tie);
            const bool take = above || (tie && ties_taken + __popc(tie_mask & ((1u << lane) - 1u)) < quota);
            const unsigned take_mask = __ballot_sync(0xffffffffu, take);
            if (take) keys[pos + __popc(take_mask & ((1u << lane) - 1u))] = ((unsigned long long)(~u) << 32) | (unsigned)i;
            pos += __popc(take_mask);
            ties_taken += __popc(tie_mask);
        }
    }
    __syncthreads();
    // ---- bitonic sort of the (at most 2048) entries, ascending = best first.  Exchanges at a distance below 32
    //      stay inside the 64 entries one warp owns and need only a warp barrier.
    for (int size = 2; size <= TK_MAX_K; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int i = tid;  // TK_MAX_K / 2 == TK_THREADS comparators per step
            const int lo = 2 * i - (i & (stride - 1));
            const int hi = lo + stride;
            const bool up = (lo & size) == 0;
            const unsigned long long a = keys[lo], c = keys[hi];
            if ((a > c) == up) {
                keys[lo] = c;
                keys[hi] = a;
            }
            if (stride > 32)
                __syncthreads();
            else
                __syncwarp();
            if (stride == 1 && size >= 64) __syncthreads();  // the next size starts with a long distance again
        }
    __syncthreads();
    for (int i = tid; i < k; i += TK_THREADS) out[i] = i < want ? (unsigned)(keys[i] & 0xffffffffull) : TK_INVALID;
}

}  // namespace

extern "C" int32_t inf_dsa_scores(inf_ctx* ctx, const float* q, const float* weights, const float* past_keys,
                                  const float* current_key, int32_t batch, int32_t past_tokens, int32_t heads,
                                  int32_t head_dim, float* scores) {
    INF_CHECK_CTX(ctx);
    if (!q || !weights || !current_key || !scores || (past_tokens > 0 && !past_keys))
        return inf_fail(ctx, INF_E_ARG, "dsa_scores: null pointer");
    if (batch <= 0 || past_tokens < 0 || heads <= 0 || head_dim <= 0)
        return inf_fail(ctx, INF_E_SHAPE, "dsa_scores: sizes must be positive");
    if (head_dim % 4 != 0) return inf_fail(ctx, INF_E_SHAPE, "dsa_scores: head_dim %d must be a multiple of 4", head_dim);
    if (batch > 65535) return inf_fail(ctx, INF_E_SHAPE, "dsa_scores: batch %d exceeds the launch grid", batch);
    const size_t smem = ((size_t)SC_TOKENS * (head_dim + 4) + (size_t)heads * head_dim + heads + SC_HG * SC_TOKENS) * sizeof(float);
    if (smem > 200 * 1024) return INF_UNSUPPORTED;
    if (smem > 48 * 1024 && !(ctx->func_attr_done & 4096u)) {
        INF_CUDA(ctx, cudaFuncSetAttribute(dsa_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        ctx->func_attr_done |= 4096u;
    }
    dim3 grid((past_tokens + 1 + SC_TOKENS - 1) / SC_TOKENS, batch);
    {
        inf_prof_scope prof(ctx, "dsa_scores_kernel");
        INF_CUDA(ctx, inf_launch_pdl(dsa_scores_kernel, grid, dim3(SC_THREADS), smem, ctx->stream, q, weights, past_keys,
                                     current_key, scores, past_tokens, heads, head_dim));
    }
    return INF_OK;
}

extern "C" int32_t inf_dsa_topk(inf_ctx* ctx, const float* scores, int32_t batch, int32_t key_tokens, int32_t top_k,
                                uint32_t* selected, int32_t selected_stride) {
    INF_CHECK_CTX(ctx);
    if (!scores || !selected) return inf_fail(ctx, INF_E_ARG, "dsa_topk: null pointer");
    if (batch <= 0 || key_tokens <= 0 || top_k <= 0 || selected_stride < top_k)
        return inf_fail(ctx, INF_E_SHAPE, "dsa_topk: sizes must be positive and the stride at least top_k");
    if (top_k > TK_MAX_K) return INF_UNSUPPORTED;
    {
        inf_prof_scope prof(ctx, "dsa_topk_kernel");
        const int in_smem = key_tokens <= TK_SMEM_ROWS ? 1 : 0;
        const size_t smem = in_smem ? (size_t)key_tokens * sizeof(unsigned) : 0;
        if (smem > 48 * 1024 && !(ctx->func_attr_done & 8192u)) {
            INF_CUDA(ctx, cudaFuncSetAttribute(dsa_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               TK_SMEM_ROWS * (int)sizeof(unsigned)));
            ctx->func_attr_done |= 8192u;
        }
        INF_CUDA(ctx, inf_launch_pdl(dsa_topk_kernel, dim3(batch), dim3(TK_THREADS), smem, ctx->stream, scores, selected,
                                     key_tokens, top_k, selected_stride, in_smem));
    }
    return INF_OK;
}

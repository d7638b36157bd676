// DSA indexer for sparse decode: per-token index scores and the top-k selection that feeds
// inf_mla_decode_absorbed_selected.  Reference: dsa_scores_f32_kernel and dsa_topk_block_sort / dsa_topk_merge
// (crates/backend/src/metal/kernels/dsa_kernels.metal:137-176, 178-393).
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>

#include "common.cuh"
#include "ptx.cuh"

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

// The same scores on the tensor cores (tcgen05, kind::tf32), for 128-dim keys and head counts that are multiples of
// 16.  The register-blocked kernel above spends ~8 us of fp32 multiply-adds per launch at 32 768 tokens; a 128-token
// tile is 32 MMAs here.  fp32 inputs are split into two tf32 terms (hi = x with the 13 low mantissa bits cleared,
// lo = x - hi, exact) and each product is taken as hi*hi + hi*lo + lo*hi with fp32 accumulation, which keeps the error
// of a dot product near 2^-20 of its magnitude: as good as the fp32 reference sum, whose own rounding depends on the
// order of addition.  The tensor core reads only the 19 leading bits of a tf32 operand, so the key tile as it landed
// is its own hi term and only the lo tile is written (q's hi term is stored masked); the accuracy test against exact
// arithmetic would fail by two orders of magnitude if an operand were rounded instead.
//
// A CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  Key tiles arrive by TMA (the f32 rows described to the
// copy engine as twice as many 16-bit values; K-major, 128-byte swizzle: four blocks of 32 dims).  Warps 0-3 split a
// landed tile block by block (the lo terms into a tile of their own), and hand each block to warp 4 as soon as
// it is done; warp 4 issues, per 8 dims, hi x [q_hi; q_lo] (N = 2 x heads) and lo x q_hi (N = heads) into a
// [128 tokens x 2 heads] fp32 accumulator in tensor memory.  The same four warps then read their token's row back, add
// the two halves, apply scale, relu and the head weights, and store the score.  With two key buffers the next tile's
// copy is in flight during all of that.
constexpr int TU_TOKENS = 128;
constexpr int TU_DIM = 128;
constexpr int TU_WORKERS = 128;
constexpr int TU_THREADS = TU_WORKERS + 32;
constexpr int TU_KEY_TILE = TU_TOKENS * TU_DIM * 4;  // 64 KB: four 128-byte-wide blocks of 128 rows
constexpr int TU_BLOCK = TU_TOKENS * 128;             // one block of a key tile

__host__ __device__ constexpr uint32_t umma_idesc_tf32(uint32_t M, uint32_t N) {  // tf32 A/B, K-major both, fp32 accumulation
    return (1u << 4) | (2u << 7) | (2u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
__device__ __forceinline__ void umma_ss_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// x = hi + lo exactly; hi has at most 11 significant bits
__device__ __forceinline__ void tf32_split(const float4& v, uint4& hi, float4& lo) {
    hi.x = __float_as_uint(v.x) & 0xffffe000u, hi.y = __float_as_uint(v.y) & 0xffffe000u;
    hi.z = __float_as_uint(v.z) & 0xffffe000u, hi.w = __float_as_uint(v.w) & 0xffffe000u;
    lo.x = v.x - __uint_as_float(hi.x), lo.y = v.y - __uint_as_float(hi.y);
    lo.z = v.z - __uint_as_float(hi.z), lo.w = v.w - __uint_as_float(hi.w);
}

__global__ void __launch_bounds__(TU_THREADS, 1)
dsa_scores_umma_kernel(const __grid_constant__ CUtensorMap tm_keys, const float* __restrict__ q,
                       const float* __restrict__ weights, const float* __restrict__ current_key,
                       float* __restrict__ scores, int past, int heads, int nbuf, int tmem_cols, int* status) {
    extern __shared__ __align__(1024) uint8_t usm[];
    __shared__ uint64_t k_full[2], a_ready[4], mma_done;
    __shared__ uint32_t tmem_slot;
    using namespace inf;
    uint8_t* s_lo = usm;                                 // lo terms of the tile being multiplied
    uint8_t* s_key = usm + TU_KEY_TILE;                  // nbuf key tiles as they landed
    uint8_t* s_q = s_key + (size_t)nbuf * TU_KEY_TILE;    // four blocks of [q_hi: heads rows; q_lo: heads rows][128 bytes]
    float* s_w = reinterpret_cast<float*>(s_q + (size_t)2 * heads * TU_DIM * 4);  // [heads]
    const int b = blockIdx.y, n = past + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tiles = (n + TU_TOKENS - 1) / TU_TOKENS;
    if (tid == 0) {
        mbar_init(&k_full[0], 1);
        mbar_init(&k_full[1], 1);
        for (int i = 0; i < 4; ++i) mbar_init(&a_ready[i], TU_WORKERS);
        mbar_init(&mma_done, 1);
        mbar_fence_init();
    }
    if (warp == 4) {
        tmem_alloc(&tmem_slot, (uint32_t)tmem_cols);
        tmem_relinquish();
    }
    inf_pdl_wait();
    inf_pdl_release();
    __syncthreads();
    auto load_tile = [&](int tile, int buf) {  // one thread; rows past the end of the tensor arrive as zeros
        mbar_arrive_expect_tx(&k_full[buf], TU_KEY_TILE);
        const int row = b * past + tile * TU_TOKENS;
#pragma unroll
        for (int blk = 0; blk < 4; ++blk)
            tma_load_2d(s_key + buf * TU_KEY_TILE + blk * TU_BLOCK, &tm_keys, blk * 64, row, &k_full[buf]);
    };
    if (tid == 0)
        for (int i = 0; i < nbuf; ++i)
            if ((int)(blockIdx.x + i * gridDim.x) < tiles) load_tile(blockIdx.x + i * gridDim.x, i);
    if (warp < 4) {
        // q: hi and lo terms in the same swizzled K-major layout, 2 x heads rows per 128-byte block
        for (int i = tid; i < heads * (TU_DIM / 4); i += TU_WORKERS) {
            const int h = i >> 5, qc = i & 31;
            const float4 v = reinterpret_cast<const float4*>(q + ((size_t)b * heads + h) * TU_DIM)[qc];
            uint4 hi;
            float4 lo;
            tf32_split(v, hi, lo);
            uint8_t* blk = s_q + (size_t)(qc >> 3) * 2 * heads * 128;
            *reinterpret_cast<uint4*>(blk + h * 128 + (((qc & 7) ^ (h & 7)) << 4)) = hi;
            *reinterpret_cast<float4*>(blk + (heads + h) * 128 + (((qc & 7) ^ ((heads + h) & 7)) << 4)) = lo;
        }
        for (int i = tid; i < heads; i += TU_WORKERS) s_w[i] = weights[(size_t)b * heads + i];
        fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    const float scale = rsqrtf((float)TU_DIM);
    if (warp < 4) {
        // this thread's share of every block: 16-byte chunk c8 of rows rbase, rbase + 16, ...
        const int c8 = tid & 7, rbase = tid >> 3;
        int i = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++i) {
            const int buf = nbuf == 2 ? (i & 1) : 0;
            uint8_t* cur = s_key + buf * TU_KEY_TILE;
            int ok = mbar_wait(&k_full[buf], (uint32_t)((nbuf == 2 ? (i >> 1) : i) & 1));
            const int cur_row = past - tile * TU_TOKENS;  // where the current key goes, if it is in this tile
#pragma unroll 1
            for (int blk = 0; ok && blk < 4; ++blk) {
                float4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int r = rbase + 16 * j;
                    v[j] = *reinterpret_cast<const float4*>(cur + blk * TU_BLOCK + r * 128 + ((c8 ^ (r & 7)) << 4));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int r = rbase + 16 * j;
                    const uint32_t off = (uint32_t)(blk * TU_BLOCK + r * 128 + ((c8 ^ (r & 7)) << 4));
                    if (r == cur_row) {
                        v[j] = reinterpret_cast<const float4*>(current_key + (size_t)b * TU_DIM)[blk * 8 + c8];
                        *reinterpret_cast<float4*>(cur + off) = v[j];
                    }
                    uint4 hi;
                    float4 lo;
                    tf32_split(v[j], hi, lo);
                    *reinterpret_cast<float4*>(s_lo + off) = lo;  // the raw tile serves as hi: see the kernel's header
                }
                fence_proxy_async_smem();
                mbar_arrive(&a_ready[blk]);
            }
            if (ok) ok = mbar_wait(&mma_done, (uint32_t)(i & 1));
            if (!ok) {
                atomicOr(status, INF_STATUS_WAIT_TIMEOUT);
                break;
            }
            tc_fence_after();
            if (tid == 0 && tile + nbuf * (int)gridDim.x < tiles) load_tile(tile + nbuf * gridDim.x, buf);  // the buffer is free
            __syncwarp();
            float sum = 0.f;
            const uint32_t trow = tbase + ((uint32_t)(warp * 32) << 16);
            for (int h0 = 0; h0 < heads; h0 += 16) {
                uint32_t d[16], e[16];
                tmem_ld16(trow + (uint32_t)h0, d);            // hi x q_hi + lo x q_hi
                tmem_ld16(trow + (uint32_t)(heads + h0), e);  // hi x q_lo
                tc_wait_ld();
#pragma unroll
                for (int x = 0; x < 16; ++x)
                    sum = fmaf(s_w[h0 + x], fmaxf((__uint_as_float(d[x]) + __uint_as_float(e[x])) * scale, 0.f), sum);
            }
            tc_fence_before();  // the row is in registers before the next hand-over lets the accumulator be overwritten
            const int tok = tile * TU_TOKENS + tid;
            if (tok < n) scores[(size_t)b * n + tok] = sum;
        }
    } else if (lane == 0) {
        const uint32_t idesc_wide = umma_idesc_tf32(TU_TOKENS, (uint32_t)(2 * heads));
        const uint32_t idesc_narrow = umma_idesc_tf32(TU_TOKENS, (uint32_t)heads);
        const uint32_t lo_addr = smem_u32(s_lo), q_addr = smem_u32(s_q);
        int i = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++i) {
            const uint32_t hi_addr = smem_u32(s_key + (nbuf == 2 ? (i & 1) : 0) * TU_KEY_TILE);
            int ok = 1;
            for (int blk = 0; ok && blk < 4; ++blk) {
                ok = mbar_wait(&a_ready[blk], (uint32_t)(i & 1));
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {  // eight tf32 values = 32 bytes per step, four steps per block
                    const uint32_t a_off = (uint32_t)(blk * TU_BLOCK + ks * 32);
                    const uint64_t a_hi = umma_smem_desc(hi_addr + a_off, 16, 1024, UMMA_SW128);
                    const uint64_t a_lo = umma_smem_desc(lo_addr + a_off, 16, 1024, UMMA_SW128);
                    const uint64_t b_q = umma_smem_desc(q_addr + (uint32_t)(blk * 2 * heads * 128 + ks * 32), 16, 1024, UMMA_SW128);
                    umma_ss_tf32(tbase, a_hi, b_q, idesc_wide, (blk | ks) != 0);  // [hi.q_hi | hi.q_lo]
                    umma_ss_tf32(tbase, a_lo, b_q, idesc_narrow, 1u);             // + lo.q_hi on the first half
                }
            }
            if (!ok) {
                atomicOr(status, INF_STATUS_WAIT_TIMEOUT);
                break;
            }
            tc_commit(&mma_done);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tbase, (uint32_t)tmem_cols);
}

// ---------------------------------------------------------------------------------------------- preparation
// The two small operators in front of the scores: the index key of new tokens (LayerNorm over the key, then rotary
// position encoding of the first rope_dim values, interleaved pairs in, halves out) and, per decode step, the query
// heads under the same rotation plus the per-head weights hidden . weights_proj / sqrt(heads).  Semantics follow the
// reference's CPU indexer (crates/model/src/indexer.rs:174-203 key, :397-428 LayerNorm, :483-514 rotation, :516-543
// weights), which rotates out of a temporary; its Metal kernel for the key (dsa_kernels.metal:23-81) rotates in
// place and reads values it has already replaced once rope_dim >= 4, so it is not the model followed here.
struct DsaFreq {
    float v[64];  // 1 / theta^(pair / pair_count), computed on the host
};

__device__ __forceinline__ void dsa_rotate(float x0, float x1, float angle, float& out0, float& out1) {
    const float c = cosf(angle), s = sinf(angle);
    out0 = x0 * c - x1 * s;
    out1 = x1 * c + x0 * s;
}

// one warp per key row; head_dim <= 1024
__global__ void __launch_bounds__(128)
dsa_index_key_kernel(const float* __restrict__ raw, const float* __restrict__ weight, const float* __restrict__ bias,
                     float* __restrict__ out, long long rows, int tokens, int head_dim, int rope_dim, int position_offset,
                     float eps, DsaFreq f) {
    extern __shared__ float s_rows[];  // [4 warps][head_dim] normalised rows
    inf_pdl_wait();
    inf_pdl_release();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * 4 + warp;
    if (row >= rows) return;
    const float* x = raw + row * head_dim;
    float* y = s_rows + warp * head_dim;
    float sum = 0.f;
    for (int d = lane; d < head_dim; d += 32) sum += x[d];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / (float)head_dim;
    float var = 0.f;
    for (int d = lane; d < head_dim; d += 32) {
        const float c = x[d] - mean;
        var += c * c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
    const float inv_std = 1.0f / sqrtf(var / (float)head_dim + eps);
    for (int d = lane; d < head_dim; d += 32) y[d] = (x[d] - mean) * inv_std * weight[d] + bias[d];
    __syncwarp();
    const int pairs = rope_dim / 2;
    const int position = position_offset + (int)(row % tokens);
    float* o = out + row * head_dim;
    for (int p = lane; p < pairs; p += 32) {
        float a, b;
        dsa_rotate(y[2 * p], y[2 * p + 1], (float)position * f.v[p], a, b);
        o[p] = a;
        o[pairs + p] = b;
    }
    for (int d = rope_dim + lane; d < head_dim; d += 32) o[d] = y[d];
}

// one CTA of 256 threads per sequence: the weights (eight warps share the hidden dimension, lane = head within a
// group of 32), then the rotated query heads
__global__ void __launch_bounds__(256)
dsa_query_weights_kernel(const float* __restrict__ hidden, const float* __restrict__ q_raw, const float* __restrict__ proj,
                         float* __restrict__ q_out, float* __restrict__ w_out, int hidden_size, int heads, int head_dim,
                         int rope_dim, int position, DsaFreq f) {
    __shared__ float part[8][32];
    inf_pdl_wait();
    inf_pdl_release();
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* h = hidden + (size_t)b * hidden_size;
    const int per = (hidden_size + 7) / 8, d0 = warp * per, d1 = min(hidden_size, d0 + per);
    for (int h0 = 0; h0 < heads; h0 += 32) {
        const int head = h0 + lane;
        float acc = 0.f;
        if (head < heads)
            for (int d = d0; d < d1; ++d) acc = fmaf(h[d], proj[(size_t)d * heads + head], acc);
        part[warp][lane] = acc;
        __syncthreads();
        if (warp == 0 && head < heads) {
            float total = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) total += part[w][lane];
            w_out[(size_t)b * heads + head] = total * (1.0f / sqrtf((float)heads));
        }
        __syncthreads();
    }
    const int pairs = rope_dim / 2;
    const float* q = q_raw + (size_t)b * heads * head_dim;
    float* o = q_out + (size_t)b * heads * head_dim;
    for (int i = tid; i < heads * head_dim; i += 256) {
        const int head = i / head_dim, d = i % head_dim;
        if (d >= rope_dim) {
            o[i] = q[i];
        } else if (d < pairs) {  // this thread produces both outputs of pair d
            float a, c;
            dsa_rotate(q[head * head_dim + 2 * d], q[head * head_dim + 2 * d + 1], (float)position * f.v[d], a, c);
            o[head * head_dim + d] = a;
            o[head * head_dim + pairs + d] = c;
        }
    }
}

void dsa_host_freq(float theta, int rope_dim, DsaFreq* f) {
    const int pairs = rope_dim / 2;
    for (int p = 0; p < 64; ++p) f->v[p] = p < pairs ? 1.0f / powf(theta, (float)(2 * p) / (float)rope_dim) : 0.0f;
}

// ---------------------------------------------------------------------------------------------- top-k
// ids of the k best tokens, best first, where a precedes b iff score_a > score_b or (score_a == score_b and
// id_a < id_b) (dsa_precedes, dsa_kernels.metal:182-196); missing entries are 0xffffffff.  The reference sorts
// 256-token blocks and merges runs; here one CTA per sequence finds the k-th largest score with a three-pass radix
// select (12 + 10 + 10 bits) over the order-preserving integer image of the scores, collects everything above it
// plus the lowest-id ties in id order, and sorts those k entries by score with a stable counting sort in shared memory.
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
// The k-th largest value is found 12 + 10 + 10 bits at a time: twelve leading bits spread real scores (a few
// exponents, sixteen mantissa steps each) over enough bins that the shared-memory adds of a warp rarely meet.
constexpr int TK_SMEM_ROWS = 45056;  // 176 KB of ordered scores
constexpr int TK_CAND_CAP = 2 * TK_THREADS;  // candidates of the threshold bin that are kept as a list
constexpr int TK_WARPS = TK_THREADS / 32;
constexpr int TK_BINS = 4096;
constexpr int TK_SORT_TABLE_BYTES = TK_WARPS * 256 * (int)sizeof(unsigned);
static_assert(TK_BINS * sizeof(unsigned) == TK_MAX_K * sizeof(unsigned long long), "the histogram doubles as the sort's second buffer");
constexpr int TK_LOAD_DEPTH = 8;  // 16-byte global loads in flight per thread while the row comes in

// the lanes of the warp that hold the same eight-bit digit, one vote per bit
__device__ __forceinline__ unsigned tk_same_digit_lanes(unsigned digit) {
    unsigned lanes = 0xffffffffu;
#pragma unroll
    for (int bit = 0; bit < 8; ++bit) {
        const bool set = (digit >> bit) & 1u;
        const unsigned vote = __ballot_sync(0xffffffffu, set);
        lanes &= set ? vote : ~vote;
    }
    return lanes;
}

__global__ void __launch_bounds__(TK_THREADS)
dsa_topk_kernel(const float* __restrict__ scores, unsigned* __restrict__ out_ids, int n, int k, int out_stride,
                int row_in_smem) {
    extern __shared__ __align__(16) unsigned srow[];
    __shared__ __align__(16) unsigned hist[TK_BINS];
    __shared__ unsigned sort_part[4][256];
    __shared__ unsigned long long keys[TK_MAX_K];
    __shared__ int w_above[TK_WARPS], w_tie[TK_WARPS];
    __shared__ unsigned sh_prefix, sh_mask, sh_any, sh_all;
    __shared__ int sh_remaining, sh_cand;
    __shared__ unsigned cand_ids[TK_CAND_CAP];
    inf_pdl_wait();
    inf_pdl_release();
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = scores + (size_t)b * n;
    unsigned* out = out_ids + (size_t)b * out_stride;
    const int want = min(k, n);
    auto value = [&](int i) -> unsigned { return row_in_smem ? srow[i] : ordered_bits(row[i]); };
    for (int i = tid; i < TK_MAX_K; i += TK_THREADS) keys[i] = ~0ull;
    if (tid == 0) {
        sh_prefix = 0u;
        sh_mask = 0u;
        sh_any = 0u;
        sh_all = ~0u;
        sh_remaining = want;
    }
    // ---- collect everything above the threshold and the ties with the lowest ids.  In each round thread t owns
    //      the 32 consecutive tokens [round + 32t, round + 32t + 32): it records which are above and which tie as
    //      two bit masks, a scan over the CTA gives its place in the output, and it writes its own entries.  Lane l
    //      starts its walk at element l of its chunk, so the 32 lanes of a warp hit 32 different banks.
    int out_base = 0, ties_before = 0;  // the same in every thread
    // exclusive places of this thread's (above, tie) counts among all threads, and the totals; one barrier inside
    auto scan_counts = [&](int ca, int ct, int& ex_a, int& ex_t, int& total_a, int& total_t) {
        int ia = ca, it = ct;  // inclusive scans inside the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int ya = __shfl_up_sync(0xffffffffu, ia, o), yt = __shfl_up_sync(0xffffffffu, it, o);
            if (lane >= o) {
                ia += ya;
                it += yt;
            }
        }
        if (lane == 31) {
            w_above[warp] = ia;
            w_tie[warp] = it;
        }
        __syncthreads();
        int wa = w_above[lane], wt = w_tie[lane];  // every warp scans the 32 warp totals for itself
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int ya = __shfl_up_sync(0xffffffffu, wa, o), yt = __shfl_up_sync(0xffffffffu, wt, o);
            if (lane >= o) {
                wa += ya;
                wt += yt;
            }
        }
        total_a = __shfl_sync(0xffffffffu, wa, 31);
        total_t = __shfl_sync(0xffffffffu, wt, 31);
        const int warp_a = warp ? __shfl_sync(0xffffffffu, wa, (warp + 31) & 31) : 0;  // totals of the warps before
        const int warp_t = warp ? __shfl_sync(0xffffffffu, wt, (warp + 31) & 31) : 0;
        ex_a = warp_a + ia - ca;  // entries of earlier threads
        ex_t = warp_t + it - ct;
    };
    // threshold and ties compare on (value >> shift).  to_list: the ties are not entries yet but candidates, all of
    // them kept (ids only, in id order) in cand_ids, ties_before counting them.
    auto sweep = [&](unsigned threshold, int shift, int ties_wanted, bool to_list) {
    for (int round = 0; round < n; round += 32 * TK_THREADS) {
        const int c = round + tid * 32;
        unsigned above_mask = 0u, tie_mask = 0u;
        if (row_in_smem && c + 32 <= n) {
            // eight 16-byte reads; bit p of the masks built here belongs to element (p + 4 * lane) mod 32
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint4 v = reinterpret_cast<const uint4*>(srow + c)[(q + lane) & 7];
                above_mask |= ((unsigned)((v.x >> shift) > threshold) << (4 * q)) | ((unsigned)((v.y >> shift) > threshold) << (4 * q + 1)) |
                              ((unsigned)((v.z >> shift) > threshold) << (4 * q + 2)) | ((unsigned)((v.w >> shift) > threshold) << (4 * q + 3));
                tie_mask |= ((unsigned)((v.x >> shift) == threshold) << (4 * q)) | ((unsigned)((v.y >> shift) == threshold) << (4 * q + 1)) |
                            ((unsigned)((v.z >> shift) == threshold) << (4 * q + 2)) | ((unsigned)((v.w >> shift) == threshold) << (4 * q + 3));
            }
            above_mask = __funnelshift_l(above_mask, above_mask, 4 * lane);
            tie_mask = __funnelshift_l(tie_mask, tie_mask, 4 * lane);
        } else if (c < n) {
            for (int j = 0; j < 32; ++j) {
                const int jj = (j + lane) & 31;
                if (c + jj < n) {
                    const unsigned u = value(c + jj) >> shift;
                    above_mask |= (unsigned)(u > threshold) << jj;
                    tie_mask |= (unsigned)(u == threshold) << jj;
                }
            }
        }
        const int ca = __popc(above_mask), ct = __popc(tie_mask);
        int ex_a, ex_t, round_above, round_ties;
        scan_counts(ca, ct, ex_a, ex_t, round_above, round_ties);
        const int ties_open = max(ties_wanted - ties_before, 0);     // ties this pass may still take
        const int quota = max(0, min(ct, ties_open - ex_t));
        unsigned take = tie_mask;
        if (quota < ct) {  // the lowest `quota` ids of this thread's ties
            take = 0u;
            unsigned m = tie_mask;
            for (int x = 0; x < quota; ++x) {
                const unsigned low = m & (0u - m);
                take |= low;
                m ^= low;
            }
        }
        int pos = out_base + ex_a + (to_list ? 0 : min(ties_open, ex_t));
        unsigned sel = to_list ? above_mask : (above_mask | take);
        while (sel) {
            const int jj = __ffs(sel) - 1;
            sel &= sel - 1u;
            const int i = c + jj;
            keys[pos++] = ((unsigned long long)(~value(i)) << 32) | (unsigned)i;
        }
        if (to_list) {
            int at = ties_before + ex_t;
            unsigned m = tie_mask;
            while (m) {
                const int jj = __ffs(m) - 1;
                m &= m - 1u;
                cand_ids[at++] = (unsigned)(c + jj);
            }
        }
        out_base += round_above + (to_list ? 0 : min(ties_open, round_ties));
        ties_before += round_ties;
        __syncthreads();
    }
    };
    bool compact = false;  // the threshold bin's members have been few enough to be kept as a list
    int cand_n = 0;
    const int n4 = n >> 2;  // whole groups of four scores
    for (int pass = 0; pass < 3; ++pass) {
        const int shift = pass == 0 ? 20 : (pass == 1 ? 10 : 0);
        const int bins = pass == 0 ? TK_BINS : 1024;
        for (int i = tid; i < bins; i += TK_THREADS) hist[i] = 0u;
        __syncthreads();
        const unsigned prefix = sh_prefix, mask = sh_mask, digit_mask = (unsigned)bins - 1u;
        if (pass > 0 && compact) {
            for (int i = tid; i < cand_n; i += TK_THREADS) {
                const unsigned u = value((int)cand_ids[i]);
                if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & digit_mask], 1u);
            }
        } else if (pass == 0 && row_in_smem && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
            // The first pass also brings the row into shared memory, TK_LOAD_DEPTH groups of four per thread at a
            // time.  A warp whose 128 scores all share one digit (constant rows, padding) adds once.
            for (int base = warp * 32; base < n4; base += TK_THREADS * TK_LOAD_DEPTH) {
                float4 f[TK_LOAD_DEPTH];
#pragma unroll
                for (int d = 0; d < TK_LOAD_DEPTH; ++d) {
                    const int v = base + d * TK_THREADS + lane;
                    if (v < n4) f[d] = reinterpret_cast<const float4*>(row)[v];
                }
#pragma unroll
                for (int d = 0; d < TK_LOAD_DEPTH; ++d) {
                    const int v = base + d * TK_THREADS + lane;
                    if (base + d * TK_THREADS >= n4) break;  // the whole warp is past the end
                    const bool valid = v < n4;
                    uint4 q = make_uint4(0u, 0u, 0u, 0u);
                    if (valid) {
                        q = make_uint4(ordered_bits(f[d].x), ordered_bits(f[d].y), ordered_bits(f[d].z), ordered_bits(f[d].w));
                        reinterpret_cast<uint4*>(srow)[v] = q;
                    }
                    const unsigned d0 = q.x >> 20, d1 = q.y >> 20, d2 = q.z >> 20, d3 = q.w >> 20;
                    const unsigned first = __shfl_sync(0xffffffffu, d0, 0);  // lane 0 is valid whenever the warp is here
                    const bool same = !valid || (d0 == first && d1 == first && d2 == first && d3 == first);
                    if (__all_sync(0xffffffffu, same)) {
                        const unsigned live = __ballot_sync(0xffffffffu, valid);
                        if (lane == 0) atomicAdd(&hist[first], 4u * (unsigned)__popc(live));
                    } else if (valid) {
                        atomicAdd(&hist[d0], 1u);
                        atomicAdd(&hist[d1], 1u);
                        atomicAdd(&hist[d2], 1u);
                        atomicAdd(&hist[d3], 1u);
                    }
                }
            }
            if (n4 * 4 + tid < n) {
                const unsigned u = ordered_bits(row[n4 * 4 + tid]);
                srow[n4 * 4 + tid] = u;
                atomicAdd(&hist[u >> 20], 1u);
            }
        } else if (pass == 0 || !row_in_smem) {
            for (int i = tid; i < n; i += TK_THREADS) {
                const unsigned u = ordered_bits(row[i]);
                if (pass == 0 && row_in_smem) srow[i] = u;
                if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & digit_mask], 1u);
            }
        } else {
            for (int v = tid; v < n4; v += TK_THREADS) {
                const uint4 q = reinterpret_cast<const uint4*>(srow)[v];
                if ((q.x & mask) == prefix) atomicAdd(&hist[(q.x >> shift) & digit_mask], 1u);
                if ((q.y & mask) == prefix) atomicAdd(&hist[(q.y >> shift) & digit_mask], 1u);
                if ((q.z & mask) == prefix) atomicAdd(&hist[(q.z >> shift) & digit_mask], 1u);
                if ((q.w & mask) == prefix) atomicAdd(&hist[(q.w >> shift) & digit_mask], 1u);
            }
            if (n4 * 4 + tid < n) {
                const unsigned u = srow[n4 * 4 + tid];
                if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & digit_mask], 1u);
            }
        }
        __syncthreads();
        {
            // The bin that holds the remaining-th largest candidate.  Thread t owns `per` consecutive bins; the
            // candidates in bins above a thread come from a suffix sum over the CTA, the owner then walks its bins.
            const int per = bins / TK_THREADS;  // 4 or 1
            const int remaining = sh_remaining;
            int mine[TK_BINS / TK_THREADS], sum = 0;
#pragma unroll
            for (int i = 0; i < TK_BINS / TK_THREADS; ++i) {
                mine[i] = i < per ? (int)hist[tid * per + i] : 0;
                sum += mine[i];
            }
            int suffix = sum;  // inclusive suffix sum over the lanes of this warp
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_down_sync(0xffffffffu, suffix, o);
                if (lane + o < 32) suffix += y;
            }
            if (lane == 0) w_above[warp] = suffix;
            __syncthreads();
            int warps = w_above[lane];  // inclusive suffix sum over the warps
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_down_sync(0xffffffffu, warps, o);
                if (lane + o < 32) warps += y;
            }
            const int next_warp = __shfl_sync(0xffffffffu, warps, (warp + 1) & 31);
            const int above = (warp < 31 ? next_warp : 0) + suffix - sum;  // candidates in bins of later threads
            if (above < remaining && remaining <= above + sum) {
                int left = remaining - above, bin = per - 1;
                for (; bin > 0; --bin) {
                    if (mine[bin] >= left) break;
                    left -= mine[bin];
                }
                sh_prefix = prefix | ((unsigned)(tid * per + bin) << shift);
                sh_mask = mask | (digit_mask << shift);
                sh_remaining = left;  // how many entries equal to the final value are taken
                sh_cand = mine[bin];   // members of the chosen bin
            }
        }
        __syncthreads();
        if (!compact && pass < 2 && sh_cand <= TK_CAND_CAP) {
            // Few members in the threshold bin (after the first pass for widely spread scores, after the second for
            // scores that share their leading bits): one sweep writes everything in higher bins as entries and lists
            // the bin's members; the remaining passes and the final choice then touch only that list.
            compact = true;
            sweep(sh_prefix >> shift, shift, 0x7fffffff, true);
            cand_n = ties_before;
        }
    }
    const unsigned threshold = sh_prefix;
    const int ties_wanted = sh_remaining;
    // ---- collect everything above the threshold and the ties with the lowest ids.  In each round thread t owns
    //      the 32 consecutive tokens [round + 32t, round + 32t + 32): it records which are above and which tie as
    //      two bit masks, a scan over the CTA gives its place in the output, and it writes its own entries.  Lane l
    //      starts its walk at element l of its chunk, so the 32 lanes of a warp hit 32 different banks.
    if (!compact) {
        sweep(threshold, 0, ties_wanted, false);
    } else {  // the same choice among the listed candidates, two consecutive ones per thread
        unsigned u[2] = {0u, 0u}, id[2] = {0u, 0u};
        bool above[2] = {false, false}, tie[2] = {false, false};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int i = 2 * tid + e;
            if (i < cand_n) {
                id[e] = cand_ids[i];
                u[e] = value((int)id[e]);
                above[e] = u[e] > threshold;
                tie[e] = u[e] == threshold;
            }
        }
        int ex_a, ex_t, total_a, total_t;
        scan_counts((int)above[0] + (int)above[1], (int)tie[0] + (int)tie[1], ex_a, ex_t, total_a, total_t);
        int pos = out_base + ex_a + min(ties_wanted, ex_t), ties_seen = ex_t;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (above[e] || (tie[e] && ties_seen < ties_wanted)) keys[pos++] = ((unsigned long long)(~u[e]) << 32) | id[e];
            ties_seen += (int)tie[e];
        }
        __syncthreads();
    }
    // ---- sort of the 2048 entries, best first.  The sweep above wrote them in id order, so a stable sort on the score
    //      word alone gives the reference's order (ties by lower id; the all-ones padding stays last).  Four stable
    //      counting passes of eight bits: warp w owns entries 64w .. 64w+63, counts their digits in its own row of a
    //      32 x 256 table (the dead row buffer), a scan over bins and warps turns counts into places, each entry moves.
    const unsigned long long* sorted;
    {
        unsigned long long* from = keys;
        unsigned long long* to = reinterpret_cast<unsigned long long*>(hist);  // TK_BINS words = TK_MAX_K entries
        unsigned* table = srow;
        unsigned* my_row = table + warp * 256;
        const unsigned lanes_below = (1u << lane) - 1u;
        const int group = tid >> 8, bin = tid & 255;  // scan roles: 4 groups of 8 warps x 256 bins
        // score bits that are the same in every real entry need no pass (the leading byte of the best scores of a
        // long row usually is): a skipped pass would have moved nothing, the padding already sits last
        {
            const int e = warp * 64 + lane;
            const unsigned h0 = (unsigned)(keys[e] >> 32), h1 = (unsigned)(keys[e + 32] >> 32);
            unsigned any = (e < want ? h0 : 0u) | (e + 32 < want ? h1 : 0u);
            unsigned all = (e < want ? h0 : ~0u) & (e + 32 < want ? h1 : ~0u);
            any = __reduce_or_sync(0xffffffffu, any);
            all = __reduce_and_sync(0xffffffffu, all);
            if (lane == 0) {
                atomicOr(&sh_any, any);
                atomicAnd(&sh_all, all);
            }
            __syncthreads();
        }
        const unsigned varying = sh_any ^ sh_all;
        for (int pass = 0; pass < 4; ++pass) {
            if (((varying >> (8 * pass)) & 255u) == 0u) continue;
            const int shift = 32 + 8 * pass;
            for (int i = tid; i < TK_WARPS * 256; i += TK_THREADS) table[i] = 0u;
            __syncthreads();
            const unsigned long long x0 = from[warp * 64 + lane], x1 = from[warp * 64 + 32 + lane];
            const unsigned d0 = (unsigned)(x0 >> shift) & 255u, d1 = (unsigned)(x1 >> shift) & 255u;
            const unsigned m0 = tk_same_digit_lanes(d0);
            const unsigned r0 = (unsigned)__popc(m0 & lanes_below);
            if ((m0 & lanes_below) == 0u) my_row[d0] = (unsigned)__popc(m0);
            __syncwarp();
            const unsigned m1 = tk_same_digit_lanes(d1);
            const unsigned before = my_row[d1];  // entries with this digit among the warp's first 32
            const unsigned r1 = before + (unsigned)__popc(m1 & lanes_below);
            __syncwarp();
            if ((m1 & lanes_below) == 0u) my_row[d1] = before + (unsigned)__popc(m1);
            __syncthreads();
            {  // counts of one bin over the 8 warps of a group -> places inside the group, group total aside
                unsigned run = 0u;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    unsigned* cell = table + (group * 8 + w) * 256 + bin;
                    const unsigned c = *cell;
                    *cell = run;
                    run += c;
                }
                sort_part[group][bin] = run;
            }
            __syncthreads();
            unsigned p0 = 0u, p1 = 0u, p2 = 0u, total = 0u, incl = 0u;
            if (tid < 256) {
                p0 = sort_part[0][tid], p1 = sort_part[1][tid], p2 = sort_part[2][tid];
                total = p0 + p1 + p2 + sort_part[3][tid];
                incl = total;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned y = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += y;
                }
                if (lane == 31) w_above[warp] = (int)incl;
            }
            __syncthreads();
            if (tid < 256) {
                unsigned start = incl - total;  // entries in lower bins
                for (int w = 0; w < warp; ++w) start += (unsigned)w_above[w];
                sort_part[0][tid] = start;
                sort_part[1][tid] = start + p0;
                sort_part[2][tid] = start + p0 + p1;
                sort_part[3][tid] = start + p0 + p1 + p2;
            }
            __syncthreads();
            to[sort_part[warp >> 3][d0] + my_row[d0] + r0] = x0;
            to[sort_part[warp >> 3][d1] + my_row[d1] + r1] = x1;
            __syncthreads();
            unsigned long long* t = from;
            from = to;
            to = t;
        }
        sorted = from;
    }
    for (int i = tid; i < k; i += TK_THREADS) out[i] = i < want ? (unsigned)(sorted[i] & 0xffffffffull) : TK_INVALID;
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
    if (head_dim == TU_DIM && heads % 16 == 0 && heads <= 128 && past_tokens > 0 &&
        (reinterpret_cast<uintptr_t>(past_keys) & 15u) == 0) {
        const size_t q_bytes = (2 * (size_t)heads * TU_DIM + heads) * sizeof(float);  // hi and lo tiles, the weights
        const size_t smem_limit = 227 * 1024 - 2048;  // static shared memory and the 1 KB alignment of the tiles
        const int nbuf = (3 * (size_t)TU_KEY_TILE + q_bytes <= smem_limit) ? 2 : 1;
        const size_t smem_umma = (size_t)(1 + nbuf) * TU_KEY_TILE + q_bytes;
        if (smem_umma <= smem_limit) {
            if (ctx->dsa_scores_smem < smem_umma) {
                INF_CUDA(ctx, cudaFuncSetAttribute(dsa_scores_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_umma));
                ctx->dsa_scores_smem = smem_umma;
            }
            // the f32 key rows as 16-bit pairs: 256 per row, boxes of 64 (one 128-byte swizzle line) x 128 rows
            CUtensorMap tm_keys;
            uint64_t dims[2] = {2 * (uint64_t)TU_DIM, (uint64_t)batch * past_tokens};
            uint64_t strides[1] = {(uint64_t)TU_DIM * sizeof(float)};
            uint32_t box[2] = {64, (uint32_t)TU_TOKENS};
            int rc = inf_make_tmap(ctx, past_keys, 2, dims, strides, box, &tm_keys);
            if (rc != INF_OK) return rc;
            int tmem_cols = 32;
            while (tmem_cols < 2 * heads) tmem_cols *= 2;
            const int tiles = (past_tokens + 1 + TU_TOKENS - 1) / TU_TOKENS;
            // one CTA per SM; every CTA takes the same number of tiles where that is possible
            const int per_cta = (tiles * batch + ctx->sm_count - 1) / ctx->sm_count;
            dim3 grid((tiles + per_cta - 1) / per_cta, batch);
            inf_prof_scope prof(ctx, "dsa_scores_kernel");
            INF_CUDA(ctx, inf_launch_pdl(dsa_scores_umma_kernel, grid, dim3(TU_THREADS), smem_umma, ctx->stream, tm_keys, q,
                                         weights, current_key, scores, past_tokens, heads, nbuf, tmem_cols, ctx->status));
            return INF_OK;
        }
    }
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
        // the row when it fits; never less than the sort's 32 x 256 table, which reuses the space
        const size_t smem = max(in_smem ? (size_t)((key_tokens + 3) & ~3) * sizeof(unsigned) : (size_t)0, (size_t)TK_SORT_TABLE_BYTES);
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

extern "C" int32_t inf_dsa_index_key(inf_ctx* ctx, const float* raw_key, const float* weight, const float* bias,
                                     int32_t batch, int32_t tokens, int32_t head_dim, int32_t rope_dim,
                                     int32_t position_offset, float theta, float eps, float* out) {
    INF_CHECK_CTX(ctx);
    if (!raw_key || !weight || !bias || !out) return inf_fail(ctx, INF_E_ARG, "dsa_index_key: null pointer");
    if (batch <= 0 || tokens <= 0 || head_dim <= 0 || head_dim > 1024)
        return inf_fail(ctx, INF_E_SHAPE, "dsa_index_key: sizes must be positive and head_dim at most 1024");
    if (rope_dim % 2 != 0) return inf_fail(ctx, INF_E_CONFIG, "DSA indexer RoPE dim must be even");
    if (rope_dim < 0 || rope_dim > head_dim)
        return inf_fail(ctx, INF_E_CONFIG, "DSA indexer RoPE dim %d exceeds head dim %d", rope_dim, head_dim);
    if (rope_dim > 128) return INF_UNSUPPORTED;
    if (position_offset < 0 || !(theta > 0.f)) return inf_fail(ctx, INF_E_CONFIG, "dsa_index_key: bad position or theta");
    DsaFreq f;
    dsa_host_freq(theta, rope_dim, &f);
    const long long rows = (long long)batch * tokens;
    INF_CUDA(ctx, inf_launch_pdl(dsa_index_key_kernel, dim3((unsigned)((rows + 3) / 4)), dim3(128),
                                 (size_t)4 * head_dim * sizeof(float), ctx->stream, raw_key, weight, bias, out, rows, tokens,
                                 head_dim, rope_dim, position_offset, eps, f));
    return INF_OK;
}

extern "C" int32_t inf_dsa_query_weights(inf_ctx* ctx, const float* hidden_states, const float* q_raw,
                                         const float* weights_proj, int32_t batch, int32_t hidden_size, int32_t heads,
                                         int32_t head_dim, int32_t rope_dim, int32_t position_offset, float theta,
                                         float* q_out, float* weights_out) {
    INF_CHECK_CTX(ctx);
    if (!hidden_states || !q_raw || !weights_proj || !q_out || !weights_out)
        return inf_fail(ctx, INF_E_ARG, "dsa_query_weights: null pointer");
    if (batch <= 0 || hidden_size <= 0 || heads <= 0 || head_dim <= 0)
        return inf_fail(ctx, INF_E_SHAPE, "dsa_query_weights: sizes must be positive");
    if (rope_dim % 2 != 0) return inf_fail(ctx, INF_E_CONFIG, "DSA indexer RoPE dim must be even");
    if (rope_dim < 0 || rope_dim > head_dim)
        return inf_fail(ctx, INF_E_CONFIG, "DSA indexer RoPE dim %d exceeds head dim %d", rope_dim, head_dim);
    if (rope_dim > 128) return INF_UNSUPPORTED;
    if (position_offset < 0 || !(theta > 0.f)) return inf_fail(ctx, INF_E_CONFIG, "dsa_query_weights: bad position or theta");
    DsaFreq f;
    dsa_host_freq(theta, rope_dim, &f);
    INF_CUDA(ctx, inf_launch_pdl(dsa_query_weights_kernel, dim3(batch), dim3(256), 0, ctx->stream, hidden_states, q_raw,
                                 weights_proj, q_out, weights_out, hidden_size, heads, head_dim, rope_dim, position_offset, f));
    return INF_OK;
}

// Paged GQA decode: split-KV partial kernel + combine kernel.
//
// HBM-bound (6 flop per KV byte at 6 query heads per KV head), so the design is about
// bytes in flight: one CTA per (sequence, KV head, run of up to 2048 keys = several split-KV
// chunks); a producer warp streams
// 16-token page tiles with TMA (one tensor map over the whole pool, the page id becomes a
// row coordinate, 128-byte swizzle) through a 3-stage mbarrier ring; four consumer warps each
// take one 16-key page tile of a stage, run QK^T and PV on mma.sync with all the query heads
// of the group stacked into the 16 rows of the M dimension (K/V are read once per KV head,
// not once per query head), and keep an online softmax in registers with quad shuffles.
// The per-chunk (max, sum, acc) triples go to scratch; the combine kernel merges them,
// applies softplus(gate)/sum and writes the output.
//
// CUDA cores alone cannot keep up with HBM here: 6.5 TB/s x 6 flop/B = 39 TFLOP/s of fp32
// FMA plus as many fp16->fp32 conversions, against ~70 TFLOP/s peak; hence mma.sync.
// Reference kernels: f16_attention_kernels.metal:325-510 (segmented partial + merge).
#include <cuda_fp16.h>
#include <math.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "fp8.cuh"
#include "ptx.cuh"

using namespace inf;

namespace {

constexpr int D = 128;
constexpr int TILE_KEYS = 64;
constexpr int BLOCK_BYTES = TILE_KEYS * 128;  // one [64 keys][128 bytes] swizzled block
constexpr int CONSUMER_WARPS = 4;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int MAX_CHUNK = 2048;
constexpr float M_INIT = -1.0e30f;

// A stage holds 64 keys: fp16 pages as four blocks (K dims 0-63, K dims 64-127, V dims 0-63, V dims 64-127),
// FP8 pages as two (a 128-dim row is 128 bytes, one block each for K and V).  Either way the ring is 96 KB.
#ifndef INF_FP8_STAGES
#define INF_FP8_STAGES 3   // ring depth and resident CTAs per SM of the FP8 instantiation (build-time experiment knobs)
#define INF_FP8_CTAS 3
#endif
template <bool FP8>
struct Ring {
    static constexpr int BLOCKS = FP8 ? 2 : 4;
    static constexpr int STAGE_BYTES = BLOCKS * BLOCK_BYTES;
    static constexpr int STAGES = FP8 ? INF_FP8_STAGES : 3;
    static constexpr int BYTES = STAGES * STAGE_BYTES;
    static constexpr int V_BLOCK = FP8 ? 1 : 2;
};

struct DecodeParams {
    const __half* q;
    const int* pages;
    const int* lens;
    int max_pages, q_heads, kv_heads, group, page_size, num_pages;
    int chunk, window;
    int chunks_per_cta;  // consecutive chunks one CTA streams (chunks_per_cta * chunk <= 2048)
    int len_add;  // added to lens[b]: lets a caller that counts cached rows before the current token reuse its table
    int cur_extra;  // 1 when the current token is not among the cached keys (FP8 form): it still counts for the window
    float scale_log2;  // score scale (times the key scale of an FP8 pool) in the log2 domain
    float v_scale;     // value scale of an FP8 pool, 1 otherwise; applied to the partial accumulators
    float* part_acc;
    float* part_ml;
    int max_chunks;
    int* status;
    int drop_tile;  // diagnostic (inf_debug_drop_next_load): the producer skips this tile's loads; -1 = none
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One CTA streams a RUN of consecutive chunks of one (sequence, KV head): the producer warp keeps the TMA ring
// full across chunk boundaries while the consumers finish a chunk (merge the four warps, write its partial) and
// start the next, so the per-chunk prologue and epilogue no longer drain the loads in flight.  Partials are still
// one (max, sum, acc) triple per chunk of `chunk` keys, exactly what the combine kernel expects.
//
// FP8 pages: the same kernel with byte tiles.  mma.sync wants fp16 fragments, so bytes become fp16 pairs in
// registers (one cvt per two values).  A sum does not care in which order its terms are taken, so the fragments
// are laid out for the loads, not for the natural index order: in QK^T lane (g, qd) takes dims [32 qd, 32 qd + 32)
// of key row g, two 16-byte loads, and the query fragments are permuted the same way; in PV the lane takes dims
// [16 g, 16 g + 16) of the four key rows its P fragment covers, so accumulator column c of tile j is output dim
// 16 c + j, which the merge step undoes when it writes the partial.
template <bool FP8, int NT>
__global__ void __launch_bounds__(THREADS, (FP8 && NT == 1) ? INF_FP8_CTAS : 2)
gqa_decode_partial_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                          DecodeParams p) {
    using R = Ring<FP8>;
    constexpr int STAGES = R::STAGES, STAGE_BYTES = R::STAGE_BYTES;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES];
    __shared__ int row_y[MAX_CHUNK / 16];
    __shared__ float warp_m[CONSUMER_WARPS][16], warp_l[CONSUMER_WARPS][16];
    float* merge = reinterpret_cast<float*>(smem + R::BYTES);  // [warp][group rows][128], not in the ring

    inf_pdl_wait();  // the appended K/V rows and the roped query come from the kernel before this one
    inf_pdl_release();
    const int b = blockIdx.z, kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int kv_len = p.lens[b] + p.len_add;
    if (kv_len <= 0) return;
    // A length beyond what the launch was sized for (max_len -> max_chunks partial slots per sequence) is cut
    // to that size and reported: no partial slot past the sequence's own is ever written.
    if (kv_len > p.max_chunks * p.chunk) {
        kv_len = p.max_chunks * p.chunk;
        if (tid == 0 && blockIdx.x == 0 && kvh == 0) atomicOr(p.status, INF_STATUS_BAD_LEN);
    }
    const int seen = kv_len + p.cur_extra;  // keys the query sees, for the window
    const int win_start = (p.window > 0 && seen > p.window) ? seen - p.window : 0;
    const int first_chunk = win_start / p.chunk;
    const int cpc = p.chunks_per_cta;
    const int run_chunk0 = (int)blockIdx.x * cpc;  // chunk index relative to first_chunk
    const int run_begin = (first_chunk + run_chunk0) * p.chunk;
    if (run_begin >= kv_len) return;
    const int run_end = min(kv_len, run_begin + cpc * p.chunk);
    if ((smem_u32(smem) & 1023u) != 0) {
        if (tid == 0) atomicOr(p.status, INF_STATUS_BAD_SMEM);
        return;
    }

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    {
        const int n_sub = (run_end - run_begin + 15) / 16;
        const int oob_row = p.num_pages * p.kv_heads * p.page_size;  // outside the tensor: TMA fills zeros
        for (int i = tid; i < n_sub; i += THREADS) {
            int token = run_begin + i * 16;
            int slot = token / p.page_size;
            int y = oob_row;
            if (token + 16 <= win_start) {
                // wholly below the window: every key is masked, and the page may have been returned to the pool
            } else if (slot < p.max_pages) {
                int page = p.pages[(long long)b * p.max_pages + slot];
                if (page >= 0 && page < p.num_pages)
                    y = (page * p.kv_heads + kvh) * p.page_size + token % p.page_size;
                else
                    atomicOr(p.status, INF_STATUS_BAD_PAGE);
            } else {
                atomicOr(p.status, INF_STATUS_BAD_LEN);
            }
            row_y[i] = y;
        }
    }
    __syncthreads();

    // Both roles walk the same sequence of tiles: for every chunk of the run, the tiles that hold visible keys.
    // `it` counts tiles across the whole run and drives the ring stage and phase.
    if (warp == CONSUMER_WARPS) {
        // ---------------- producer: one lane issues the TMA loads ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            int it = 0;
            bool ok = true;
            for (int cc = 0; cc < cpc && ok; ++cc) {
                const int key_begin = run_begin + cc * p.chunk;
                if (key_begin >= kv_len) break;
                const int key_end = min(kv_len, key_begin + p.chunk);
                const int lo = max(key_begin, win_start);
                const int tile0 = (lo - key_begin) / TILE_KEYS;
                const int n_tiles = (key_end - key_begin + TILE_KEYS - 1) / TILE_KEYS;
                for (int t = tile0; t < n_tiles; ++t, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1u)) {
                        atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                        ok = false;
                        break;
                    }
                    if (it == p.drop_tile && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) continue;
                    const int remaining = key_end - (key_begin + t * TILE_KEYS);
                    const int nsub = min(4, (remaining + 15) / 16);
                    uint8_t* base = smem + s * STAGE_BYTES;
                    mbar_arrive_expect_tx(&full_bar[s], (uint32_t)nsub * (uint32_t)R::BLOCKS * 2048u);
                    const int sub0 = (key_begin - run_begin) / 16 + t * 4;
                    for (int sub = 0; sub < nsub; ++sub) {
                        const int y = row_y[sub0 + sub];
                        if (FP8) {
                            tma_load_2d(base + 0 * BLOCK_BYTES + sub * 2048, &tm_k, 0, y, &full_bar[s]);
                            tma_load_2d(base + 1 * BLOCK_BYTES + sub * 2048, &tm_v, 0, y, &full_bar[s]);
                        } else {
                            tma_load_2d(base + 0 * BLOCK_BYTES + sub * 2048, &tm_k, 0, y, &full_bar[s]);
                            tma_load_2d(base + 1 * BLOCK_BYTES + sub * 2048, &tm_k, 64, y, &full_bar[s]);
                            tma_load_2d(base + 2 * BLOCK_BYTES + sub * 2048, &tm_v, 0, y, &full_bar[s]);
                            tma_load_2d(base + 3 * BLOCK_BYTES + sub * 2048, &tm_v, 64, y, &full_bar[s]);
                        }
                    }
                }
            }
        }
        return;  // the producer takes no part in the consumers' named barriers
    }

    // ---------------- consumers ----------------
    // Keys are the M rows of the MMAs and the group's query heads the N columns: S^T[16 keys x 8 heads] = K Q^T and
    // O^T[128 dims x 8 heads] += V^T P^T.  A group of up to eight heads fills one 8-wide tile (NT = 1) instead of
    // six of sixteen M rows, which halves the MMAs and the accumulator registers; nine to sixteen heads take two.
    const int g = lane >> 2, qd = lane & 3;
    // Q^T as the B operand: lane (g, qd) holds head g (and g + 8), two dim pairs per k-step
    uint32_t qb[NT][8][2];
    {
        const __half* q0 = p.q + ((long long)b * p.q_heads + (long long)kvh * p.group) * D;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int head = nt * 8 + g;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                // dims behind fragment rows (2 qd, 2 qd + 1) and (2 qd + 8, 2 qd + 9) of k-step kk
                const int c0 = FP8 ? 32 * qd + 4 * kk : kk * 16 + qd * 2;
                const int c1 = FP8 ? c0 + 2 : c0 + 8;
                qb[nt][kk][0] = head < p.group ? *reinterpret_cast<const uint32_t*>(q0 + head * D + c0) : 0u;
                qb[nt][kk][1] = head < p.group ? *reinterpret_cast<const uint32_t*>(q0 + head * D + c1) : 0u;
            }
        }
    }
    const uint32_t smem_base = smem_u32(smem);
    int it = 0;
    bool failed = false;
    for (int cc = 0; cc < cpc; ++cc) {
        const int key_begin = run_begin + cc * p.chunk;
        if (key_begin >= kv_len) break;  // uniform over the CTA
        const int key_end = min(kv_len, key_begin + p.chunk);
        const int lo = max(key_begin, win_start);
        const int tile0 = (lo - key_begin) / TILE_KEYS;
        const int n_tiles = (key_end - key_begin + TILE_KEYS - 1) / TILE_KEYS;

        float o[NT][8][4];  // tile j: dims (d(j, g), d(j, g + 8)) x heads (2 qd, 2 qd + 1)
        float m_run[NT][2], l_run[NT][2];  // per head 2 qd + e; the sums are partial over this lane's keys
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            m_run[nt][0] = m_run[nt][1] = M_INIT;
            l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) o[nt][j][0] = o[nt][j][1] = o[nt][j][2] = o[nt][j][3] = 0.f;
        }

        for (int t = tile0; t < n_tiles; ++t, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            if (!failed && !mbar_wait(&full_bar[s], ph)) {
                if (lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                failed = true;
            }
            const int k0 = key_begin + t * TILE_KEYS + warp * 16;  // first key of this warp's page tile
            bool wrote_smem = false;
            if (!failed && k0 < key_end && k0 + 16 > lo) {
                const uint32_t stage = smem_base + s * STAGE_BYTES;
                const bool edge = (k0 < lo) || (k0 + 16 > key_end);
                if (edge) {
                    // slots of a page past the sequence end may hold anything: zero those V rows so that
                    // 0 * garbage cannot poison the accumulators
                    constexpr int CH = FP8 ? 8 : 16;  // 16-byte chunks per V row
                    for (int i = lane; i < 16 * CH; i += 32) {
                        int r = i / CH, ch = i % CH;
                        int key = k0 + r;
                        if (key < lo || key >= key_end) {
                            uint8_t* dst = smem + s * STAGE_BYTES + (R::V_BLOCK + (ch >> 3)) * BLOCK_BYTES +
                                           (warp * 16 + r) * 128 + (ch & 7) * 16;
                            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
                        }
                    }
                    wrote_smem = true;
                    __syncwarp();
                }
                // ---- S^T = K Q^T for 16 keys: rows g and g + 8 are keys, columns 2 qd, 2 qd + 1 heads
                float sc[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
                if (FP8) {
                    // lane (g, qd) takes bytes [32 qd, 32 qd + 32) of key rows g and g + 8 (row & 7 == g)
                    const uint32_t r_lo = stage + (warp * 16 + g) * 128, r_hi = r_lo + 8 * 128;
                    const uint32_t x0 = ((2 * qd) ^ g) << 4, x1 = ((2 * qd + 1) ^ g) << 4;
                    const uint4 a0 = lds128(r_lo + x0), a1 = lds128(r_lo + x1);
                    const uint4 b0 = lds128(r_hi + x0), b1 = lds128(r_hi + x1);
                    const uint32_t wl[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                    const uint32_t wh[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        uint32_t ka[4];
                        fp8x4_to_f16x4(wl[kk], ka[0], ka[2]);
                        fp8x4_to_f16x4(wh[kk], ka[1], ka[3]);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_16816(sc[nt], ka, qb[nt][kk][0], qb[nt][kk][1]);
                    }
                } else {
                    const int krow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const int dchunk = kk * 2 + (lane >> 4);
                        uint32_t ka[4];
                        ldsm_x4(stage + (dchunk >> 3) * BLOCK_BYTES + sw128_offset(krow, (dchunk & 7) * 8), ka);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_16816(sc[nt], ka, qb[nt][kk][0], qb[nt][kk][1]);
                    }
                }
                // ---- online softmax (log2 domain) per head; this lane holds keys k0 + g and k0 + g + 8
                const bool dead_lo = edge && (k0 + g < lo || k0 + g >= key_end);
                const bool dead_hi = edge && (k0 + g + 8 < lo || k0 + g + 8 >= key_end);
                uint32_t pb[NT][2];
                bool moved = false;
                float alpha[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) sc[nt][e] *= p.scale_log2;
                    if (dead_lo) sc[nt][0] = sc[nt][1] = -INFINITY;
                    if (dead_hi) sc[nt][2] = sc[nt][3] = -INFINITY;
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        float mx = fmaxf(sc[nt][e], sc[nt][2 + e]);
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                        const float m_new = fmaxf(m_run[nt][e], mx);
                        alpha[nt][e] = ex2_approx(m_run[nt][e] - m_new);
                        moved |= m_new != m_run[nt][e];
                        m_run[nt][e] = m_new;
                        const float p_lo = ex2_approx(sc[nt][e] - m_new), p_hi = ex2_approx(sc[nt][2 + e] - m_new);
                        sc[nt][e] = p_lo;
                        sc[nt][2 + e] = p_hi;
                        l_run[nt][e] = l_run[nt][e] * alpha[nt][e] + p_lo + p_hi;
                    }
                    // P^T as the B operand of PV: the 8 x 8 blocks (keys g | g + 8) x heads transposed across the warp
                    uint32_t lo8 = pack_half2(sc[nt][0], sc[nt][1]), hi8 = pack_half2(sc[nt][2], sc[nt][3]);
                    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb[nt][0]) : "r"(lo8));
                    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb[nt][1]) : "r"(hi8));
                }
                // the accumulators only need rescaling when a maximum moved, which becomes rare after the first tiles
                if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            o[nt][j][0] *= alpha[nt][0];
                            o[nt][j][1] *= alpha[nt][1];
                            o[nt][j][2] *= alpha[nt][0];
                            o[nt][j][3] *= alpha[nt][1];
                        }
                }
                // ---- O^T += V^T P^T
                if (FP8) {
                    // lane (g, qd) takes dims [16 g, 16 g + 16) of key rows 2 qd, 2 qd + 1, 2 qd + 8, 2 qd + 9: tile j
                    // covers dims 16 g + 2 j (fragment row g) and 16 g + 2 j + 1 (fragment row g + 8)
                    const uint32_t vb = stage + R::V_BLOCK * BLOCK_BYTES;
                    const int r0 = warp * 16 + 2 * qd;
                    const uint4 v0 = lds128(vb + r0 * 128 + ((g ^ (r0 & 7)) << 4));
                    const uint4 v1 = lds128(vb + (r0 + 1) * 128 + ((g ^ ((r0 + 1) & 7)) << 4));
                    const uint4 v2 = lds128(vb + (r0 + 8) * 128 + ((g ^ (r0 & 7)) << 4));
                    const uint4 v3 = lds128(vb + (r0 + 9) * 128 + ((g ^ ((r0 + 1) & 7)) << 4));
                    const uint32_t ra[4] = {v0.x, v0.y, v0.z, v0.w}, rb[4] = {v1.x, v1.y, v1.z, v1.w};
                    const uint32_t rc[4] = {v2.x, v2.y, v2.z, v2.w}, rd[4] = {v3.x, v3.y, v3.z, v3.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        // bytes of two key rows side by side: [a0 b0 a1 b1] and [a2 b2 a3 b3]
                        const uint32_t t01 = __byte_perm(ra[w], rb[w], 0x5140), t23 = __byte_perm(ra[w], rb[w], 0x7362);
                        const uint32_t u01 = __byte_perm(rc[w], rd[w], 0x5140), u23 = __byte_perm(rc[w], rd[w], 0x7362);
                        uint32_t va[4], vc[4];
                        fp8x4_to_f16x4(t01, va[0], va[1]);
                        fp8x4_to_f16x4(u01, va[2], va[3]);
                        fp8x4_to_f16x4(t23, vc[0], vc[1]);
                        fp8x4_to_f16x4(u23, vc[2], vc[3]);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            mma_16816(o[nt][2 * w], va, pb[nt][0], pb[nt][1]);
                            mma_16816(o[nt][2 * w + 1], vc, pb[nt][0], pb[nt][1]);
                        }
                    }
                } else {
                    const int mat = lane >> 3, rin = lane & 7;
                    const int vrow = warp * 16 + (mat >> 1) * 8 + rin;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int dchunk = 2 * j + (mat & 1);
                        uint32_t va[4];
                        ldsm_x4_trans(stage + (2 + (dchunk >> 3)) * BLOCK_BYTES + sw128_offset(vrow, (dchunk & 7) * 8), va);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_16816(o[nt][j], va, pb[nt][0], pb[nt][1]);
                    }
                }
            }
            if (wrote_smem) fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
        // ---------------- merge the four warps of this chunk through their own shared-memory buffer ----------------
        {
            float* mw = merge + warp * p.group * D;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    // the row sums are spread over the eight lanes that share qd
                    float l = l_run[nt][e];
                    l += __shfl_xor_sync(0xffffffffu, l, 4);
                    l += __shfl_xor_sync(0xffffffffu, l, 8);
                    l += __shfl_xor_sync(0xffffffffu, l, 16);
                    const int head = nt * 8 + 2 * qd + e;
                    if (head < p.group) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int d_lo = FP8 ? 16 * g + 2 * j : 16 * j + g, d_hi = FP8 ? d_lo + 1 : d_lo + 8;
                            mw[head * D + d_lo] = o[nt][j][e];
                            mw[head * D + d_hi] = o[nt][j][2 + e];
                        }
                        if (g == 0) {
                            warp_m[warp][head] = m_run[nt][e];
                            warp_l[warp][head] = l;
                        }
                    }
                }
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four consumer warps only
        {
            const long long prow0 =
                ((long long)b * p.max_chunks + run_chunk0 + cc) * p.q_heads + (long long)kvh * p.group;
            for (int r = 0; r < p.group; ++r) {
                float M = fmaxf(fmaxf(warp_m[0][r], warp_m[1][r]), fmaxf(warp_m[2][r], warp_m[3][r]));
                float acc = 0.f, L = 0.f;
#pragma unroll
                for (int w = 0; w < CONSUMER_WARPS; ++w) {
                    float sc = ex2_approx(warp_m[w][r] - M);
                    acc += sc * merge[(w * p.group + r) * D + tid];
                    L += sc * warp_l[w][r];
                }
                p.part_acc[(prow0 + r) * D + tid] = FP8 ? acc * p.v_scale : acc;
                if (tid == 0) {
                    p.part_ml[(prow0 + r) * 2 + 0] = M;
                    p.part_ml[(prow0 + r) * 2 + 1] = L;
                }
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the merge buffer is free again
    }
}

// kernels/fp8_attention_kernels.metal:56-64
__device__ __forceinline__ float softplus_ref(float v) {
    if (v > 20.0f) return v;
    if (v < -20.0f) return expf(v);
    return logf(1.0f + expf(v));
}

// The other ranks' copies of the gathered output when the batch is sharded by sequence, each already offset to this
// rank's first sequence like `out` itself (peer memory mapped into this process; plain stores).
struct DecodePeerOuts {
    void* out[INF_MAX_PEERS];
    int count;
};

// Merge of the per-chunk partials.  The chunk weights are computed once in shared memory so that the
// accumulation is a stream of independent coalesced loads.  When cur_k / cur_v are given (FP8 pages), the current
// token is not among the cached keys: its score q . k and its value enter here as one more term, at full precision
// (fp8_attention_kernels.metal:155-163, 199-207).
template <typename OutT>
__global__ void __launch_bounds__(D)
gqa_decode_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                          const int* __restrict__ lens, const float* __restrict__ gate, OutT* __restrict__ out,
                          int q_heads, int max_chunks, int chunk, int window, int len_add,
                          const __half* __restrict__ q, const __half* __restrict__ cur_k,
                          const __half* __restrict__ cur_v, int group, float cur_scale_log2, DecodePeerOuts peers) {
    __shared__ float w[MAX_CHUNK / TILE_KEYS * 16];  // up to 512 chunks
    __shared__ float red[4];
    inf_pdl_wait();
    inf_pdl_release();
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const bool has_cur = cur_k != nullptr;
    int kv_len = lens[b] + len_add;
    const long long orow = ((long long)b * q_heads + h) * D + d;
    if (kv_len < 0 || (kv_len == 0 && !has_cur)) {
        out[orow] = OutT(0.f);
        for (int pr = 0; pr < peers.count; ++pr) reinterpret_cast<OutT*>(peers.out[pr])[orow] = OutT(0.f);
        return;
    }
    kv_len = min(kv_len, max_chunks * chunk);  // the partial kernel cut it the same way and raised the status word
    const int seen = kv_len + (has_cur ? 1 : 0);
    const int win_start = (window > 0 && seen > window) ? seen - window : 0;
    const int first_chunk = win_start / chunk;
    const int n = max(0, (kv_len + chunk - 1) / chunk - first_chunk);  // <= max_chunks <= 512
    const long long prow0 = ((long long)b * max_chunks) * q_heads + h;
    float s_cur = M_INIT, v_cur = 0.f;
    if (has_cur) {
        const long long krow = ((long long)b * (q_heads / group) + h / group) * D + d;
        float prod = __half2float(q[orow]) * __half2float(cur_k[krow]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) prod += __shfl_xor_sync(0xffffffffu, prod, o);
        if ((d & 31) == 0) red[d >> 5] = prod;
        __syncthreads();
        s_cur = (red[0] + red[1] + red[2] + red[3]) * cur_scale_log2;
        v_cur = __half2float(cur_v[krow]);
        __syncthreads();
    }
    float mloc = s_cur;
    for (int c = d; c < n; c += D) mloc = fmaxf(mloc, part_ml[(prow0 + (long long)c * q_heads) * 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
    if ((d & 31) == 0) red[d >> 5] = mloc;
    __syncthreads();
    const float M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    float lloc = 0.f;
    for (int c = d; c < n; c += D) {
        const float wc = ex2_approx(part_ml[(prow0 + (long long)c * q_heads) * 2] - M);
        w[c] = wc;
        lloc += wc * part_ml[(prow0 + (long long)c * q_heads) * 2 + 1];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lloc += __shfl_xor_sync(0xffffffffu, lloc, o);
    if ((d & 31) == 0) red[d >> 5] = lloc;
    __syncthreads();
    const float w_cur = has_cur ? ex2_approx(s_cur - M) : 0.f;
    const float L = red[0] + red[1] + red[2] + red[3] + w_cur;
    const float* src = part_acc + prow0 * D + d;
    float acc = w_cur * v_cur;
#pragma unroll 8
    for (int c = 0; c < n; ++c) acc += w[c] * src[(long long)c * q_heads * D];
    const float gain = (gate ? softplus_ref(gate[(long long)b * q_heads + h]) : 1.0f) / L;
    const OutT o = OutT(acc * gain);
    out[orow] = o;
    // a batch sharded by sequence: the row also goes into the other ranks' copies of the gathered output
    for (int pr = 0; pr < peers.count; ++pr) reinterpret_cast<OutT*>(peers.out[pr])[orow] = o;
}

}  // namespace

// What distinguishes the FP8 form of a launch: byte pools with their scales, and the current token given separately.
struct DecodeFp8 {
    float key_scale, value_scale;
    const void* cur_k;
    const void* cur_v;
};

int inf_gqa_decode_launch(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                          int q_heads, int max_len, int split_chunk, int sliding_window, const float* gate,
                          float scale, void* out, int out_dtype, void* scratch, size_t scratch_bytes, int len_add,
                          const DecodeFp8* fp8, void* const* peer_outs, int n_peers);

extern "C" size_t inf_gqa_decode_workspace_bytes(int32_t batch, int32_t q_heads, int32_t head_dim, int32_t max_len,
                                                 int32_t split_chunk) {
    if (batch <= 0 || q_heads <= 0 || head_dim <= 0 || max_len <= 0 || split_chunk <= 0) return 0;
    size_t max_chunks = (size_t)(max_len + split_chunk - 1) / split_chunk;
    return (size_t)batch * max_chunks * q_heads * (head_dim + 2) * sizeof(float);
}

// Shared by the allocating entry point below and by callers that bring their own scratch.
int inf_gqa_decode_launch(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                          int q_heads, int max_len, int split_chunk, int sliding_window, const float* gate,
                          float scale, void* out, int out_dtype, void* scratch, size_t scratch_bytes, int len_add,
                          const DecodeFp8* fp8, void* const* peer_outs, int n_peers) {
    if (!q_f16 || !pool || !table || !out) return inf_fail(ctx, INF_E_ARG, "gqa_decode: null pointer");
    if (!pool->k || !pool->v) return inf_fail(ctx, INF_E_ARG, "gqa_decode: pool has no storage");
    if (pool->head_dim != D) return inf_fail(ctx, INF_E_SHAPE, "gqa_decode: head_dim must be 128, got %d", pool->head_dim);
    if (pool->page_size % 16 != 0) return inf_fail(ctx, INF_E_CACHE, "gqa_decode: page_size must be a multiple of 16");
    if (q_heads <= 0 || q_heads % pool->kv_heads != 0)
        return inf_fail(ctx, INF_E_SHAPE, "gqa_decode: q_heads %d must be a positive multiple of kv_heads %d", q_heads,
                        pool->kv_heads);
    const int group = q_heads / pool->kv_heads;
    if (group > 16) return INF_UNSUPPORTED;
    if (split_chunk <= 0 || split_chunk % TILE_KEYS != 0 || split_chunk > MAX_CHUNK)
        return inf_fail(ctx, INF_E_CONFIG, "gqa_decode: split_chunk must be a multiple of 64 in [64, 2048], got %d",
                        split_chunk);
    if (max_len <= 0) return inf_fail(ctx, INF_E_SHAPE, "gqa_decode: max_len must be positive");
    if (sliding_window < 0) return inf_fail(ctx, INF_E_CONFIG, "gqa_decode: sliding_window must be >= 0");
    if (out_dtype != INF_DTYPE_F32 && out_dtype != INF_DTYPE_F16)
        return inf_fail(ctx, INF_E_DTYPE, "gqa_decode: output dtype must be f32 or f16");
    if (fp8 && (!fp8->cur_k || !fp8->cur_v)) return inf_fail(ctx, INF_E_ARG, "gqa_decode_fp8: null current key / value");
    if (fp8 && (!(fp8->key_scale > 0.f) || !(fp8->value_scale > 0.f) || !isfinite(fp8->key_scale) || !isfinite(fp8->value_scale)))
        return inf_fail(ctx, INF_E_CONFIG, "gqa_decode_fp8: scales must be positive and finite");
    if (n_peers < 0 || n_peers > INF_MAX_PEERS)
        return inf_fail(ctx, INF_E_CONFIG, "gqa_decode: %d peers, at most %d are supported", n_peers, INF_MAX_PEERS);
    if (n_peers > 0 && !peer_outs) return inf_fail(ctx, INF_E_ARG, "gqa_decode: null peer list");
    DecodePeerOuts peers;
    peers.count = n_peers;
    for (int i = 0; i < INF_MAX_PEERS; ++i) {
        peers.out[i] = i < n_peers ? peer_outs[i] : nullptr;
        if (i < n_peers && (!peers.out[i] || (reinterpret_cast<uintptr_t>(peers.out[i]) & 3u)))
            return inf_fail(ctx, INF_E_ARG, "gqa_decode: peer output %d is null or misaligned", i);
    }
    const int cur_extra = fp8 ? 1 : 0;  // the FP8 form counts cached rows; the current token comes on top
    int rc = inf_validate_table(ctx, table, pool->num_pages, pool->page_size, len_add, "gqa_decode", sliding_window, 1);
    if (rc != INF_OK) return rc;
    if (table->host_lens)
        for (int b = 0; b < table->batch; ++b)
            if (table->host_lens[b] + len_add + cur_extra > max_len)
                return inf_fail(ctx, INF_E_SHAPE, "gqa_decode: sequence %d length %d exceeds max_len %d", b,
                                table->host_lens[b] + cur_extra, max_len);
    // with a window only ceil(window/chunk)+1 chunks can be visible
    int max_chunks = (max_len + split_chunk - 1) / split_chunk;
    if (max_chunks > 512)
        return inf_fail(ctx, INF_E_CONFIG, "gqa_decode: %d chunks of %d keys exceed the 512 the combine step holds; "
                        "use a larger split_chunk", max_chunks, split_chunk);
    size_t need = inf_gqa_decode_workspace_bytes(table->batch, q_heads, D, max_len, split_chunk);
    if (scratch_bytes < need)
        return inf_fail(ctx, INF_E_ARG, "gqa_decode: scratch of %zu bytes is smaller than the %zu needed", scratch_bytes,
                        need);

    const uint64_t rows_total = (uint64_t)pool->num_pages * pool->kv_heads * pool->page_size;
    const uint32_t elem = fp8 ? 1u : 2u;
    uint64_t dims[2] = {(uint64_t)D, rows_total};
    uint64_t strides[1] = {(uint64_t)D * elem};
    uint32_t box[2] = {fp8 ? 128u : 64u, 16};  // 128 bytes wide either way
    CUtensorMap tm_k, tm_v;
    rc = inf_make_tmap_typed(ctx, pool->k, 2, dims, strides, box, &tm_k, elem);
    if (rc != INF_OK) return rc;
    rc = inf_make_tmap_typed(ctx, pool->v, 2, dims, strides, box, &tm_v, elem);
    if (rc != INF_OK) return rc;

    const float base_scale = scale > 0.f ? scale : 1.0f / sqrtf((float)D);
    DecodeParams p;
    p.q = (const __half*)q_f16;
    p.pages = table->pages;
    p.lens = table->lens;
    p.max_pages = table->max_pages;
    p.q_heads = q_heads;
    p.kv_heads = pool->kv_heads;
    p.group = group;
    p.page_size = pool->page_size;
    p.num_pages = pool->num_pages;
    p.chunk = split_chunk;
    p.window = sliding_window;
    p.len_add = len_add;
    p.cur_extra = cur_extra;
    p.scale_log2 = base_scale * (fp8 ? fp8->key_scale * FP8_CVT_GAIN : 1.0f) * 1.4426950408889634f;
    p.v_scale = fp8 ? fp8->value_scale * FP8_CVT_GAIN : 1.0f;
    p.part_acc = (float*)scratch;
    p.part_ml = p.part_acc + (size_t)table->batch * max_chunks * q_heads * D;
    p.max_chunks = max_chunks;
    // A CTA streams a run of up to four chunks (2 048 keys), which keeps its ring full across chunk boundaries; a small
    // batch gets shorter runs, so that the launch still has about two waves of CTAs to spread over the SMs.
    p.chunks_per_cta = MAX_CHUNK / split_chunk;
    {
        const long long upper = (long long)table->batch * pool->kv_heads * max_chunks;  // chunks if every sequence were full
        const long long two_waves = 2LL * 2 * ctx->sm_count;
        while (p.chunks_per_cta > 1 && upper / p.chunks_per_cta < two_waves) p.chunks_per_cta >>= 1;
    }
    p.status = ctx->status;
    p.drop_tile = ctx->debug_drop_tile;
    ctx->debug_drop_tile = -1;  // one launch only

    const size_t ring = fp8 ? Ring<true>::BYTES : Ring<false>::BYTES;
    const size_t smem = ring + (size_t)CONSUMER_WARPS * group * D * sizeof(float);
    // four instantiations: fp16 or FP8 pages, one or two 8-head tiles per KV group
    void (*kernel)(CUtensorMap, CUtensorMap, DecodeParams) =
        fp8 ? (group <= 8 ? gqa_decode_partial_kernel<true, 1> : gqa_decode_partial_kernel<true, 2>)
            : (group <= 8 ? gqa_decode_partial_kernel<false, 1> : gqa_decode_partial_kernel<false, 2>);
    const uint32_t attr_bit = (fp8 ? 32u : 1u) << (group <= 8 ? 0 : 6);  // bits 0, 5, 6, 11
    if (!(ctx->func_attr_done & attr_bit)) {
        const int limit = (int)(ring + CONSUMER_WARPS * 16 * D * sizeof(float));
        INF_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, limit));
        ctx->func_attr_done |= attr_bit;
    }
    dim3 grid((max_chunks + p.chunks_per_cta - 1) / p.chunks_per_cta, pool->kv_heads, table->batch);
    {
        inf_prof_scope prof(ctx, fp8 ? "gqa_decode_partial_fp8_kernel" : "gqa_decode_partial_kernel");
        INF_CUDA(ctx, inf_launch_pdl(kernel, grid, dim3(THREADS), smem, ctx->stream, tm_k, tm_v, p));
    }
    INF_LAUNCH_CHECK(ctx, "gqa_decode_partial_kernel");
    dim3 cgrid(q_heads, table->batch);
    const __half* cq = fp8 ? (const __half*)q_f16 : nullptr;
    const __half* ck = fp8 ? (const __half*)fp8->cur_k : nullptr;
    const __half* cv = fp8 ? (const __half*)fp8->cur_v : nullptr;
    const float cur_scale_log2 = base_scale * 1.4426950408889634f;
    if (out_dtype == INF_DTYPE_F32)
        INF_CUDA(ctx, inf_launch_pdl(gqa_decode_combine_kernel<float>, cgrid, dim3(D), 0, ctx->stream, p.part_acc, p.part_ml,
                                     table->lens, gate, (float*)out, q_heads, max_chunks, split_chunk, sliding_window,
                                     len_add, cq, ck, cv, group, cur_scale_log2, peers));
    else
        INF_CUDA(ctx, inf_launch_pdl(gqa_decode_combine_kernel<__half>, cgrid, dim3(D), 0, ctx->stream, p.part_acc,
                                     p.part_ml, table->lens, gate, (__half*)out, q_heads, max_chunks, split_chunk,
                                     sliding_window, len_add, cq, ck, cv, group, cur_scale_log2, peers));
    INF_LAUNCH_CHECK(ctx, "gqa_decode_combine_kernel");
    return INF_OK;
}

extern "C" int32_t inf_debug_drop_next_load(inf_ctx* ctx, int32_t tile) {
    INF_CHECK_CTX(ctx);
    ctx->debug_drop_tile = tile;
    return INF_OK;
}

extern "C" int32_t inf_gqa_decode_paged(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                        const inf_page_table* table, int32_t q_heads, int32_t max_len,
                                        int32_t split_chunk, int32_t sliding_window, const float* gate, float scale,
                                        void* out, int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
    if (!table) return inf_fail(ctx, INF_E_ARG, "gqa_decode: null page table");
    size_t need = inf_gqa_decode_workspace_bytes(table->batch, q_heads, D, max_len, split_chunk);
    if (need == 0) return inf_fail(ctx, INF_E_SHAPE, "gqa_decode: sizes must be positive");
    int rc = inf_ensure_workspace(ctx, need);
    if (rc != INF_OK) return rc;
    return inf_gqa_decode_launch(ctx, q_f16, pool, table, q_heads, max_len, split_chunk, sliding_window, gate, scale,
                                 out, out_dtype, ctx->workspace, ctx->workspace_bytes, 0, nullptr, nullptr, 0);
}

// The same decode for a batch sharded by sequence over the GPUs of one box: `out` points at this rank's rows inside
// its own copy of the gathered [all sequences][q_heads][128] output and peer_outs[i] at the same rows inside rank i's
// copy (inf_peer_open), so the combine kernel's stores are the all-gather.  inf_comm_barrier ends the step.
extern "C" int32_t inf_gqa_decode_paged_peers(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                              const inf_page_table* table, int32_t q_heads, int32_t max_len,
                                              int32_t split_chunk, int32_t sliding_window, const float* gate,
                                              float scale, void* out, int32_t out_dtype, void* const* peer_outs,
                                              int32_t n_peers) {
    INF_CHECK_CTX(ctx);
    if (!table) return inf_fail(ctx, INF_E_ARG, "gqa_decode: null page table");
    size_t need = inf_gqa_decode_workspace_bytes(table->batch, q_heads, D, max_len, split_chunk);
    if (need == 0) return inf_fail(ctx, INF_E_SHAPE, "gqa_decode: sizes must be positive");
    int rc = inf_ensure_workspace(ctx, need);
    if (rc != INF_OK) return rc;
    return inf_gqa_decode_launch(ctx, q_f16, pool, table, q_heads, max_len, split_chunk, sliding_window, gate, scale,
                                 out, out_dtype, ctx->workspace, ctx->workspace_bytes, 0, nullptr, peer_outs, n_peers);
}

extern "C" int32_t inf_gqa_decode_paged_fp8(inf_ctx* ctx, const void* q_f16, const void* cur_k_f16, const void* cur_v_f16,
                                            const inf_kv_pool_fp8* pool, const inf_page_table* table, int32_t q_heads,
                                            int32_t max_len, int32_t split_chunk, int32_t sliding_window,
                                            const float* gate, float scale, void* out, int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
    if (!table || !pool) return inf_fail(ctx, INF_E_ARG, "gqa_decode_fp8: null pool or page table");
    size_t need = inf_gqa_decode_workspace_bytes(table->batch, q_heads, D, max_len, split_chunk);
    if (need == 0) return inf_fail(ctx, INF_E_SHAPE, "gqa_decode_fp8: sizes must be positive");
    int rc = inf_ensure_workspace(ctx, need);
    if (rc != INF_OK) return rc;
    const inf_kv_pool shape = {pool->k, pool->v, pool->num_pages, pool->page_size, pool->kv_heads, pool->head_dim};
    const DecodeFp8 fp8 = {pool->key_scale, pool->value_scale, cur_k_f16, cur_v_f16};
    return inf_gqa_decode_launch(ctx, q_f16, &shape, table, q_heads, max_len, split_chunk, sliding_window, gate, scale,
                                 out, out_dtype, ctx->workspace, ctx->workspace_bytes, 0, &fp8, nullptr, 0);
}

// ------------------------------------------------------------------------------------------------
// Decode without any allocation.
//
// inf_gqa_decode_paged keeps its split-KV partials in the context's workspace, which it grows with
// cudaMalloc whenever a call needs more than any earlier one did.  Some callers cannot afford that:
// a serving loop that has already handed every free byte of HBM to its KV pool, so that a late
// cudaMalloc may simply fail; a latency-bound decode loop, for which the device-wide synchronisation
// hidden inside cudaMalloc / cudaFree is a stall in the middle of a token; a host whose device memory
// belongs to another allocator and must not be touched behind its back.  For them the partials live
// in the fixed array below, which is part of the library image: every GPU that loads the library
// holds these INF_GQA_DECODE_STATIC_SCRATCH_BYTES until the process exits.
//
// In host code the name of a __device__ array is only a host-side stand-in, not a device address, so
// the address is looked up once per device with cudaGetSymbolAddress (with that device current) and
// that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_decode_static_scratch[INF_GQA_DECODE_STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
// Written once per device under the mutex, read afterwards through the atomic: two host threads making
// their first call on one device at the same time both end up with the same, fully resolved pointer.
std::atomic<void*> g_static_scratch_ptr[MAX_DEVICES];
std::mutex g_static_scratch_mutex;
}  // namespace

extern "C" int32_t inf_gqa_decode_paged_static(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                               const inf_page_table* table, int32_t q_heads, int32_t max_len,
                                               int32_t split_chunk, int32_t sliding_window, const float* gate,
                                               float scale, void* out, int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
    if (!table) return inf_fail(ctx, INF_E_ARG, "gqa_decode_static: null page table");
    const size_t need = inf_gqa_decode_workspace_bytes(table->batch, q_heads, D, max_len, split_chunk);
    if (need == 0) return inf_fail(ctx, INF_E_SHAPE, "gqa_decode_static: sizes must be positive");
    if (need > (size_t)INF_GQA_DECODE_STATIC_SCRATCH_BYTES)
        return inf_fail(ctx, INF_E_CONFIG,
                        "gqa_decode_static: batch %d x %d chunks x %d heads needs %zu bytes of split-KV scratch, the "
                        "built-in array holds %zu; use a larger split_chunk, a smaller batch, or inf_gqa_decode_paged",
                        table->batch, (max_len + split_chunk - 1) / split_chunk, q_heads, need,
                        (size_t)INF_GQA_DECODE_STATIC_SCRATCH_BYTES);
    if (ctx->device < 0 || ctx->device >= MAX_DEVICES)
        return inf_fail(ctx, INF_E_ARG, "gqa_decode_static: device ordinal %d is out of range", ctx->device);
    void* scratch = g_static_scratch_ptr[ctx->device].load(std::memory_order_acquire);
    if (!scratch) {
        // first call on this device: resolve the array's device address with this device current
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        scratch = g_static_scratch_ptr[ctx->device].load(std::memory_order_relaxed);
        if (!scratch) {
            int current = -1;
            INF_CUDA(ctx, cudaGetDevice(&current));
            if (current != ctx->device) INF_CUDA(ctx, cudaSetDevice(ctx->device));
            cudaError_t e = cudaGetSymbolAddress(&scratch, g_decode_static_scratch);
            if (current != ctx->device) cudaSetDevice(current);
            if (e != cudaSuccess || !scratch)
                return inf_fail(ctx, INF_E_BACKEND, "gqa_decode_static: cudaGetSymbolAddress failed: %s",
                                cudaGetErrorString(e));
            g_static_scratch_ptr[ctx->device].store(scratch, std::memory_order_release);
        }
    }
    // Nothing in the array has to start at zero: every partial the combine kernel reads is written
    // by the partial kernel of the same call first.
    return inf_gqa_decode_launch(ctx, q_f16, pool, table, q_heads, max_len, split_chunk, sliding_window, gate, scale,
                                 out, out_dtype, scratch, (size_t)INF_GQA_DECODE_STATIC_SCRATCH_BYTES, 0, nullptr, nullptr, 0);
}

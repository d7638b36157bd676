// Causal flash attention for prefill on tcgen05 / TMEM, fed by TMA.
//
// One CTA per SM runs TWO query streams of 128 rows each against one shared ring of 128-key K/V tiles,
// so every K/V tile is fetched once for 256 query rows.  The two streams are either two query heads of the
// same KV group at the same rows (GQA: identical causal structure, perfectly balanced) or two consecutive
// 128-row tiles of one head (MHA / MLA prefill).
//
// Twelve warps, specialised:
//   warps 0-3   softmax + epilogue of stream 0; thread r owns query row r and TMEM lane r
//   warps 4-7   the same for stream 1
//   warp 8      TMA producer for Q and the K ring (64-column blocks, returned one by one)
//   warp 9      allocates TMEM; one thread issues every QK^T
//   warp 10     TMA producer for the V ring
//   warp 11     one thread issues every PV
// After set-up setmaxnreg moves registers from warps 8-11 (40 each) to the softmax warpgroups (232 each), so
// a whole 128-key S row lives in registers and the softmax is a single pass.
// Per stream and 128-key tile:
//   S = Q K^T    SS MMA, M128 N128 K16, both operands K-major with the 128-byte swizzle, into the ONE S buffer
//                the two streams share; the softmax warpgroup copies its row out at once, which frees the
//                buffer for the other stream's next QK^T
//   softmax      row maximum, lazy rescale of O (only when a maximum grew by more than 2^8), exponentials;
//                in the dense instantiation the streams take turns at the exponentials, which keeps them in
//                anti-phase; P goes back to
//                TMEM as packed fp16, each 64-key half handed to the PV issuer as soon as it is written
//   O += P V     TS MMA, A = P from TMEM, B = V MN-major straight from its [key][dim] tile
// TMEM (512 columns): S 128, then per stream P 64 (fp16 pairs) and O 128 (fp32).
//
// Work order: CTAs are numbered so that those in flight together share K/V: all query-tile pairs of a small
// group of heads, latest (heaviest) rows first, before the next group.  With the head as the fast index the
// CTAs in flight covered every head at two or three query tiles and their K/V working set was several
// times the L2.
//
// Two instantiations: paged GQA prefill (head_dim 128; a K/V tile is eight 16-token page boxes addressed
// through the page table; reference kernel f16_attention_kernels.metal:153-316) and dense MLA prefill
// over expanded heads (qk 128+64 with the rope tail shared by all heads, v 128; reference kernel
// attention_kernels.metal:723-968 with no past, K laid out as in layout_kernels.metal:148-183).
#include <cuda_fp16.h>
#include <math.h>

#include <stdlib.h>

#include <algorithm>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

using namespace inf;

namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int NUM_THREADS = 384;
constexpr float M_INIT = -1.0e30f;
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr uint32_t TMEM_COLS = 512;
// TMEM columns: one S buffer shared by both streams (a stream's softmax copies its S row into registers at
// once, which frees the buffer for the other stream's next QK), then per stream P (fp16 pairs) and O (fp32).
constexpr uint32_t COL_S = 0, COL_STREAM0 = 128, STREAM_COLS = 192, COL_P = 0, COL_O = 64;

struct FlashParams {
    int tokens, q_heads, kv_heads, group, batch;
    int pair_heads;  // 1: streams are heads (2c, 2c+1) at the same rows; 0: streams are row tiles (2c, 2c+1) of one head
    int grid_heads, grid_tiles;  // work items per batch entry: head (pair) count x query-tile (pair) count
    int raster_heads;            // heads (pairs) whose work items are interleaved before the next group starts
    const int* pages;
    const int* lens;
    int max_pages, page_size, num_pages;
    int window;
    float scale_log2;
    const float* gate;  // [batch][tokens][q_heads] or null
    void* out;
    int out_f16;
    long long o_ts, o_hs, o_bs;  // element strides of the output: token, head, batch
    // Head-sharded runs: the same output rows are also stored into the other ranks' copies of the gathered tensor
    // (peer memory over NVLink, plain stores), same strides as `out`: the all-gather happens tile by tile in the
    // epilogue instead of as a collective after the kernel.
    void* peer_out[INF_MAX_PEERS];
    int n_peers;
    int* status;
#ifdef INF_KPROF
    long long* kprof;      // debug builds only: cycle counters of CTA (0,0,0)
    long long* kprof_cta;  // debug builds only: per CTA {sm id, ns at entry, after set-up, before the last sync, at exit}
#endif
};

#ifdef INF_KPROF
#define KP_T0() long long kp_t = clock64()
#define KP_ADD(slot) do { long long kp_n = clock64(); if (kp_on) kp_acc[slot] += kp_n - kp_t; kp_t = kp_n; } while (0)
#else
#define KP_T0() do {} while (0)
#define KP_ADD(slot) do {} while (0)
#endif

// kernels/fp8_attention_kernels.metal:56-64
__device__ __forceinline__ float softplus_ref(float v) {
    if (v > 20.0f) return v;
    if (v < -20.0f) return expf(v);
    return logf(1.0f + expf(v));
}

template <int DQK, int DV, int KB, int VS>
struct SmemLayout {
    static constexpr int Q_BYTES = BM * DQK * 2;  // per stream
    static constexpr int KBLK_BYTES = BN * 128;   // one [128 keys][64 dims] block of a K tile
    static constexpr int V_BYTES = BN * DV * 2;
    static constexpr int OFF_K = 2 * Q_BYTES;
    static constexpr int OFF_V = OFF_K + KB * KBLK_BYTES;
    static constexpr int OFF_BAR = OFF_V + VS * V_BYTES;
    static constexpr int TOTAL = OFF_BAR + 512;
};

struct Stream {
    int head, q0, kt_begin, kt_end;  // key-tile range [kt_begin, kt_end); empty when the stream has no rows
};

template <int DQK, int DV, int KB, int VS, bool PAGED>
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_k2, const __grid_constant__ CUtensorMap tm_v,
                     FlashParams p) {
    using L = SmemLayout<DQK, DV, KB, VS>;
    constexpr int NB = DQK / 64;  // 64-column blocks per K tile
    constexpr int SR = (KB + NB - 1) / NB + 1;
    static_assert(VS >= 1 && VS <= 2, "the o_ready rotation covers a V ring of at most two tiles");
    static_assert((1 + 2 * KB + VS + 2 * SR + 4 + 4 + 2 + 1) * 8 + 4 <= 512, "barrier area");
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = smem + L::OFF_K;
    uint8_t* sV = smem + L::OFF_V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
    uint64_t* q_full = bars;            // [1]
    // Every tcgen05.commit costs tensor-pipe time, so a stream commits exactly twice per tile: s_full after its QK
    // and o_ready after its PV.  The same two barriers also tell the producers when ring slots are free again,
    // which is why they rotate over SR (resp. 2) barriers: a producer may look at a tile's barrier long after the
    // softmax did, and the rotation keeps the phase parity it tests unambiguous (the ring holds fewer than SR - 1
    // K tiles and VS = 2 V tiles, so the barrier cannot have been reused twice in between).
    uint64_t* k_full = bars + 1;        // [KB]: one per 64-column block of the K ring
    uint64_t* v_full = k_full + KB;     // [VS]
    uint64_t* s_full = v_full + VS;     // [2 streams][SR]: S of local tile jl is in TMEM (its K blocks are consumed)
    uint64_t* p_full = s_full + 2 * SR; // [2][2]: P of keys 0-63 / 64-127 of the current tile is in TMEM
    uint64_t* o_ready = p_full + 4;     // [2][2]: PV of local tile jl has retired (its V tile is consumed)
    uint64_t* sm_done = o_ready + 4;    // [2]: a stream's softmax warpgroup has finished the exponentials of a tile
    uint64_t* s_free = sm_done + 2;     // [1]: the shared S buffer has been copied into registers (one arrival per softmax warp)
    uint64_t* k_free = s_free + 1;      // [KB]: the last QK that reads this K block has retired
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(k_free + KB);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef INF_KPROF
    const long long kp_cta = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (tid == 0 && p.kprof_cta && kp_cta < 8192) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        p.kprof_cta[kp_cta * 5 + 0] = smid;
        p.kprof_cta[kp_cta * 5 + 1] = (long long)global_timer_ns();
    }
#endif
    // Set-up that needs nothing from global memory comes first, so that under a programmatic dependent launch
    // it overlaps the tail of the kernel before this one (the fused RoPE + append of the same prompt).
    const bool smem_ok = (smem_u32(smem) & 1023u) == 0;  // the swizzled tiles need a 1024-byte aligned base
    if (tid == 0 && smem_ok) {
        mbar_init(q_full, 1);
        for (int i = 0; i < KB; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_free[i], 1);
        }
        for (int i = 0; i < VS; ++i) mbar_init(&v_full[i], 1);
        for (int i = 0; i < 2 * SR; ++i) mbar_init(&s_full[i], 1);
        for (int i = 0; i < 4; ++i) mbar_init(&o_ready[i], 1);
        // the softmax barriers take one arrival per warp: tcgen05.wait is warp-wide, so lane 0 can speak for its warp
        for (int i = 0; i < 4; ++i) mbar_init(&p_full[i], 4);
        mbar_init(&sm_done[0], 4);
        mbar_init(&sm_done[1], 4);
        mbar_init(s_free, 4);
        mbar_fence_init();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 8 && lane == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    inf_pdl_wait();  // Q, the appended K/V rows and the page table come from work earlier in the stream
    inf_pdl_release();

    const int b = blockIdx.z;
    const int past = PAGED ? p.lens[b] : 0;
    const int kv_total = past + p.tokens;
    // work item -> (head or head pair, query tile or tile pair): groups of raster_heads heads, inside a group the
    // latest (heaviest) query rows first, the heads of the group side by side
    int item_head, qtile;
    {
        const int per_group = p.raster_heads * p.grid_tiles;
        const int grp = (int)blockIdx.x / per_group, within = (int)blockIdx.x % per_group;
        const int g_heads = min(p.raster_heads, p.grid_heads - grp * p.raster_heads);
        item_head = grp * p.raster_heads + within % g_heads;
        qtile = p.grid_tiles - 1 - within / g_heads;
    }

    Stream st[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        st[s].head = p.pair_heads ? 2 * item_head + s : item_head;
        st[s].q0 = p.pair_heads ? qtile * BM : (2 * qtile + s) * BM;
        if (st[s].q0 < p.tokens && st[s].head < p.q_heads) {
            const int q_last = min(st[s].q0 + BM, p.tokens) - 1;
            st[s].kt_end = (past + q_last + 1 + BN - 1) / BN;
            const int lo_key = p.window > 0 ? max(0, past + st[s].q0 + 1 - p.window) : 0;
            st[s].kt_begin = lo_key / BN;
        } else {
            st[s].kt_begin = st[s].kt_end = 0;
        }
    }
    const bool act0 = st[0].kt_end > st[0].kt_begin, act1 = st[1].kt_end > st[1].kt_begin;
    const int kt_lo = act0 && act1 ? min(st[0].kt_begin, st[1].kt_begin) : (act0 ? st[0].kt_begin : st[1].kt_begin);
    const int kt_hi = act0 && act1 ? max(st[0].kt_end, st[1].kt_end) : (act0 ? st[0].kt_end : st[1].kt_end);
    // a CTA with nothing to do (no rows, or a misaligned shared-memory base) runs every role with zero tiles
    const int n = (smem_ok && (act0 || act1)) ? kt_hi - kt_lo : 0;
    if (n == 0) st[0].kt_begin = st[0].kt_end = st[1].kt_begin = st[1].kt_end = 0;
    if (!smem_ok && tid == 0) atomicOr(p.status, INF_STATUS_BAD_SMEM);
    // Both streams start at the CTA's first key tile (with a sliding window the later rows' stream then sees one
    // fully masked tile, which contributes exact zeros): an issuer that skipped leading tiles would have to test
    // ring barriers whose phase it has not followed.
    if (n > 0 && act0) st[0].kt_begin = kt_lo;
    if (n > 0 && act1) st[1].kt_begin = kt_lo;
    // lowest key any row of this CTA can see: 16-token page tiles wholly below it are masked for every row and may
    // have been returned to the pool, so they are requested as zeros without looking at the page table
    const int q0_min = act0 && act1 ? min(st[0].q0, st[1].q0) : (act0 ? st[0].q0 : st[1].q0);
    const int lo_visible = p.window > 0 ? max(0, past + q0_min + 1 - p.window) : 0;
    // both streams of a CTA read the same KV head (pair_heads pairs lie inside one KV group)
    const int kvh = PAGED ? st[act0 ? 0 : 1].head / p.group : st[act0 ? 0 : 1].head;
#ifdef INF_KPROF
    if (tid == 0 && p.kprof_cta && kp_cta < 8192) p.kprof_cta[kp_cta * 5 + 2] = (long long)global_timer_ns();
#endif

    // 384 threads start with 168 registers each; the data-movement / issue warpgroup keeps 40 and the two softmax
    // warpgroups take the rest (256 * 232 + 128 * 40 = 384 * 168), so a 128-key S row fits in registers
    if (warp >= 8) setmaxnreg_dec<40>();

    if (warp == 8) {
        // ------------------------------------------------ Q + K producer
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, (uint32_t)((act0 ? 1 : 0) + (act1 ? 1 : 0)) * L::Q_BYTES);
#pragma unroll
            for (int s = 0; s < 2; ++s)
                if (st[s].kt_end > st[s].kt_begin)
#pragma unroll
                    for (int blk = 0; blk < DQK / 64; ++blk)
                        tma_load_3d(sQ + s * L::Q_BYTES + blk * BM * 128, &tm_q, blk * 64, st[s].head,
                                    b * p.tokens + st[s].q0, q_full);
        }
        const int oob_row = p.num_pages * p.kv_heads * p.page_size;
        int g = 0;  // running block index over the whole CTA: ring slot g % KB, phase (g / KB) & 1
        bool alive = true;
        for (int j = 0; j < n && alive; ++j) {
            const int k0 = (kt_lo + j) * BN;
            int y = oob_row;
            if (PAGED && lane < 8) {
                const int token = k0 + lane * 16;
                const int slot = token / p.page_size;
                if (token < kv_total && token + 16 > lo_visible && slot < p.max_pages) {
                    const int page = p.pages[(long long)b * p.max_pages + slot];
                    if (page >= 0 && page < p.num_pages)
                        y = (page * p.kv_heads + kvh) * p.page_size + token % p.page_size;
                    else
                        atomicOr(p.status, INF_STATUS_BAD_PAGE);
                }
            }
            int ys[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) ys[i] = __shfl_sync(0xffffffffu, y, i);
#pragma unroll
            for (int blk = 0; blk < NB; ++blk, ++g) {
                const int slot = g % KB;
                int ok = 1;
                if (lane == 0 && g >= KB)  // the slot held block g - KB: free once the last QK that reads it has retired
                    ok = mbar_wait(&k_free[slot], ((uint32_t)(g / KB - 1)) & 1u) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                    alive = false;
                    break;
                }
                if (lane == 0) {
                    uint8_t* dst = sK + slot * L::KBLK_BYTES;
                    mbar_arrive_expect_tx(&k_full[slot], L::KBLK_BYTES);
                    if (PAGED) {
#pragma unroll
                        for (int sub = 0; sub < 8; ++sub)
                            tma_load_2d(dst + sub * 2048, &tm_k, blk * 64, ys[sub], &k_full[slot]);
                    } else if (blk < 2) {
                        tma_load_3d(dst, &tm_k, blk * 64, kvh, k0, &k_full[slot]);  // no-rope dims of this head
                    } else {
                        tma_load_2d(dst, &tm_k2, 0, k0, &k_full[slot]);  // the rope tail shared by every head
                    }
                }
            }
        }
    } else if (warp == 10) {
        // ------------------------------------------------ V producer
        const int oob_row = p.num_pages * p.kv_heads * p.page_size;
        for (int j = 0; j < n; ++j) {
            const int k0 = (kt_lo + j) * BN;
            const int vs = j % VS;
            int y = oob_row;
            if (PAGED && lane < 8) {
                const int token = k0 + lane * 16;
                const int slot = token / p.page_size;
                if (token < kv_total && token + 16 > lo_visible && slot < p.max_pages) {
                    const int page = p.pages[(long long)b * p.max_pages + slot];
                    if (page >= 0 && page < p.num_pages) y = (page * p.kv_heads + kvh) * p.page_size + token % p.page_size;
                }
            }
            int ok = 1;
            if (lane == 0 && j >= VS) {
                // the slot held tile j - VS: free once every stream that uses it has retired its PV
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const int jl = j - VS - (st[s].kt_begin - kt_lo);
                    if (ok && jl >= 0 && jl < st[s].kt_end - st[s].kt_begin)
                        ok = mbar_wait(&o_ready[s * 2 + (jl & 1)], ((uint32_t)(jl >> 1)) & 1u) ? 1 : 0;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                break;
            }
            int ys[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) ys[i] = __shfl_sync(0xffffffffu, y, i);
            if (lane == 0) {
                uint8_t* dst = sV + vs * L::V_BYTES;
                mbar_arrive_expect_tx(&v_full[vs], L::V_BYTES);
                if (PAGED) {
#pragma unroll
                    for (int sub = 0; sub < 8; ++sub)
#pragma unroll
                        for (int blk = 0; blk < DV / 64; ++blk)
                            tma_load_2d(dst + blk * BN * 128 + sub * 2048, &tm_v, blk * 64, ys[sub], &v_full[vs]);
                } else {
#pragma unroll
                    for (int blk = 0; blk < DV / 64; ++blk)
                        tma_load_3d(dst + blk * BN * 128, &tm_v, blk * 64, kvh, k0, &v_full[vs]);
                }
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------ QK issuer (one thread): S_s(j) = Q_s K(j)^T into the
        // shared S buffer, in the fixed order (s, j) = (0,0) (1,0) (0,1) (1,1) ...  A QK only needs the buffer
        // (the previous S has been copied out by its softmax warpgroup) and its K blocks: it depends neither on
        // the same stream's softmax nor on its PV, so the next S is normally waiting when a softmax finishes.
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(BM, BN, 0, 0);
            constexpr uint32_t hi_k = umma_desc_hi(1024, UMMA_SW128);
            const uint32_t k_lo0 = umma_desc_lo(smem_u32(sK), 16);
            const uint32_t s_col = tbase + COL_S;
            bool ok = true;
#ifdef INF_KPROF
            const bool kp_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
            long long kp_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long kp_start = clock64();
#endif
            ok = mbar_wait(q_full, 0);
            uint32_t seq = 0;  // number of S tiles produced so far
            const int first[2] = {st[0].kt_begin - kt_lo, st[1].kt_begin - kt_lo};
            const int count[2] = {st[0].kt_end - st[0].kt_begin, st[1].kt_end - st[1].kt_begin};
            const uint32_t q_los[2] = {umma_desc_lo(smem_u32(sQ), 16), umma_desc_lo(smem_u32(sQ) + L::Q_BYTES, 16)};
#pragma unroll 1
            for (int j = 0; ok && j < n; ++j) {
#pragma unroll 1
                for (int s = 0; s < 2; ++s) {
                    const int jl = j - first[s];
                    if (jl < 0 || jl >= count[s]) continue;
                    KP_T0();
                    if (seq > 0) {
                        ok = mbar_wait(s_free, (seq - 1) & 1u);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    KP_ADD(0);
                    const uint32_t q_lo = q_los[s];
                    // K blocks go back to the producer one by one, after the last stream that reads them
                    const int jl1 = j - first[1];
                    const bool last_user = s == 1 || jl1 < 0 || jl1 >= count[1];
#pragma unroll
                    for (int blk = 0; blk < NB; ++blk) {
                        const int g = j * NB + blk;
                        const int slot = g % KB;
                        ok = mbar_wait(&k_full[slot], ((uint32_t)(g / KB)) & 1u);
                        KP_ADD(1);
                        if (!ok) break;
                        const uint32_t k_lo = k_lo0 + (uint32_t)slot * (L::KBLK_BYTES >> 4);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma_ss(s_col, umma_desc_pack(q_lo + ((blk * BM * 128 + kk * 32) >> 4), hi_k),
                                    umma_desc_pack(k_lo + ((kk * 32) >> 4), hi_k), idesc_qk, (blk > 0 || kk > 0) ? 1u : 0u);
                        if (last_user) tc_commit(&k_free[slot]);
                        KP_ADD(2);
                    }
                    if (!ok) break;
                    tc_commit(&s_full[s * SR + jl % SR]);
                    ++seq;
                }
            }
            if (!ok) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
#ifdef INF_KPROF
            if (kp_on && p.kprof) {
                for (int i = 0; i < 6; ++i) p.kprof[i] = kp_acc[i];
                p.kprof[6] = clock64() - kp_start;
                p.kprof[7] = n;
            }
#endif
        }
    } else if (warp == 11) {
        // ------------------------------------------------ PV issuer (one thread): O_s += P_s V(j), in the order the
        // softmax warpgroups produce P (stream 0 then stream 1 of every tile), each 64-key half as it arrives.
        if (lane == 0) {
            constexpr uint32_t idesc_pv = umma_idesc_f16(BM, DV, 0, 1);
            constexpr uint32_t hi_k = umma_desc_hi(1024, UMMA_SW128);
            const uint32_t v_lo0 = umma_desc_lo(smem_u32(sV), BN * 128);
            bool ok = true;
            const int first[2] = {st[0].kt_begin - kt_lo, st[1].kt_begin - kt_lo};
            const int count[2] = {st[0].kt_end - st[0].kt_begin, st[1].kt_end - st[1].kt_begin};
#ifdef INF_KPROF
            const bool kp_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
            long long kp_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long kp_start = clock64();
#endif
#pragma unroll 1
            for (int j = 0; ok && j < n; ++j) {
                const int vs = j % VS;
                KP_T0();
                ok = mbar_wait(&v_full[vs], ((uint32_t)(j / VS)) & 1u);
                KP_ADD(0);
                if (!ok) break;
                const uint32_t v_lo = v_lo0 + (uint32_t)vs * (L::V_BYTES >> 4);
#pragma unroll 1
                for (int s = 0; s < 2; ++s) {
                    const int jl = j - first[s];
                    if (jl < 0 || jl >= count[s]) continue;
                    const uint32_t p_col = tbase + COL_STREAM0 + s * STREAM_COLS + COL_P;
                    const uint32_t o_col = tbase + COL_STREAM0 + s * STREAM_COLS + COL_O;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {  // the two 64-key halves of P arrive separately
                        ok = mbar_wait(&p_full[s * 2 + h], ((uint32_t)jl) & 1u);
                        KP_ADD(1);
                        if (!ok) break;
                        tc_fence_after();
                        if (h == 0) {
                            const uint32_t acc0 = jl > 0 ? 1u : 0u;
#pragma unroll
                            for (int kk = 0; kk < BN / 32; ++kk)
                                umma_ts(o_col, p_col + kk * 8, umma_desc_pack(v_lo + kk * (2048 >> 4), hi_k), idesc_pv,
                                        kk > 0 ? 1u : acc0);
                        } else {
#pragma unroll
                            for (int kk = BN / 32; kk < BN / 16; ++kk)
                                umma_ts(o_col, p_col + kk * 8, umma_desc_pack(v_lo + kk * (2048 >> 4), hi_k), idesc_pv, 1u);
                        }
                        KP_ADD(2);
                    }
                    if (!ok) break;
                    tc_commit(&o_ready[s * 2 + (jl & 1)]);
                }
            }
            if (!ok) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
#ifdef INF_KPROF
            if (kp_on && p.kprof) {
                for (int i = 0; i < 6; ++i) p.kprof[8 + i] = kp_acc[i];
                p.kprof[8 + 6] = clock64() - kp_start;
            }
#endif
        }
    } else if (warp < 8) {
        setmaxnreg_inc<232>();
        // ------------------------------------------------ softmax + epilogue: thread = query row of its stream
        const int s = warp >> 2;
        const Stream me = st[s];
        const int n_s = me.kt_end - me.kt_begin;
        const int n_other = st[s ^ 1].kt_end - st[s ^ 1].kt_begin;
        if (n_s > 0) {
            const int r = tid & 127;
            const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
            const uint32_t col_s = tbase + lane_addr + COL_S;
            const uint32_t col0 = tbase + lane_addr + COL_STREAM0 + s * STREAM_COLS;
            const int qpos = past + me.q0 + r;
            const int first_key = p.window > 0 ? qpos + 1 - p.window : 0;
            float m_used = M_INIT, l = 0.f;
            bool ok = true;
#ifdef INF_KPROF
            const bool kp_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (tid & 127) == 0;
            long long kp_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long kp_start = clock64();
            const bool kp_tl = tid == 0 && p.kprof_cta && kp_cta < 8192 && p.kprof;  // timeline of every CTA's thread 0
            long long kp_ns[5] = {(long long)global_timer_ns(), 0, 0, 0, 0};
#endif
            for (int j = 0; j < n_s; ++j) {
                const int k0 = (me.kt_begin + j) * BN;
                KP_T0();
                if (!mbar_wait(&s_full[s * SR + j % SR], ((uint32_t)(j / SR)) & 1u)) {
                    ok = false;
                    break;
                }
                KP_ADD(0);
#ifdef INF_KPROF
                if (j == 0) kp_ns[1] = (long long)global_timer_ns();
#endif
                tc_fence_after();
                const bool need_mask = (k0 + BN - 1 > past + me.q0) || (k0 + BN > kv_total) ||
                                       (p.window > 0 && k0 < past + me.q0 + BM - p.window);
                // ---- the whole S row of this tile lives in registers (the softmax warpgroups run with 232 registers)
                uint32_t sraw[BN];
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) tmem_ld32(col_s + c * 32, sraw + c * 32);
                tc_wait_ld();
                tc_fence_before();
                if (lane == 0) mbar_arrive(s_free);  // the next QK (of either stream) may overwrite the buffer
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < BN; ++i) {
                        const int key = k0 + i;
                        if (key > qpos || key < first_key || key >= kv_total) sraw[i] = 0xff800000u;  // -inf
                    }
                }
                float mxs[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) mxs[i] = __uint_as_float(sraw[i]);
#pragma unroll
                for (int i = 8; i < BN; ++i) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(sraw[i]));
                const float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])),
                                       fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
                const float m_cand = fmaxf(m_used, mx * p.scale_log2);  // scale > 0, so max and scale commute
                KP_ADD(1);
                // ---- P(j) will overwrite P(j-1) and O may be rescaled: PV(j-1) must have retired (it normally has)
                if (j > 0) {
                    if (!mbar_wait(&o_ready[s * 2 + ((j - 1) & 1)], ((uint32_t)((j - 1) >> 1)) & 1u)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                }
                if (j == 0) {
                    m_used = m_cand;
                } else {
                    const bool need = (m_cand - m_used) > RESCALE_THRESHOLD;
                    if (__any_sync(0xffffffffu, need)) {
                        const float alpha = ex2_approx(m_used - m_cand);
                        m_used = m_cand;
                        l *= alpha;
#pragma unroll
                        for (int c = 0; c < DV / 32; ++c) {
                            uint32_t o[32];
                            tmem_ld32(col0 + COL_O + c * 32, o);
                            tc_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(col0 + COL_O + c * 32, o);
                        }
                        tc_wait_st();
                    }
                }
                KP_ADD(2);
                // The two streams take turns at the exponentials (0, 1, 0, 1, ... while both have tiles left): the
                // special-function unit is shared, and the turn order is the order in which the issuers serve them.
                // Only the dense instantiation: for the long MLA prompt turns and no turns measure the same
                // (19.8-19.9 ms), while the 2 048-token paged prompt runs 2.5 % faster without them (88.9 against
                // 91.1 us a step).
                if (!PAGED && (s == 0 ? (j >= 1 && j - 1 < n_other) : (j < n_other))) {
                    if (!mbar_wait(&sm_done[s ^ 1], ((uint32_t)(s == 0 ? j - 1 : j)) & 1u)) {
                        ok = false;
                        break;
                    }
                }
                KP_ADD(5);
                // ---- exponentials; the packed pairs overwrite the front of the same register array, and each
                //      32-key chunk of P is stored as soon as it is ready
                const float neg_m = -m_used;
                float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) {
#pragma unroll
                    for (int i = c * 32; i < c * 32 + 32; i += 2) {
                        const float p0 = ex2_approx(fmaf(__uint_as_float(sraw[i]), p.scale_log2, neg_m));
                        const float p1 = ex2_approx(fmaf(__uint_as_float(sraw[i + 1]), p.scale_log2, neg_m));
                        sums[(i >> 1) & 3] += p0 + p1;
                        sraw[i / 2] = pack_half2(p0, p1);
                    }
                    tmem_st16(col0 + COL_P + c * 16, sraw + c * 16);
                    if (c & 1) {  // a 64-key half of P is complete: its PV MMAs may start while the rest is computed
                        tc_wait_st();
                        tc_fence_before();
                        if (lane == 0) mbar_arrive(&p_full[s * 2 + (c >> 1)]);
                    }
                }
                l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
                KP_ADD(3);
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm_done[s]);
                KP_ADD(4);
            }
#ifdef INF_KPROF
            if (kp_on && p.kprof) {
                for (int i = 0; i < 6; ++i) p.kprof[16 + s * 8 + i] = kp_acc[i];
                p.kprof[16 + s * 8 + 6] = clock64() - kp_start;
                p.kprof[16 + s * 8 + 7] = n_s;
            }
#endif
#ifdef INF_KPROF
            kp_ns[2] = (long long)global_timer_ns();
#endif
            if (ok && !mbar_wait(&o_ready[s * 2 + ((n_s - 1) & 1)], ((uint32_t)((n_s - 1) >> 1)) & 1u)) ok = false;
#ifdef INF_KPROF
            kp_ns[3] = (long long)global_timer_ns();
#endif
            if (!ok) {
                if (lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
            } else {
                tc_fence_after();
                const bool valid = (me.q0 + r) < p.tokens;
                float gain = 1.0f / l;
                if (p.gate && valid)
                    gain *= softplus_ref(p.gate[((long long)b * p.tokens + me.q0 + r) * p.q_heads + me.head]);
                const long long obase =
                    (long long)b * p.o_bs + (long long)(me.q0 + r) * p.o_ts + (long long)me.head * p.o_hs;
                if (p.out_f16 && DV == 128) {
                    // fp16 rows go through this stream's Q tile (dead since its last QK^T): each thread parks its row
                    // there, then the warp writes its 32 rows back out as whole 256-byte lines.  16-byte chunks are
                    // XORed with the row so that neither pass collides on banks.
                    uint8_t* stage = sQ + s * L::Q_BYTES + (warp & 3) * (32 * 256);
#pragma unroll
                    for (int c = 0; c < DV / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld32(col0 + COL_O + c * 32, o);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 v;
                            v.x = pack_half2(__uint_as_float(o[i]) * gain, __uint_as_float(o[i + 1]) * gain);
                            v.y = pack_half2(__uint_as_float(o[i + 2]) * gain, __uint_as_float(o[i + 3]) * gain);
                            v.z = pack_half2(__uint_as_float(o[i + 4]) * gain, __uint_as_float(o[i + 5]) * gain);
                            v.w = pack_half2(__uint_as_float(o[i + 6]) * gain, __uint_as_float(o[i + 7]) * gain);
                            const int chunk = c * 4 + (i >> 3);
                            *reinterpret_cast<uint4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = v;
                        }
                    }
                    __syncwarp();
                    const int chunk = lane & 15;
#pragma unroll 4
                    for (int rr = 0; rr < 16; ++rr) {
                        const int row_l = rr * 2 + (lane >> 4);
                        const int row_g = me.q0 + (warp & 3) * 32 + row_l;
                        const uint4 v = *reinterpret_cast<const uint4*>(stage + row_l * 256 + ((chunk ^ (row_l & 15)) << 4));
                        if (row_g < p.tokens) {
                            const long long off = (long long)b * p.o_bs + (long long)row_g * p.o_ts + (long long)me.head * p.o_hs + chunk * 8;
                            *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.out) + off) = v;
                            for (int pr = 0; pr < p.n_peers; ++pr)
                                *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.peer_out[pr]) + off) = v;
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < DV / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld32(col0 + COL_O + c * 32, o);
                        tc_wait_ld();
                        if (valid) {
                            if (p.out_f16) {
                                __half* dst = reinterpret_cast<__half*>(p.out) + obase + c * 32;
#pragma unroll
                                for (int i = 0; i < 32; i += 8) {
                                    uint4 v;
                                    v.x = pack_half2(__uint_as_float(o[i]) * gain, __uint_as_float(o[i + 1]) * gain);
                                    v.y = pack_half2(__uint_as_float(o[i + 2]) * gain, __uint_as_float(o[i + 3]) * gain);
                                    v.z = pack_half2(__uint_as_float(o[i + 4]) * gain, __uint_as_float(o[i + 5]) * gain);
                                    v.w = pack_half2(__uint_as_float(o[i + 6]) * gain, __uint_as_float(o[i + 7]) * gain);
                                    *reinterpret_cast<uint4*>(dst + i) = v;
                                    for (int pr = 0; pr < p.n_peers; ++pr)
                                        *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.peer_out[pr]) + obase + c * 32 + i) = v;
                                }
                            } else {
                                float* dst = reinterpret_cast<float*>(p.out) + obase + c * 32;
#pragma unroll
                                for (int i = 0; i < 32; i += 4) {
                                    const float4 v = make_float4(__uint_as_float(o[i]) * gain, __uint_as_float(o[i + 1]) * gain,
                                                                 __uint_as_float(o[i + 2]) * gain, __uint_as_float(o[i + 3]) * gain);
                                    *reinterpret_cast<float4*>(dst + i) = v;
                                    for (int pr = 0; pr < p.n_peers; ++pr)
                                        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.peer_out[pr]) + obase + c * 32 + i) = v;
                                }
                            }
                        }
                    }
                }
            }
#ifdef INF_KPROF
            if (kp_tl) {
                kp_ns[4] = (long long)global_timer_ns();
                const long long e = p.kprof_cta[kp_cta * 5 + 1];
                // accumulate over CTAs (atomics): softmax loop start, first S, loop end, last PV retired, stores done
                for (int i = 0; i < 5; ++i) atomicAdd((unsigned long long*)&p.kprof[40 + i], (unsigned long long)(kp_ns[i] - e));
                atomicAdd((unsigned long long*)&p.kprof[45], 1ull);
                atomicAdd((unsigned long long*)&p.kprof[46], (unsigned long long)(clock64() - kp_start));
                atomicAdd((unsigned long long*)&p.kprof[47], (unsigned long long)(kp_ns[4] - kp_ns[0]));
            }
#endif
        }
    }
#ifdef INF_KPROF
    if (tid == 0 && p.kprof_cta && kp_cta < 8192) p.kprof_cta[kp_cta * 5 + 3] = (long long)global_timer_ns();
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tbase, TMEM_COLS);
#ifdef INF_KPROF
    if (tid == 32 * 9 && p.kprof_cta && kp_cta < 8192) p.kprof_cta[kp_cta * 5 + 4] = (long long)global_timer_ns();
#endif
}

template <int DQK, int DV, int KB, int VS, bool PAGED>
int launch_flash(inf_ctx* ctx, uint32_t attr_bit, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tk2,
                 const CUtensorMap& tv, const FlashParams& p, const char* name) {
    using L = SmemLayout<DQK, DV, KB, VS>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA per SM");
    auto kernel = flash_prefill_kernel<DQK, DV, KB, VS, PAGED>;
    if (!(ctx->func_attr_done & attr_bit)) {
        INF_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        ctx->func_attr_done |= attr_bit;
    }
    const int q_tiles = (p.tokens + BM - 1) / BM;
    FlashParams pp = p;
    pp.grid_heads = p.pair_heads ? p.q_heads / 2 : p.q_heads;
    pp.grid_tiles = p.pair_heads ? q_tiles : (q_tiles + 1) / 2;
    // Work items of a group of heads run together so that the K/V they stream stay in L2, latest (heaviest) rows first
    // inside a group.  Paged GQA prompts are short enough for every head's pages to fit.  Long dense prompts take the
    // smallest group that still holds about two waves of work items, so that the light items at the end of a group
    // fill the gaps the heavy ones leave.  Measured: at 32 768 tokens (128 items per head, groups of three heads)
    // groups of one to ten heads are within 1 % of each other and 12-14 % faster than all 64 heads in flight at once,
    // where the same K/V bytes crossed HBM four to five times; at 8 192 tokens (groups of ten) head-by-head order is
    // 4 % slower, because one head's tail is then a tenth of the run.
    pp.raster_heads = PAGED ? pp.grid_heads
                            : std::max(1, std::min(pp.grid_heads, (2 * ctx->sm_count + pp.grid_tiles - 1) / pp.grid_tiles));
    dim3 grid((unsigned)(pp.grid_heads * pp.grid_tiles), 1, p.batch);
#ifdef INF_KPROF
    static long long* d_kprof = nullptr;
    if (!d_kprof) cudaMalloc(&d_kprof, 64 * sizeof(long long));
    cudaMemsetAsync(d_kprof, 0, 64 * sizeof(long long), ctx->stream);
    pp.kprof = d_kprof;
    static long long* d_cta = nullptr;
    if (!d_cta) cudaMalloc(&d_cta, 8192 * 5 * sizeof(long long));
    cudaMemsetAsync(d_cta, 0, 8192 * 5 * sizeof(long long), ctx->stream);
    pp.kprof_cta = d_cta;
    kernel<<<grid, NUM_THREADS, L::TOTAL, ctx->stream>>>(tq, tk, tk2, tv, pp);
    long long h[64];
    cudaMemcpy(h, d_kprof, sizeof(h), cudaMemcpyDeviceToHost);
    fprintf(stderr, "KPROF %s qk issuer: wait_free %lld wait_k %lld issue %lld total %lld tiles %lld\n", name, h[0], h[1], h[2], h[6], h[7]);
    fprintf(stderr, "KPROF %s pv issuer: wait_v %lld wait_p %lld issue %lld total %lld\n", name, h[8], h[9], h[10], h[14]);
    for (int s2 = 0; s2 < 2; ++s2)
        fprintf(stderr, "KPROF %s softmax%d: wait_s %lld pass1 %lld rescale %lld pass2 %lld st+arrive %lld turn %lld total %lld tiles %lld\n",
                name, s2, h[16 + s2 * 8], h[16 + s2 * 8 + 1], h[16 + s2 * 8 + 2], h[16 + s2 * 8 + 3], h[16 + s2 * 8 + 4], h[16 + s2 * 8 + 5],
                h[16 + s2 * 8 + 6], h[16 + s2 * 8 + 7]);
    {   // per-SM schedule: where the time between and inside CTAs goes
        const int ncta = (int)std::min<long long>(8192, (long long)grid.x * grid.y * grid.z);
        std::vector<long long> c(ncta * 5);
        cudaMemcpy(c.data(), d_cta, c.size() * sizeof(long long), cudaMemcpyDeviceToHost);
        long long t0 = c[1], t1 = 0;
        for (int i = 0; i < ncta; ++i) { t0 = std::min(t0, c[i * 5 + 1]); t1 = std::max(t1, c[i * 5 + 4]); }
        std::vector<std::vector<int>> per_sm(256);
        for (int i = 0; i < ncta; ++i) per_sm[c[i * 5] & 255].push_back(i);
        double setup = 0, body = 0, tail = 0, gap = 0, idle_end = 0; int ngap = 0, nsm = 0;
        for (auto& v : per_sm) {
            if (v.empty()) continue;
            ++nsm;
            std::sort(v.begin(), v.end(), [&](int a, int b) { return c[a * 5 + 1] < c[b * 5 + 1]; });
            for (size_t k = 0; k < v.size(); ++k) {
                const long long* e = &c[v[k] * 5];
                setup += e[2] - e[1]; body += e[3] - e[2]; tail += e[4] - e[3];
                if (k > 0) { gap += e[1] - c[v[k - 1] * 5 + 4]; ++ngap; }
            }
            idle_end += t1 - c[v.back() * 5 + 4];
        }
        if (grid.y <= 64) {
            fprintf(stderr, "KPROF %s body us by blockIdx.y:", name);
            for (unsigned y = 0; y < grid.y; ++y) {
                double sum = 0; int cnt = 0;
                for (int i = 0; i < ncta; ++i)
                    if ((unsigned)((i / grid.x) % grid.y) == y) { sum += c[i * 5 + 3] - c[i * 5 + 2]; ++cnt; }
                fprintf(stderr, " %.1f", cnt ? sum / cnt * 1e-3 : 0.0);
            }
            fprintf(stderr, "\n");
        }
        fprintf(stderr, "KPROF %s thread-0 timeline, mean over %lld CTAs, us after CTA entry: softmax loop entered %.2f, first S %.2f, loop left %.2f, last PV retired %.2f, output stored %.2f\n",
                name, h[45], h[40] * 1e-3 / std::max(1ll, h[45]), h[41] * 1e-3 / std::max(1ll, h[45]), h[42] * 1e-3 / std::max(1ll, h[45]),
                h[43] * 1e-3 / std::max(1ll, h[45]), h[44] * 1e-3 / std::max(1ll, h[45]));
        fprintf(stderr, "KPROF %s SM clock inside the kernel: %.0f MHz (cycles / globaltimer over the softmax thread's life)\n", name,
                h[47] ? (double)h[46] / (double)h[47] * 1e3 : 0.0);
        fprintf(stderr, "KPROF %s schedule: span %.1f us, %d CTAs on %d SMs; per CTA: set-up %.2f us, body %.2f us, exit %.2f us; gap between CTAs on an SM %.2f us; idle at the end per SM %.2f us; first start spread n/a\n",
                name, (t1 - t0) * 1e-3, ncta, nsm, setup / ncta * 1e-3, body / ncta * 1e-3, tail / ncta * 1e-3,
                ngap ? gap / ngap * 1e-3 : 0.0, idle_end / nsm * 1e-3);
    }
    INF_LAUNCH_CHECK(ctx, name);
    return INF_OK;
#else
    {
        inf_prof_scope prof(ctx, name);
        INF_CUDA(ctx, inf_launch_pdl(kernel, grid, dim3(NUM_THREADS), (size_t)L::TOTAL, ctx->stream, tq, tk, tk2, tv, pp));
    }
    INF_LAUNCH_CHECK(ctx, name);
    return INF_OK;
#endif
}

}  // namespace

// Shared with the fused operator entry point.
// Where the rows go when the heads are sharded over ranks: the token stride of the gathered tensor (elements) and the
// other ranks' copies of it, each already offset to this rank's first head like `out` itself.
struct PrefillPeers {
    long long token_stride;
    void* const* outs;
    int count;
};

static int check_peers(inf_ctx* ctx, const PrefillPeers* peers, const char* what) {
    if (!peers) return INF_OK;
    if (peers->count < 0 || peers->count > INF_MAX_PEERS)
        return inf_fail(ctx, INF_E_CONFIG, "%s: %d peers, at most %d are supported", what, peers->count, INF_MAX_PEERS);
    if (peers->count > 0 && !peers->outs) return inf_fail(ctx, INF_E_ARG, "%s: null peer list", what);
    for (int i = 0; i < peers->count; ++i)
        if (!peers->outs[i] || (reinterpret_cast<uintptr_t>(peers->outs[i]) & 15u))
            return inf_fail(ctx, INF_E_ARG, "%s: peer output %d is null or not 16-byte aligned", what, i);
    return INF_OK;
}

int inf_gqa_prefill_launch(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                           int tokens, int q_heads, int sliding_window, const float* gate, float scale, void* out,
                           int out_dtype, const PrefillPeers* peers) {
    if (!q_f16 || !pool || !table || !out) return inf_fail(ctx, INF_E_ARG, "gqa_prefill: null pointer");
    if (!pool->k || !pool->v) return inf_fail(ctx, INF_E_ARG, "gqa_prefill: pool has no storage");
    if (pool->head_dim != 128) return inf_fail(ctx, INF_E_SHAPE, "gqa_prefill: head_dim must be 128, got %d", pool->head_dim);
    if (pool->page_size % 16 != 0) return inf_fail(ctx, INF_E_CACHE, "gqa_prefill: page_size must be a multiple of 16");
    if (tokens <= 0) return inf_fail(ctx, INF_E_SHAPE, "gqa_prefill: tokens must be positive");
    if (q_heads <= 0 || q_heads % pool->kv_heads != 0)
        return inf_fail(ctx, INF_E_SHAPE, "gqa_prefill: q_heads %d must be a positive multiple of kv_heads %d", q_heads,
                        pool->kv_heads);
    if (sliding_window < 0) return inf_fail(ctx, INF_E_CONFIG, "gqa_prefill: sliding_window must be >= 0");
    if (out_dtype != INF_DTYPE_F32 && out_dtype != INF_DTYPE_F16)
        return inf_fail(ctx, INF_E_DTYPE, "gqa_prefill: output dtype must be f32 or f16");
    int rc = inf_validate_table(ctx, table, pool->num_pages, pool->page_size, tokens, "gqa_prefill", sliding_window, tokens);
    if (rc != INF_OK) return rc;

    CUtensorMap tq, tk, tv;
    {
        uint64_t dims[3] = {128, (uint64_t)q_heads, (uint64_t)table->batch * tokens};
        uint64_t strides[2] = {128 * 2, (uint64_t)q_heads * 128 * 2};
        uint32_t box[3] = {64, 1, BM};
        rc = inf_make_tmap(ctx, q_f16, 3, dims, strides, box, &tq);
        if (rc != INF_OK) return rc;
    }
    {
        uint64_t dims[2] = {128, (uint64_t)pool->num_pages * pool->kv_heads * pool->page_size};
        uint64_t strides[1] = {128 * 2};
        uint32_t box[2] = {64, 16};
        rc = inf_make_tmap(ctx, pool->k, 2, dims, strides, box, &tk);
        if (rc != INF_OK) return rc;
        rc = inf_make_tmap(ctx, pool->v, 2, dims, strides, box, &tv);
        if (rc != INF_OK) return rc;
    }
    FlashParams p{};
    p.tokens = tokens;
    p.q_heads = q_heads;
    p.kv_heads = pool->kv_heads;
    p.group = q_heads / pool->kv_heads;
    p.pair_heads = (p.group % 2 == 0) ? 1 : 0;
    p.batch = table->batch;
    p.pages = table->pages;
    p.lens = table->lens;
    p.max_pages = table->max_pages;
    p.page_size = pool->page_size;
    p.num_pages = pool->num_pages;
    p.window = sliding_window;
    p.scale_log2 = (scale > 0.f ? scale : 1.0f / sqrtf(128.0f)) * 1.4426950408889634f;
    p.gate = gate;
    p.out = out;
    p.out_f16 = out_dtype == INF_DTYPE_F16;
    p.o_hs = 128;
    p.o_ts = (long long)q_heads * 128;
    if (peers) {
        rc = check_peers(ctx, peers, "gqa_prefill");
        if (rc != INF_OK) return rc;
        if (peers->token_stride < (long long)q_heads * 128 || peers->token_stride % 8)
            return inf_fail(ctx, INF_E_SHAPE, "gqa_prefill: output token stride %lld must be a multiple of 8 and at least %d",
                            peers->token_stride, q_heads * 128);
        p.o_ts = peers->token_stride;
        p.n_peers = peers->count;
        for (int i = 0; i < peers->count; ++i) p.peer_out[i] = peers->outs[i];
    }
    p.o_bs = (long long)tokens * p.o_ts;
    p.status = ctx->status;
    return launch_flash<128, 128, 6, 2, true>(ctx, 2u, tq, tk, tk, tv, p, "flash_prefill_gqa_kernel");
}

extern "C" int32_t inf_gqa_prefill_paged(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                         const inf_page_table* table, int32_t tokens, int32_t q_heads,
                                         int32_t sliding_window, const float* gate, float scale, void* out,
                                         int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
    return inf_gqa_prefill_launch(ctx, q_f16, pool, table, tokens, q_heads, sliding_window, gate, scale, out,
                                  out_dtype, nullptr);
}

extern "C" int32_t inf_gqa_prefill_paged_peers(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                               const inf_page_table* table, int32_t tokens, int32_t q_heads,
                                               int32_t sliding_window, const float* gate, float scale, void* out,
                                               int32_t out_dtype, int64_t out_token_stride, void* const* peer_outs,
                                               int32_t n_peers) {
    INF_CHECK_CTX(ctx);
    const PrefillPeers peers = {out_token_stride, peer_outs, n_peers};
    return inf_gqa_prefill_launch(ctx, q_f16, pool, table, tokens, q_heads, sliding_window, gate, scale, out,
                                  out_dtype, &peers);
}

static int mla_prefill_any(inf_ctx* ctx, const void* q, int64_t q_ts, int64_t q_hs, const void* k_nope, int64_t kn_ts,
                           int64_t kn_hs, const void* k_rope, int64_t kr_ts, const void* v, int64_t v_ts, int64_t v_hs,
                           int32_t tokens, int32_t heads, int32_t nope_dim, int32_t rope_dim, int32_t v_dim, float scale,
                           void* out, int64_t o_ts, int64_t o_hs, int32_t out_dtype, const PrefillPeers* peers) {
    if (!q || !k_nope || !v || !out) return inf_fail(ctx, INF_E_ARG, "mla_prefill: null pointer");
    if (tokens <= 0 || heads <= 0) return inf_fail(ctx, INF_E_SHAPE, "mla_prefill: sizes must be positive");
    if (nope_dim != 128 || v_dim != 128 || (rope_dim != 64 && rope_dim != 0)) return INF_UNSUPPORTED;
    if (rope_dim && !k_rope) return inf_fail(ctx, INF_E_ARG, "mla_prefill: null rope tail");
    if (!(scale > 0.f)) return inf_fail(ctx, INF_E_CONFIG, "mla_prefill: scale must be positive");
    if (out_dtype != INF_DTYPE_F32 && out_dtype != INF_DTYPE_F16)
        return inf_fail(ctx, INF_E_DTYPE, "mla_prefill: output dtype must be f32 or f16");
    const int dqk = nope_dim + rope_dim;
    CUtensorMap tq, tk, tk2, tv;
    int rc;
    {
        uint64_t dims[3] = {(uint64_t)dqk, (uint64_t)heads, (uint64_t)tokens};
        uint64_t strides[2] = {(uint64_t)q_hs * 2, (uint64_t)q_ts * 2};
        uint32_t box[3] = {64, 1, BM};
        rc = inf_make_tmap(ctx, q, 3, dims, strides, box, &tq);
        if (rc != INF_OK) return rc;
    }
    {
        uint64_t dims[3] = {(uint64_t)nope_dim, (uint64_t)heads, (uint64_t)tokens};
        uint64_t strides[2] = {(uint64_t)kn_hs * 2, (uint64_t)kn_ts * 2};
        uint32_t box[3] = {64, 1, BN};
        rc = inf_make_tmap(ctx, k_nope, 3, dims, strides, box, &tk);
        if (rc != INF_OK) return rc;
    }
    if (rope_dim) {
        uint64_t dims[2] = {(uint64_t)rope_dim, (uint64_t)tokens};
        uint64_t strides[1] = {(uint64_t)kr_ts * 2};
        uint32_t box[2] = {64, BN};
        rc = inf_make_tmap(ctx, k_rope, 2, dims, strides, box, &tk2);
        if (rc != INF_OK) return rc;
    } else {
        tk2 = tk;
    }
    {
        uint64_t dims[3] = {(uint64_t)v_dim, (uint64_t)heads, (uint64_t)tokens};
        uint64_t strides[2] = {(uint64_t)v_hs * 2, (uint64_t)v_ts * 2};
        uint32_t box[3] = {64, 1, BN};
        rc = inf_make_tmap(ctx, v, 3, dims, strides, box, &tv);
        if (rc != INF_OK) return rc;
    }
    FlashParams p{};
    p.tokens = tokens;
    p.q_heads = heads;
    p.kv_heads = heads;
    p.group = 1;
    p.pair_heads = 0;
    p.batch = 1;
    p.window = 0;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = out;
    p.out_f16 = out_dtype == INF_DTYPE_F16;
    p.o_ts = o_ts;
    p.o_hs = o_hs;
    p.o_bs = 0;
    if (peers) {
        rc = check_peers(ctx, peers, "mla_prefill");
        if (rc != INF_OK) return rc;
        if ((o_ts % 8) || (o_hs % 8)) return inf_fail(ctx, INF_E_SHAPE, "mla_prefill: output strides must be multiples of 8");
        p.n_peers = peers->count;
        for (int i = 0; i < peers->count; ++i) p.peer_out[i] = peers->outs[i];
    }
    p.status = ctx->status;
    if (rope_dim) return launch_flash<192, 128, 4, 2, false>(ctx, 4u, tq, tk, tk2, tv, p, "flash_prefill_mla_kernel");
    return launch_flash<128, 128, 6, 2, false>(ctx, 8u, tq, tk, tk2, tv, p, "flash_prefill_mha_kernel");
}

extern "C" int32_t inf_mla_prefill_causal(inf_ctx* ctx, const void* q, int64_t q_ts, int64_t q_hs, const void* k_nope,
                                          int64_t kn_ts, int64_t kn_hs, const void* k_rope, int64_t kr_ts,
                                          const void* v, int64_t v_ts, int64_t v_hs, int32_t tokens, int32_t heads,
                                          int32_t nope_dim, int32_t rope_dim, int32_t v_dim, float scale, void* out,
                                          int64_t o_ts, int64_t o_hs, int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
    return mla_prefill_any(ctx, q, q_ts, q_hs, k_nope, kn_ts, kn_hs, k_rope, kr_ts, v, v_ts, v_hs, tokens, heads, nope_dim,
                           rope_dim, v_dim, scale, out, o_ts, o_hs, out_dtype, nullptr);
}

extern "C" int32_t inf_mla_prefill_causal_peers(inf_ctx* ctx, const void* q, int64_t q_ts, int64_t q_hs,
                                                const void* k_nope, int64_t kn_ts, int64_t kn_hs, const void* k_rope,
                                                int64_t kr_ts, const void* v, int64_t v_ts, int64_t v_hs, int32_t tokens,
                                                int32_t heads, int32_t nope_dim, int32_t rope_dim, int32_t v_dim,
                                                float scale, void* out, int64_t o_ts, int64_t o_hs, int32_t out_dtype,
                                                void* const* peer_outs, int32_t n_peers) {
    INF_CHECK_CTX(ctx);
    const PrefillPeers peers = {o_ts, peer_outs, n_peers};
    return mla_prefill_any(ctx, q, q_ts, q_hs, k_nope, kn_ts, kn_hs, k_rope, kr_ts, v, v_ts, v_hs, tokens, heads, nope_dim,
                           rope_dim, v_dim, scale, out, o_ts, o_hs, out_dtype, &peers);
}

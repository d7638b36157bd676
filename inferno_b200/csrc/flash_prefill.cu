// Causal flash attention for prefill on tcgen05 / TMEM, fed by TMA.
//
// One CTA per SM runs TWO query streams of 128 rows each against one shared ring of K/V tiles, so
// every K/V tile is fetched once for 256 query rows and the tensor pipe always has the other
// stream's MMAs to run while one stream is in softmax.  The two streams are either two query heads
// of the same KV group at the same rows (GQA: identical causal structure, perfectly balanced) or
// two consecutive 128-row tiles of one head (MHA / MLA prefill).
//
// Twelve warps, specialised:
//   warps 0-3   softmax + epilogue of stream 0; thread r owns query row r and TMEM lane r
//   warps 4-7   the same for stream 1
//   warp 8      TMA producer for Q and the K tiles
//   warp 9      allocates TMEM and issues every tcgen05.mma
//   warp 10     TMA producer for the V tiles            (warp 11 only pads the third warpgroup)
// Per stream and 64-key tile:  S = Q K^T  (SS MMA, M128 N64, both operands K-major, 128-byte swizzle)
//                              softmax in registers, P written back to TMEM as packed fp16 over its S buffer
//                              O += P V   (TS MMA, A = P from TMEM, B = V MN-major from its [key][dim] tile)
// TMEM: 256 columns per stream (S double-buffered in 0-63 / 64-127, O in 128-255).  O is rescaled lazily
// (only when a row maximum grew by more than 2^8).  The K/V ring is 5 (GQA) or 3 (MLA) tiles deep,
// enough to cover L2/HBM latency at one tile per ~1000 cycles.
//
// Two instantiations: paged GQA prefill (head_dim 128; a K/V tile is four 16-token page boxes addressed
// through the page table; reference kernel f16_attention_kernels.metal:153-316) and dense MLA prefill
// over expanded heads (qk 128+64 with the rope tail shared by all heads, v 128; reference kernel
// attention_kernels.metal:723-968 with no past, K laid out as in layout_kernels.metal:148-183).
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"
#include "ptx.cuh"

using namespace inf;

namespace {

constexpr int BM = 128;
constexpr int BN = 64;
constexpr int NUM_THREADS = 384;
constexpr float M_INIT = -1.0e30f;
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t STREAM_COLS = 256, COL_S0 = 0, COL_S1 = 64, COL_O = 128;

struct FlashParams {
    int tokens, q_heads, kv_heads, group, batch;
    int pair_heads;  // 1: streams are heads (2c, 2c+1) at the same rows; 0: streams are row tiles (2c, 2c+1) of one head
    const int* pages;
    const int* lens;
    int max_pages, page_size, num_pages;
    int window;
    float scale_log2;
    const float* gate;  // [batch][tokens][q_heads] or null
    void* out;
    int out_f16;
    long long o_ts, o_hs, o_bs;  // element strides of the output: token, head, batch
    int* status;
};

// kernels/fp8_attention_kernels.metal:56-64
__device__ __forceinline__ float softplus_ref(float v) {
    if (v > 20.0f) return v;
    if (v < -20.0f) return expf(v);
    return logf(1.0f + expf(v));
}

template <int DQK, int DV, int KS, int VS>
struct SmemLayout {
    static constexpr int Q_BYTES = BM * DQK * 2;  // per stream
    static constexpr int K_BYTES = BN * DQK * 2;
    static constexpr int V_BYTES = BN * DV * 2;
    static constexpr int OFF_K = 2 * Q_BYTES;
    static constexpr int OFF_V = OFF_K + KS * K_BYTES;
    static constexpr int OFF_BAR = OFF_V + VS * V_BYTES;
    static constexpr int TOTAL = OFF_BAR + 512;
};

struct Stream {
    int head, q0, kt_begin, kt_end;  // key-tile range [kt_begin, kt_end); empty when the stream has no rows
};

template <int DQK, int DV, int KS, int VS, bool PAGED>
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_k2, const __grid_constant__ CUtensorMap tm_v,
                     FlashParams p) {
    using L = SmemLayout<DQK, DV, KS, VS>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = smem + L::OFF_K;
    uint8_t* sV = smem + L::OFF_V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
    uint64_t* q_full = bars;            // [1]
    uint64_t* k_full = bars + 1;        // [KS]
    uint64_t* k_empty = k_full + KS;    // [KS]
    uint64_t* v_full = k_empty + KS;    // [VS]
    uint64_t* v_empty = v_full + VS;    // [VS]
    uint64_t* s_full = v_empty + VS;    // [2 streams][2 buffers]
    uint64_t* p_full = s_full + 4;      // [2][2]
    uint64_t* o_ready = p_full + 4;     // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_ready + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.z;
    const int past = PAGED ? p.lens[b] : 0;
    const int kv_total = past + p.tokens;
    const int qtile = (int)gridDim.y - 1 - (int)blockIdx.y;  // heaviest (latest) query rows first

    Stream st[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        st[s].head = p.pair_heads ? 2 * (int)blockIdx.x + s : (int)blockIdx.x;
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
    if (!act0 && !act1) return;
    const int kt_lo = act0 && act1 ? min(st[0].kt_begin, st[1].kt_begin) : (act0 ? st[0].kt_begin : st[1].kt_begin);
    const int kt_hi = act0 && act1 ? max(st[0].kt_end, st[1].kt_end) : (act0 ? st[0].kt_end : st[1].kt_end);
    const int n = kt_hi - kt_lo;
    // both streams of a CTA read the same KV head (pair_heads pairs lie inside one KV group)
    const int kvh = PAGED ? st[act0 ? 0 : 1].head / p.group : st[act0 ? 0 : 1].head;

    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base
        if (tid == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
        return;
    }
    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < KS; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
        }
        for (int i = 0; i < VS; ++i) {
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
        }
        mbar_init(&o_ready[0], 1);
        mbar_init(&o_ready[1], 1);
        mbar_fence_init();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;

    if (warp == 8) {
        // ------------------------------------------------ Q + K producer
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
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
        for (int j = 0; j < n; ++j) {
            const int k0 = (kt_lo + j) * BN;
            const int ks = j % KS;
            int y = oob_row;
            if (PAGED && lane < 4) {
                const int token = k0 + lane * 16;
                const int slot = token / p.page_size;
                if (token < kv_total && slot < p.max_pages) {
                    const int page = p.pages[(long long)b * p.max_pages + slot];
                    if (page >= 0 && page < p.num_pages)
                        y = (page * p.kv_heads + kvh) * p.page_size + token % p.page_size;
                    else
                        atomicOr(p.status, INF_STATUS_BAD_PAGE);
                }
            }
            int ok = 1;
            if (lane == 0) ok = mbar_wait(&k_empty[ks], (((uint32_t)(j / KS)) & 1u) ^ 1u) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                break;
            }
            const int y0 = __shfl_sync(0xffffffffu, y, 0), y1 = __shfl_sync(0xffffffffu, y, 1);
            const int y2 = __shfl_sync(0xffffffffu, y, 2), y3 = __shfl_sync(0xffffffffu, y, 3);
            if (lane == 0) {
                uint8_t* dst = sK + ks * L::K_BYTES;
                mbar_arrive_expect_tx(&k_full[ks], L::K_BYTES);
                if (PAGED) {
                    const int ys[4] = {y0, y1, y2, y3};
#pragma unroll
                    for (int sub = 0; sub < 4; ++sub)
#pragma unroll
                        for (int blk = 0; blk < DQK / 64; ++blk)
                            tma_load_2d(dst + blk * BN * 128 + sub * 2048, &tm_k, blk * 64, ys[sub], &k_full[ks]);
                } else {
                    // 128 no-rope dims of this head, then the 64-dim rope tail shared by every head
                    tma_load_3d(dst, &tm_k, 0, kvh, k0, &k_full[ks]);
                    tma_load_3d(dst + BN * 128, &tm_k, 64, kvh, k0, &k_full[ks]);
                    if (DQK == 192) tma_load_2d(dst + 2 * BN * 128, &tm_k2, 0, k0, &k_full[ks]);
                }
            }
        }
    } else if (warp == 10) {
        // ------------------------------------------------ V producer
        if (lane == 0) tma_prefetch_desc(&tm_v);
        const int oob_row = p.num_pages * p.kv_heads * p.page_size;
        for (int j = 0; j < n; ++j) {
            const int k0 = (kt_lo + j) * BN;
            const int vs = j % VS;
            int y = oob_row;
            if (PAGED && lane < 4) {
                const int token = k0 + lane * 16;
                const int slot = token / p.page_size;
                if (token < kv_total && slot < p.max_pages) {
                    const int page = p.pages[(long long)b * p.max_pages + slot];
                    if (page >= 0 && page < p.num_pages) y = (page * p.kv_heads + kvh) * p.page_size + token % p.page_size;
                }
            }
            int ok = 1;
            if (lane == 0) ok = mbar_wait(&v_empty[vs], (((uint32_t)(j / VS)) & 1u) ^ 1u) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                break;
            }
            const int y0 = __shfl_sync(0xffffffffu, y, 0), y1 = __shfl_sync(0xffffffffu, y, 1);
            const int y2 = __shfl_sync(0xffffffffu, y, 2), y3 = __shfl_sync(0xffffffffu, y, 3);
            if (lane == 0) {
                uint8_t* dst = sV + vs * L::V_BYTES;
                mbar_arrive_expect_tx(&v_full[vs], L::V_BYTES);
                if (PAGED) {
                    const int ys[4] = {y0, y1, y2, y3};
#pragma unroll
                    for (int sub = 0; sub < 4; ++sub)
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
        // ------------------------------------------------ MMA issuer (one thread)
        // Everything this thread does between two MMAs delays the tensor pipe, so descriptors are kept as
        // precomputed 32-bit words that only receive compile-time offsets, and ring indices and phases are
        // carried incrementally instead of being recomputed with divisions.
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(BM, BN, 0, 0);
            constexpr uint32_t idesc_pv = umma_idesc_f16(BM, DV, 0, 1);
            constexpr uint32_t hi_k = umma_desc_hi(1024, UMMA_SW128);
            const uint32_t q_lo[2] = {umma_desc_lo(smem_u32(sQ), 16), umma_desc_lo(smem_u32(sQ) + L::Q_BYTES, 16)};
            const uint32_t k_lo0 = umma_desc_lo(smem_u32(sK), 16);
            const uint32_t v_lo0 = umma_desc_lo(smem_u32(sV), BN * 128);
            // per stream: first CTA tile index and tile count, so that "active" and "local index" are cheap
            const int first[2] = {st[0].kt_begin - kt_lo, st[1].kt_begin - kt_lo};
            const int count[2] = {st[0].kt_end - st[0].kt_begin, st[1].kt_end - st[1].kt_begin};
            auto issue_qk = [&](int j, int ks) {
                const uint32_t k_lo = k_lo0 + (uint32_t)ks * (L::K_BYTES >> 4);
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const int jl = j - first[s];
                    if (jl < 0 || jl >= count[s]) continue;
                    const uint32_t s_col = tbase + s * STREAM_COLS + ((jl & 1) ? COL_S1 : COL_S0);
#pragma unroll
                    for (int kk = 0; kk < DQK / 16; ++kk) {
                        const uint32_t a_off = ((kk / 4) * BM * 128 + (kk % 4) * 32) >> 4;
                        const uint32_t b_off = ((kk / 4) * BN * 128 + (kk % 4) * 32) >> 4;
                        umma_ss(s_col, umma_desc_pack(q_lo[s] + a_off, hi_k), umma_desc_pack(k_lo + b_off, hi_k),
                                idesc_qk, kk > 0 ? 1u : 0u);
                    }
                    tc_commit(&s_full[s * 2 + (jl & 1)]);
                }
                tc_commit(&k_empty[ks]);
            };
            bool ok = mbar_wait(q_full, 0);
            if (ok) ok = mbar_wait(&k_full[0], 0);
            if (ok) {
                tc_fence_after();
                issue_qk(0, 0);
            }
            int ks_next = KS > 1 ? 1 : 0;
            uint32_t k_phase = KS > 1 ? 0u : 1u;  // phase of the stage that tile j+1 lands in
            int vs = 0;
            uint32_t v_phase = 0u;
            for (int j = 0; ok && j < n; ++j) {
                if (j + 1 < n) {
                    ok = mbar_wait(&k_full[ks_next], k_phase);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(j + 1, ks_next);
                    if (++ks_next == KS) {
                        ks_next = 0;
                        k_phase ^= 1u;
                    }
                }
                ok = mbar_wait(&v_full[vs], v_phase);
                if (!ok) break;
                const uint32_t v_lo = v_lo0 + (uint32_t)vs * (L::V_BYTES >> 4);
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const int jl = j - first[s];
                    if (jl < 0 || jl >= count[s]) continue;
                    ok = mbar_wait(&p_full[s * 2 + (jl & 1)], ((uint32_t)(jl >> 1)) & 1u);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t o_col = tbase + s * STREAM_COLS + COL_O;
                    const uint32_t p_col = tbase + s * STREAM_COLS + ((jl & 1) ? COL_S1 : COL_S0);
                    if (jl == 0) {
#pragma unroll
                        for (int kk = 0; kk < BN / 16; ++kk)
                            umma_ts(o_col, p_col + kk * 8, umma_desc_pack(v_lo + kk * (2048 >> 4), hi_k), idesc_pv,
                                    kk > 0 ? 1u : 0u);
                    } else {
#pragma unroll
                        for (int kk = 0; kk < BN / 16; ++kk)
                            umma_ts(o_col, p_col + kk * 8, umma_desc_pack(v_lo + kk * (2048 >> 4), hi_k), idesc_pv, 1u);
                    }
                    tc_commit(&o_ready[s]);
                }
                if (!ok) break;
                tc_commit(&v_empty[vs]);
                if (++vs == VS) {
                    vs = 0;
                    v_phase ^= 1u;
                }
            }
            if (!ok) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
        }
    } else if (warp < 8) {
        // ------------------------------------------------ softmax + epilogue: thread = query row of its stream
        const int s = warp >> 2;
        const Stream me = st[s];
        const int n_s = me.kt_end - me.kt_begin;
        if (n_s > 0) {
            const int r = tid & 127;
            const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
            const uint32_t col0 = tbase + lane_addr + s * STREAM_COLS;
            const int qpos = past + me.q0 + r;
            float m_used = M_INIT, l = 0.f;
            bool ok = true;
            for (int j = 0; j < n_s; ++j) {
                const int k0 = (me.kt_begin + j) * BN;
                const uint32_t buf_col = (j & 1) ? COL_S1 : COL_S0;
                if (!mbar_wait(&s_full[s * 2 + (j & 1)], ((uint32_t)(j >> 1)) & 1u)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                uint32_t sraw[BN];
                tmem_ld32(col0 + buf_col, sraw);
                tmem_ld32(col0 + buf_col + 32, sraw + 32);
                tc_wait_ld();
                const bool need_mask = (k0 + BN - 1 > past + me.q0) || (k0 + BN > kv_total) ||
                                       (p.window > 0 && k0 < past + me.q0 + BM - p.window);
                if (need_mask) {
                    const int first = p.window > 0 ? qpos + 1 - p.window : 0;
#pragma unroll
                    for (int i = 0; i < BN; ++i) {
                        const int key = k0 + i;
                        if (key > qpos || key < first || key >= kv_total) sraw[i] = 0xff800000u;  // -inf
                    }
                }
                // row maximum: eight independent chains, then a short tree (keeps the dependent path short)
                float mxs[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) mxs[i] = __uint_as_float(sraw[i]);
#pragma unroll
                for (int i = 8; i < BN; ++i) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(sraw[i]));
                const float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])),
                                       fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
                const float m_cand = fmaxf(m_used, mx * p.scale_log2);  // scale > 0, so max and scale commute
                if (j == 0) {
                    m_used = m_cand;
                } else {
                    const bool need = (m_cand - m_used) > RESCALE_THRESHOLD;
                    if (__any_sync(0xffffffffu, need)) {
                        const float alpha = ex2_approx(m_used - m_cand);
                        m_used = m_cand;
                        l *= alpha;
                        if (!mbar_wait(&o_ready[s], ((uint32_t)(j - 1)) & 1u)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
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
                // exponentials in two halves of 32 keys; each half of P is stored as soon as it is packed
                const float neg_m = -m_used;
                float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2_approx(fmaf(__uint_as_float(sraw[half * 32 + i]), p.scale_log2, neg_m));
                        const float p1 = ex2_approx(fmaf(__uint_as_float(sraw[half * 32 + i + 1]), p.scale_log2, neg_m));
                        sums[(i >> 1) & 3] += p0 + p1;
                        packed[i / 2] = pack_half2(p0, p1);
                    }
                    tmem_st16(col0 + buf_col + half * 16, packed);
                }
                l += (sums[0] + sums[1]) + (sums[2] + sums[3]);
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(&p_full[s * 2 + (j & 1)]);
            }
            if (ok && !mbar_wait(&o_ready[s], ((uint32_t)(n_s - 1)) & 1u)) ok = false;
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
                            }
                        } else {
                            float* dst = reinterpret_cast<float*>(p.out) + obase + c * 32;
#pragma unroll
                            for (int i = 0; i < 32; i += 4)
                                *reinterpret_cast<float4*>(dst + i) =
                                    make_float4(__uint_as_float(o[i]) * gain, __uint_as_float(o[i + 1]) * gain,
                                                __uint_as_float(o[i + 2]) * gain, __uint_as_float(o[i + 3]) * gain);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tbase, TMEM_COLS);
}

template <int DQK, int DV, int KS, int VS, bool PAGED>
int launch_flash(inf_ctx* ctx, uint32_t attr_bit, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tk2,
                 const CUtensorMap& tv, const FlashParams& p, const char* name) {
    using L = SmemLayout<DQK, DV, KS, VS>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA per SM");
    auto kernel = flash_prefill_kernel<DQK, DV, KS, VS, PAGED>;
    if (!(ctx->func_attr_done & attr_bit)) {
        INF_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        ctx->func_attr_done |= attr_bit;
    }
    const int q_tiles = (p.tokens + BM - 1) / BM;
    dim3 grid(p.pair_heads ? p.q_heads / 2 : p.q_heads, p.pair_heads ? q_tiles : (q_tiles + 1) / 2, p.batch);
    {
        inf_prof_scope prof(ctx, name);
        kernel<<<grid, NUM_THREADS, L::TOTAL, ctx->stream>>>(tq, tk, tk2, tv, p);
    }
    INF_LAUNCH_CHECK(ctx, name);
    return INF_OK;
}

}  // namespace

// Shared with the fused operator entry point.
int inf_gqa_prefill_launch(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                           int tokens, int q_heads, int sliding_window, const float* gate, float scale, void* out,
                           int out_dtype) {
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
    int rc = inf_validate_table(ctx, table, pool->num_pages, pool->page_size, tokens, "gqa_prefill");
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
    p.o_bs = (long long)tokens * q_heads * 128;
    p.status = ctx->status;
    return launch_flash<128, 128, 5, 5, true>(ctx, 2u, tq, tk, tk, tv, p, "flash_prefill_gqa_kernel");
}

extern "C" int32_t inf_gqa_prefill_paged(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                         const inf_page_table* table, int32_t tokens, int32_t q_heads,
                                         int32_t sliding_window, const float* gate, float scale, void* out,
                                         int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
    return inf_gqa_prefill_launch(ctx, q_f16, pool, table, tokens, q_heads, sliding_window, gate, scale, out,
                                  out_dtype);
}

extern "C" int32_t inf_mla_prefill_causal(inf_ctx* ctx, const void* q, int64_t q_ts, int64_t q_hs, const void* k_nope,
                                          int64_t kn_ts, int64_t kn_hs, const void* k_rope, int64_t kr_ts,
                                          const void* v, int64_t v_ts, int64_t v_hs, int32_t tokens, int32_t heads,
                                          int32_t nope_dim, int32_t rope_dim, int32_t v_dim, float scale, void* out,
                                          int64_t o_ts, int64_t o_hs, int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
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
    p.status = ctx->status;
    if (rope_dim) return launch_flash<192, 128, 3, 3, false>(ctx, 4u, tq, tk, tk2, tv, p, "flash_prefill_mla_kernel");
    return launch_flash<128, 128, 5, 5, false>(ctx, 8u, tq, tk, tk2, tv, p, "flash_prefill_mha_kernel");
}

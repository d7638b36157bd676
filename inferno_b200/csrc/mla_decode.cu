// Absorbed-MLA decode over the paged latent cache on tcgen05 / TMEM.
//
// All query heads of a token share one cached row (512 latent + 64 rope, fp16), so the heads are the
// M dimension of the MMAs: S[64 heads x 64 keys] = Q[64 x 576] C^T, O[64 x 512] += P[64 x 64] C[:, :512],
// and each cached byte is fetched from HBM once for all heads (the reference re-reads it per head,
// attention_kernels.metal:465-603).  One CTA = (sequence, query token, 64-head block, split of the page
// range).  A page (64 rows x 576) arrives as nine [64 x 64] TMA boxes with the 128-byte swizzle; the
// same shared-memory bytes serve as the K-major B operand of QK^T and, columns 0-511, as the MN-major B
// operand of PV.  M = 64 accumulators use 16 lanes of each TMEM quadrant, so the 512 output columns are
// held as two interleaved halves (lane offset 0 and 16) over TMEM columns 0-255.  Q is the TMEM A operand of
// QK^T, stored as two halves of 288 columns (144 TMEM columns, lane offsets 0 and 16); each half multiplies
// the matching 288 columns of the page into its own partial S on the same lanes (an M = 64 MMA keeps A and D
// on the same 16 lanes of a quadrant), and the softmax threads add the two partial S rows with a shuffle.
// Keeping Q out of shared memory leaves room for a ring of three whole pages (216 KB), which is what hides
// the HBM latency at batch 1.  There is one S buffer: the softmax copies it into registers at once and hands
// it back, so QK^T of the next page overlaps the exponentials.  P goes to shared memory as the K-major A
// operand of PV, O is rescaled lazily.  Split partials (max, sum, O) are merged by a second kernel.
//
// Warps: 0-3 Q load, softmax, epilogue; 4 TMA producer; 5 TMEM allocation + MMA issue.
#include <cuda_fp16.h>
#include <math.h>
#include <stdio.h>

#include "common.cuh"
#include "ptx.cuh"

using namespace inf;

namespace {

constexpr int LAT = 512, ROPE = 64, ROW = LAT + ROPE;  // 576
constexpr int PAGE = 64;
constexpr int HB = 64;                                   // heads per CTA (MMA M)
constexpr int NBLK = ROW / 64;                           // 9 column blocks
constexpr int BLK_BYTES = 64 * 128;                      // one [64 rows][64 cols] swizzled block
constexpr int TILE_BYTES = NBLK * BLK_BYTES;             // 73728: Q tile and KV page alike
constexpr int NUM_THREADS = 192;
constexpr float M_INIT = -1.0e30f;
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr uint32_t TMEM_COLS = 512;
#ifndef INF_MLA_PREFETCH_PAGES
#define INF_MLA_PREFETCH_PAGES 1  // pages of a CTA's range requested into L2 before the dependent-launch wait
#endif
constexpr uint32_t COL_O = 0, COL_S = 256, COL_Q = 320;  // O 256 columns, S 64, Q 144 (each on both lane halves)
constexpr int STAGES = 3;
constexpr int GATHER_UNIT = 64;  // the gather form splits the row list in units of 64 rows: one full tile per unit
constexpr int QHALF = ROW / 2;  // 288 query columns per lane half

constexpr int OFF_KV = 0;
constexpr int OFF_P = OFF_KV + STAGES * TILE_BYTES;
constexpr int OFF_BAR = OFF_P + BLK_BYTES;
constexpr int SMEM_TOTAL = OFF_BAR + 128;

struct MlaParams {
    const __half* rows;     // the pool's rows; the gather form copies from them directly
    const int* pages;
    const int* lens;
    const int* sel;         // gather form: [batch][sel_stride] logical row ids; null for the contiguous form
    const int* sel_counts;  // gather form: rows selected per sequence
    int sel_stride;
    int max_pages, num_pages;
    int tokens, heads, head_blocks, batch;
    int n_splits;
    float scale_log2;
    __half* part_acc; // [batch][tokens][n_splits][heads][512], each row already divided by its own sum
    float* part_ml;   // [batch][tokens][n_splits][heads][2]: running max (log2 domain) and sum
    int* status;
#ifdef INF_KPROF
    long long* kprof;  // debug builds only: timeline of CTA 0's first softmax thread, ns after entry
#endif
};

#ifdef INF_KPROF
#define KP_MARK(i) do { if (kp_on) p.kprof[i] = (long long)global_timer_ns() - kp_t0; } while (0)
#else
#define KP_MARK(i) do {} while (0)
#endif

__device__ __forceinline__ void split_range(int n_pages, int n_splits, int s, int& begin, int& end) {
    const int per = (n_pages + n_splits - 1) / n_splits;
    begin = min(n_pages, s * per);
    end = min(n_pages, begin + per);
}

// GATHER: the keys are not the first kv_len rows of the sequence but the rows listed in p.sel (the DSA indexer's
// choice); a "page" is then any 64 listed rows, copied row by row into the swizzled tile with 16-byte asynchronous
// copies, and everything after the load is unchanged.
template <bool GATHER>
__global__ void __launch_bounds__(NUM_THREADS, 1)
mla_decode_partial_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                          MlaParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sKV = smem + OFF_KV;
    uint8_t* sP = smem + OFF_P;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;            // [STAGES]
    uint64_t* kv_empty = kv_full + STAGES;   // [STAGES]
    uint64_t* s_full = kv_empty + STAGES;    // [1]
    uint64_t* s_free = s_full + 1;           // [1]: the S buffer has been copied into registers
    uint64_t* p_full = s_full + 2;
    uint64_t* pv_done = p_full + 1;
    uint64_t* q_landed = pv_done + 1;  // Q is in the last ring stage (TMA), before it moves to TMEM
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_landed + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef INF_KPROF
    const bool kp_on = tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && p.kprof;
    const long long kp_t0 = (long long)global_timer_ns();
    const int kp_cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (tid == 0 && p.kprof && kp_cta < 256) p.kprof[64 + kp_cta * 2] = kp_t0;
#endif
    // Everything that needs nothing from the kernels before this one comes first, so that under a programmatic
    // dependent launch it runs while they finish: barriers, TMEM, descriptors -- and a request to bring this CTA's
    // pages into L2.  The request is a hint computed from the length as it reads now: pages already cached never
    // change, and a page the append kernel is still writing is coherent in L2, so a wrong guess costs nothing.
    const int split = blockIdx.x;
    const int t = blockIdx.y % p.tokens, hb = blockIdx.y / p.tokens;
    const int b = blockIdx.z;
    const bool smem_ok = (smem_u32(smem) & 1023u) == 0;
    if (tid == 0 && smem_ok) {
        mbar_init(q_full, 128);
        mbar_init(q_landed, 1);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_free, 4);  // lane 0 of each softmax warp
        mbar_init(p_full, 128);
        mbar_init(pv_done, 1);
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    if (warp == 4) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_kv);
        }
        const int guess_pages = GATHER ? 0 : (p.lens[b] + t + 1 + PAGE - 1) / PAGE;
        if (guess_pages > 0) {
            int g_begin, g_end;
            split_range(guess_pages, p.n_splits, split, g_begin, g_end);
            for (int slot = g_begin + lane; slot < min(g_end, g_begin + INF_MLA_PREFETCH_PAGES) && slot < p.max_pages; slot += 32) {
                const int page = p.pages[(long long)b * p.max_pages + slot];
                if (page >= 0 && page < p.num_pages)
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.rows + (size_t)page * PAGE * ROW),
                                 "r"((uint32_t)TILE_BYTES)
                                 : "memory");
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    inf_pdl_wait();  // the appended row and the query come from kernels earlier in the stream
    inf_pdl_release();
    const int seq_rows = p.lens[b] + t + 1;                     // rows visible to this query token
    int kv_len = GATHER ? p.sel_counts[b] : seq_rows;  // keys this call attends to
    if (GATHER && kv_len > p.sel_stride) {  // a count beyond the list's row is cut to the row and reported
        kv_len = p.sel_stride;
        if (tid == 0 && split == 0) atomicOr(p.status, INF_STATUS_BAD_LEN);
    }
    // this CTA's keys: rows [row_begin, row_end) of the sequence (contiguous form: whole pages) or of the list
    const int unit = GATHER ? GATHER_UNIT : PAGE;
    int u_begin, u_end;
    split_range((kv_len + unit - 1) / unit, p.n_splits, split, u_begin, u_end);
    const int row_begin = u_begin * unit, row_end = min(kv_len, u_end * unit);
    const int pg_begin = row_begin / PAGE;           // contiguous form only
    const int n = (row_end - row_begin + PAGE - 1) / PAGE;  // 64-row tiles
    if (!smem_ok && tid == 0) atomicOr(p.status, INF_STATUS_BAD_SMEM);
    const bool active = n > 0 && smem_ok;  // a CTA with nothing to do only gives its TMEM back
    KP_MARK(0);

    if (!active) {
    } else if (warp == 4) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            // Q first, into the last ring stage: it is needed before any page and must not queue behind them
            mbar_arrive_expect_tx(q_landed, TILE_BYTES);
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk)
                tma_load_3d(sKV + (STAGES - 1) * TILE_BYTES + blk * BLK_BYTES, &tm_q, blk * 64, hb * HB,
                            b * p.tokens + t, q_landed);
            if (!GATHER) {
                const int oob_row = p.num_pages * PAGE;
                for (int j = 0; j < n; ++j) {
                    const int slot = pg_begin + j;
                    int y = oob_row;
                    if (slot < p.max_pages) {
                        const int page = p.pages[(long long)b * p.max_pages + slot];
                        if (page >= 0 && page < p.num_pages)
                            y = page * PAGE;
                        else
                            atomicOr(p.status, INF_STATUS_BAD_PAGE);
                    } else {
                        atomicOr(p.status, INF_STATUS_BAD_LEN);
                    }
                    const int st = j % STAGES;
                    // The first pages are requested one after another, not together: every CTA of the grid asks at the
                    // same moment, and HBM then delivers everybody's first page before anybody's second (22.0 µs
                    // against 22.6 µs at 32 768 rows).
                    if (j >= 1 && j < STAGES && !mbar_wait(&kv_full[j - 1], 0)) {
                        atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                        break;
                    }
                    if (j == STAGES - 1 && !mbar_wait(q_full, 0)) {  // the stage still holds Q until it is in TMEM
                        atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                        break;
                    }
                    if (!mbar_wait(&kv_empty[st], (((uint32_t)(j / STAGES)) & 1u) ^ 1u)) {
                        atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                        break;
                    }
                    mbar_arrive_expect_tx(&kv_full[st], TILE_BYTES);
#pragma unroll
                    for (int blk = 0; blk < NBLK; ++blk)
                        tma_load_2d(sKV + st * TILE_BYTES + blk * BLK_BYTES, &tm_kv, blk * 64, y, &kv_full[st]);
                }
            }
        }
        if (GATHER) {
            // The whole warp.  Lane l resolves rows l and l + 32 of every group of 64 listed rows; the rows are then
            // copied one after another with 16-byte asynchronous copies, the 32 lanes side by side along a row (whole
            // 512-byte runs per instruction), each chunk placed where the 128-byte swizzle of the tile expects it.
            // One-row TMA boxes did the same job at a few hundred requests per tile, and the request rate, not the
            // bytes, set the time to the first score.  A tile is handed over once its copies have landed, one tile late,
            // so that the next tile's copies are already in flight.
            int pending_stage = -1;
            for (int j = 0; j < n; ++j) {
                const int rows_here = min(PAGE, row_end - (row_begin + j * PAGE));  // listed rows in this 64-row tile
                int ys[2];
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int i = row_begin + j * PAGE + lane + 32 * rr;
                    ys[rr] = -1;  // an id the query may not see is read as a row of zeros
                    if (i < row_end) {
                        const int id = p.sel[(long long)b * p.sel_stride + i];
                        if (id >= 0 && id < seq_rows && id / PAGE < p.max_pages) {
                            const int page = p.pages[(long long)b * p.max_pages + id / PAGE];
                            if (page >= 0 && page < p.num_pages)
                                ys[rr] = page * PAGE + id % PAGE;
                            else
                                atomicOr(p.status, INF_STATUS_BAD_PAGE);
                        } else {
                            atomicOr(p.status, INF_STATUS_BAD_LEN);  // a listed row the query may not see
                        }
                    }
                }
                const int st = j % STAGES;
                int ok = 1;
                if (lane == 0) {
                    if (j == STAGES - 1 && !mbar_wait(q_full, 0)) ok = 0;  // the stage still holds Q until it is in TMEM
                    if (ok && !mbar_wait(&kv_empty[st], (((uint32_t)(j / STAGES)) & 1u) ^ 1u)) ok = 0;
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
                    break;
                }
                // Rows of the tile beyond the list are cleared: a masked key still enters PV as 0 x (whatever the
                // stage held).
#pragma unroll
                for (int rr = 0; rr < 2; ++rr)
                    if (lane + 32 * rr >= rows_here)
#pragma unroll
                        for (int blk = 0; blk < NBLK; ++blk) {
                            uint4* dst = reinterpret_cast<uint4*>(sKV + st * TILE_BYTES + blk * BLK_BYTES + (lane + 32 * rr) * 128);
#pragma unroll
                            for (int c = 0; c < 8; ++c) dst[c] = make_uint4(0u, 0u, 0u, 0u);
                        }
                const uint32_t tile = smem_u32(sKV + st * TILE_BYTES);
                for (int r = 0; r < rows_here; ++r) {
                    const int y = __shfl_sync(0xffffffffu, r < 32 ? ys[0] : ys[1], r & 31);
                    const __half* src = p.rows + (size_t)(y < 0 ? 0 : y) * ROW;
                    const uint32_t bytes = y < 0 ? 0u : 16u;  // zero bytes read: the chunk is filled with zeros
#pragma unroll
                    for (int c0 = 0; c0 < ROW / 8; c0 += 32) {
                        const int c = c0 + lane;  // 16-byte chunk of the row
                        if (c < ROW / 8) {
                            const uint32_t dst = tile + (c >> 3) * BLK_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src + c * 8), "r"(bytes)
                                         : "memory");
                        }
                    }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
                if (pending_stage >= 0) {
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&kv_full[pending_stage]);
                }
                pending_stage = st;
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            if (pending_stage >= 0) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&kv_full[pending_stage]);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc_f16(HB, PAGE, 0, 0);
            const uint32_t idesc_pv = umma_idesc_f16(HB, 256, 0, 1);
            const uint32_t kv_addr = smem_u32(sKV), p_addr = smem_u32(sP);
            auto issue_qk = [&](int j) {  // two partial S = Q[:, half] C_j[:, half]^T, A from TMEM, B K-major
                const uint32_t tile = kv_addr + (j % STAGES) * TILE_BYTES;
                // the two halves are independent accumulation chains: alternate them so that one MMA does not
                // have to wait for the previous one's accumulator
#pragma unroll
                for (int i = 0; i < ROW / 32; ++i)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int kk = h * (ROW / 32) + i;
                        const uint32_t off = (kk / 4) * BLK_BYTES + (kk % 4) * 32;
                        const uint32_t lane_half = (uint32_t)(h * 16) << 16;
                        umma_ts(tbase + lane_half + COL_S, tbase + lane_half + COL_Q + i * 8,
                                umma_smem_desc(tile + off, 16, 1024, UMMA_SW128), idesc_qk, i > 0);
                    }
                tc_commit(s_full);
            };
            bool ok = mbar_wait(q_full, 0);
            if (ok) ok = mbar_wait(&kv_full[0], 0);
            if (ok) {
                tc_fence_after();
                issue_qk(0);
            }
            for (int j = 0; ok && j < n; ++j) {
                if (j + 1 < n) {
                    ok = mbar_wait(&kv_full[(j + 1) % STAGES], ((uint32_t)((j + 1) / STAGES)) & 1u);
                    if (ok) ok = mbar_wait(s_free, ((uint32_t)j) & 1u);  // S of page j is in registers
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(j + 1);
                }
                ok = mbar_wait(p_full, ((uint32_t)j) & 1u);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tile = kv_addr + (j % STAGES) * TILE_BYTES;
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int kk = 0; kk < PAGE / 16; ++kk)
                        umma_ss(tbase + COL_O + ((uint32_t)(half * 16) << 16),
                                umma_smem_desc(p_addr + kk * 32, 16, 1024, UMMA_SW128),
                                umma_smem_desc(tile + half * 4 * BLK_BYTES + kk * 2048, BLK_BYTES, 1024, UMMA_SW128),
                                idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                tc_commit(&kv_empty[j % STAGES]);
                tc_commit(pv_done);
            }
            if (!ok) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
        }
    } else {
        // ------------------------------------------------ softmax + epilogue
        // lanes 0-15 of warp w own rows 16w..16w+15 of S and of O[:, 0:256]; lanes 16-31 own the same rows of
        // O[:, 256:512] (the accumulator half that sits at TMEM lane offset 16).
        const int row = warp * 16 + (lane & 15);
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        {   // Q row of this head, columns [288 * (lane / 16), +288), from the staged tile into TMEM (packed fp16 pairs)
            bool q_ok = mbar_wait(q_landed, 0);
            const uint8_t* sq = sKV + (STAGES - 1) * TILE_BYTES;
            const int col0 = (lane >> 4) * QHALF;
#pragma unroll
            for (int c = 0; c < QHALF / 32; ++c) {  // 9 groups of 16 TMEM columns = 32 query columns
                uint32_t v[16];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int col = col0 + c * 32 + i * 8;
                    const uint4 u = *reinterpret_cast<const uint4*>(sq + (col >> 6) * BLK_BYTES + sw128_offset(row, col & 63));
                    v[4 * i] = u.x;
                    v[4 * i + 1] = u.y;
                    v[4 * i + 2] = u.z;
                    v[4 * i + 3] = u.w;
                }
                tmem_st16(tbase + lane_addr + COL_Q + c * 16, v);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(q_full);
            if (!q_ok && lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
            KP_MARK(1);
        }
        float m_used = M_INIT, l = 0.f;  // kept identically in both lane halves of a row
        bool ok = true;
        const int half = lane >> 4;  // this thread exponentiates keys [32 * half, +32) of its row
        for (int j = 0; j < n; ++j) {
            if (!mbar_wait(s_full, ((uint32_t)j) & 1u)) {
                ok = false;
                break;
            }
            if (j < 6) KP_MARK(4 + j * 4);
            tc_fence_after();
            uint32_t sraw[PAGE];
            tmem_ld32(tbase + lane_addr + COL_S, sraw);
            tmem_ld32(tbase + lane_addr + COL_S + 32, sraw + 32);
            tc_wait_ld();
            tc_fence_before();
            if (lane == 0) mbar_arrive(s_free);
            // full scores of the row = the two partial products held by lanes i and i + 16
            float x[PAGE / 2];
            const int k0 = row_begin + j * PAGE + half * (PAGE / 2);
#pragma unroll
            for (int i = 0; i < PAGE; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, __uint_as_float(sraw[i]), 16);
                if ((i >> 5) == half) {
                    const int ii = i & 31;
                    x[ii] = (__uint_as_float(sraw[i]) + other) * p.scale_log2;
                    if (k0 + ii >= row_end) x[ii] = -INFINITY;
                }
            }
            float mx = x[0];
#pragma unroll
            for (int i = 1; i < PAGE / 2; ++i) mx = fmaxf(mx, x[i]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_cand = fmaxf(m_used, mx);
            float alpha = 1.0f;
            bool rescale = false;
            if (j == 0) {
                m_used = m_cand;
            } else {
                rescale = __any_sync(0xffffffffu, (m_cand - m_used) > RESCALE_THRESHOLD);
                if (rescale) {
                    alpha = ex2_approx(m_used - m_cand);
                    m_used = m_cand;
                    l *= alpha;
                }
            }
            if (j < 6) KP_MARK(5 + j * 4);
            // P (and O) may only be touched once the previous tile's PV has drained
            if (j > 0 && !mbar_wait(pv_done, ((uint32_t)(j - 1)) & 1u)) {
                ok = false;
                break;
            }
            if (j < 6) KP_MARK(6 + j * 4);
            if (rescale) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 256 / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld32(tbase + lane_addr + COL_O + c * 32, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(tbase + lane_addr + COL_O + c * 32, o);
                }
                tc_wait_st();
            }
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < PAGE / 2 / 8; ++c) {
                float pv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    pv[i] = ex2_approx(x[c * 8 + i] - m_used);
                    sum += pv[i];
                }
                uint4 v;
                v.x = pack_half2(pv[0], pv[1]);
                v.y = pack_half2(pv[2], pv[3]);
                v.z = pack_half2(pv[4], pv[5]);
                v.w = pack_half2(pv[6], pv[7]);
                *reinterpret_cast<uint4*>(sP + sw128_offset(row, half * (PAGE / 2) + c * 8)) = v;
            }
            l += sum + __shfl_xor_sync(0xffffffffu, sum, 16);
            fence_proxy_async_smem();  // P was written through the generic proxy, the MMA reads it through the async one
            tc_fence_before();
            mbar_arrive(p_full);
            if (j < 6) KP_MARK(7 + j * 4);
        }
        if (ok && !mbar_wait(pv_done, ((uint32_t)(n - 1)) & 1u)) ok = false;
        KP_MARK(2);
        if (!ok) {
            if (lane == 0) atomicOr(p.status, INF_STATUS_WAIT_TIMEOUT);
        } else {
            tc_fence_after();
            const int head = hb * HB + row;
            const long long prow =
                ((((long long)b * p.tokens + t) * p.n_splits + split) * p.heads) + head;
            const bool valid = head < p.heads;
            // the partial row is stored normalised by its own sum, as fp16: half the bytes of an fp32 partial,
            // and the values are bounded by the largest cached latent
            const float inv_l = 1.0f / l;
            __half* dst = p.part_acc + prow * LAT + (lane >> 4) * 256;
            if (hb * HB + HB <= p.heads) {
                // A whole block of 64 heads: its partial rows are one contiguous 64 KB run.  Each thread parks its
                // half row in the first ring stage (every page has been consumed), 16-byte chunks XORed with the row
                // so that the eight rows of a store phase fall on different banks, and the warp then writes its own
                // sixteen rows back out as whole 512-byte runs.
                uint8_t* stage = sKV + (size_t)(warp * 16) * (LAT * 2);
                const int lr = lane & 15;
#pragma unroll
                for (int c = 0; c < 256 / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld32(tbase + lane_addr + COL_O + c * 32, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 v;
                        v.x = pack_half2(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l);
                        v.y = pack_half2(__uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
                        v.z = pack_half2(__uint_as_float(o[i + 4]) * inv_l, __uint_as_float(o[i + 5]) * inv_l);
                        v.w = pack_half2(__uint_as_float(o[i + 6]) * inv_l, __uint_as_float(o[i + 7]) * inv_l);
                        const int chunk = (lane >> 4) * 32 + c * 4 + (i >> 3);  // 16-byte chunk of the 1 KB row
                        *reinterpret_cast<uint4*>(stage + lr * (LAT * 2) + ((chunk ^ (lr & 7)) << 4)) = v;
                    }
                }
                __syncwarp();
                const long long prow_w = ((((long long)b * p.tokens + t) * p.n_splits + split) * p.heads) + hb * HB + warp * 16;
                uint4* out16 = reinterpret_cast<uint4*>(p.part_acc + prow_w * LAT);
#pragma unroll 4
                for (int it = 0; it < 32; ++it) {  // 16 rows x 64 chunks, 32 chunks (half a row) per step
                    const int r16 = it >> 1, chunk = (it & 1) * 32 + lane;
                    out16[r16 * 64 + chunk] =
                        *reinterpret_cast<const uint4*>(stage + r16 * (LAT * 2) + ((chunk ^ (r16 & 7)) << 4));
                }
            } else
#pragma unroll
            for (int c = 0; c < 256 / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(tbase + lane_addr + COL_O + c * 32, o);
                tc_wait_ld();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 v;
                        v.x = pack_half2(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l);
                        v.y = pack_half2(__uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
                        v.z = pack_half2(__uint_as_float(o[i + 4]) * inv_l, __uint_as_float(o[i + 5]) * inv_l);
                        v.w = pack_half2(__uint_as_float(o[i + 6]) * inv_l, __uint_as_float(o[i + 7]) * inv_l);
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
                    }
                }
            }
            if (valid && lane < 16) {
                p.part_ml[prow * 2] = m_used;
                p.part_ml[prow * 2 + 1] = l;
            }
            KP_MARK(3);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tbase, TMEM_COLS);
#ifdef INF_KPROF
    if (tid == 0 && p.kprof && kp_cta < 256) p.kprof[64 + kp_cta * 2 + 1] = (long long)global_timer_ns();
#endif
}

// Merge of the split partials.
constexpr int MAX_SPLITS = 1024;

// One CTA per (head, query row): 512 threads (four CTAs of 128 threads per head, a quarter of the columns each,
// measured slower: step 30.2 us against 29.3 us).  The split weights are computed once; for the weighted sum the
// threads form eight groups that walk the splits with stride eight, each thread owning eight adjacent columns
// (one 16-byte load per split, all of a thread's loads in flight together), and the partial sums meet in shared
// memory.
template <typename OutT>
__global__ void __launch_bounds__(512)
mla_decode_combine_kernel(const __half* __restrict__ part_acc, const float* __restrict__ part_ml,
                          const int* __restrict__ lens, const int* __restrict__ counts, OutT* __restrict__ out, int tokens,
                          int heads, int n_splits, int sel_stride) {
    __shared__ float w[MAX_SPLITS];
    __shared__ float red[16];
    __shared__ float group_acc[7][LAT];
    inf_pdl_wait();
    inf_pdl_release();
    const int h = blockIdx.x, t = blockIdx.y % tokens, b = blockIdx.y / tokens;
    const int tid = threadIdx.x;
    int kv_len = counts ? counts[b] : lens[b] + t + 1;  // keys the partial kernel saw
    if (counts) kv_len = min(kv_len, sel_stride);
    if (kv_len <= 0) {  // no key at all (an empty list, a negative length): no partial was written; the output is zero
        OutT* dst = out + ((((long long)b * tokens + t) * heads) + h) * LAT + tid;
        *dst = OutT(0.f);
        return;
    }
    const int n_pages = (kv_len + (counts ? GATHER_UNIT : PAGE) - 1) / (counts ? GATHER_UNIT : PAGE);  // split units
    const int per = (n_pages + n_splits - 1) / n_splits;
    const int n_valid = (n_pages + per - 1) / per;  // splits [0, n_valid) did work
    const long long prow0 = (((long long)b * tokens + t) * n_splits) * heads + h;
    // pass 1: global maximum
    float mloc = M_INIT;
    for (int s = tid; s < n_valid; s += 512) mloc = fmaxf(mloc, part_ml[(prow0 + (long long)s * heads) * 2]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
    if ((tid & 31) == 0) red[tid >> 5] = mloc;
    __syncthreads();
    float M = red[0];
#pragma unroll
    for (int i = 1; i < 16; ++i) M = fmaxf(M, red[i]);
    __syncthreads();
    // pass 2: weights and the normaliser
    float lloc = 0.f;
    for (int s = tid; s < n_valid; s += 512) {
        const float ws = ex2_approx(part_ml[(prow0 + (long long)s * heads) * 2] - M) *
                         part_ml[(prow0 + (long long)s * heads) * 2 + 1];  // weight of a normalised partial
        w[s] = ws;
        lloc += ws;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lloc += __shfl_xor_sync(0xffffffffu, lloc, o);
    if ((tid & 31) == 0) red[tid >> 5] = lloc;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) total += red[i];
    const float inv = 1.0f / total;
    // pass 3: weighted sum of the partial outputs
    const int g = tid >> 6, c = (tid & 63) * 8;
    const __half* src = part_acc + prow0 * LAT + c;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 8
    for (int s = g; s < n_valid; s += 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + (long long)s * heads * LAT);
        const float ws = w[s];
        const __half2* hv = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(hv[i]);
            acc[2 * i] = fmaf(ws, f.x, acc[2 * i]);
            acc[2 * i + 1] = fmaf(ws, f.y, acc[2 * i + 1]);
        }
    }
    if (g > 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) group_acc[g - 1][c + i] = acc[i];
    }
    __syncthreads();
    if (g == 0) {
        OutT* dst = out + ((((long long)b * tokens + t) * heads) + h) * LAT + c;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            dst[i] = OutT((((acc[i] + group_acc[0][c + i]) + (group_acc[1][c + i] + group_acc[2][c + i])) +
                           ((group_acc[3][c + i] + group_acc[4][c + i]) + (group_acc[5][c + i] + group_acc[6][c + i]))) * inv);
    }
}

}  // namespace

namespace {
// Split count: enough CTAs to fill the GPU, never more splits than pages, evened out so every split does work.
int mla_decode_splits(const inf_ctx* ctx, int batch, int tokens, int heads, int max_len) {
    const int head_blocks = (heads + HB - 1) / HB;
    const int max_pages_used = (max_len + PAGE - 1) / PAGE;
    const int ctas_per_split = batch * tokens * head_blocks;
    int n_splits = ctx->sm_count / ctas_per_split;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > max_pages_used) n_splits = max_pages_used;
    if (n_splits > MAX_SPLITS) n_splits = MAX_SPLITS;
    const int per = (max_pages_used + n_splits - 1) / n_splits;
    return (max_pages_used + per - 1) / per;
}
}  // namespace

size_t inf_mla_decode_scratch_bytes(const inf_ctx* ctx, int batch, int tokens, int heads, int max_len) {
    const size_t prows = (size_t)batch * tokens * mla_decode_splits(ctx, batch, tokens, heads, max_len) * heads;
    const size_t acc_bytes = (prows * LAT * sizeof(__half) + 255) & ~(size_t)255;
    return acc_bytes + prows * 2 * sizeof(float);
}

// sel == nullptr: keys are rows 0 .. lens[b]+t of each sequence (max_len bounds them).  Otherwise keys are the
// sel_counts[b] rows listed in sel[b][...] (max_len bounds the counts) and tokens must be 1.
int inf_mla_decode_launch(inf_ctx* ctx, const void* q_f16, const inf_mla_pool* pool, const inf_page_table* table,
                          int tokens, int heads, int max_len, float scale, void* out, int out_dtype, size_t ws_offset,
                          const int* sel, const int* sel_counts, int sel_stride) {
    int rc;
    const int head_blocks = (heads + HB - 1) / HB;
    // the gather form splits in units of GATHER_UNIT rows: scaling max_len makes the same split arithmetic count units
    const int n_splits = mla_decode_splits(ctx, table->batch, tokens, heads, sel ? max_len * (PAGE / GATHER_UNIT) : max_len);
    const size_t prows = (size_t)table->batch * tokens * n_splits * heads;
    const size_t acc_bytes = (prows * LAT * sizeof(__half) + 255) & ~(size_t)255;
    rc = inf_ensure_workspace(ctx, ws_offset + acc_bytes + prows * 2 * sizeof(float));
    if (rc != INF_OK) return rc;

    CUtensorMap tq, tkv;
    {
        uint64_t dims[3] = {(uint64_t)ROW, (uint64_t)heads, (uint64_t)table->batch * tokens};
        uint64_t strides[2] = {(uint64_t)ROW * 2, (uint64_t)heads * ROW * 2};
        uint32_t box[3] = {64, (uint32_t)HB, 1};
        rc = inf_make_tmap(ctx, q_f16, 3, dims, strides, box, &tq);
        if (rc != INF_OK) return rc;
    }
    {
        uint64_t dims[2] = {(uint64_t)ROW, (uint64_t)pool->num_pages * PAGE};
        uint64_t strides[1] = {(uint64_t)ROW * 2};
        uint32_t box[2] = {64, (uint32_t)PAGE};  // unused by the gather form, which copies rows itself
        rc = inf_make_tmap(ctx, pool->rows, 2, dims, strides, box, &tkv);
        if (rc != INF_OK) return rc;
    }
    MlaParams p{};
    p.rows = (const __half*)pool->rows;
    p.pages = table->pages;
    p.lens = table->lens;
    p.sel = sel;
    p.sel_counts = sel_counts;
    p.sel_stride = sel_stride;
    p.max_pages = table->max_pages;
    p.num_pages = pool->num_pages;
    p.tokens = tokens;
    p.heads = heads;
    p.head_blocks = head_blocks;
    p.batch = table->batch;
    p.n_splits = n_splits;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.part_acc = (__half*)((char*)ctx->workspace + ws_offset);
    p.part_ml = (float*)((char*)ctx->workspace + ws_offset + acc_bytes);
    p.status = ctx->status;
    if (!(ctx->func_attr_done & 16u)) {
        INF_CUDA(ctx, cudaFuncSetAttribute(mla_decode_partial_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SMEM_TOTAL));
        INF_CUDA(ctx, cudaFuncSetAttribute(mla_decode_partial_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SMEM_TOTAL));
        ctx->func_attr_done |= 16u;
    }
    dim3 grid(n_splits, tokens * head_blocks, table->batch);
#ifdef INF_KPROF
    static long long* d_kprof = nullptr;
    if (!d_kprof) cudaMalloc(&d_kprof, 576 * sizeof(long long));
    cudaMemsetAsync(d_kprof, 0, 576 * sizeof(long long), ctx->stream);
    p.kprof = d_kprof;
#endif
    {
        inf_prof_scope prof(ctx, "mla_decode_partial_kernel");
        if (sel)
            INF_CUDA(ctx, inf_launch_pdl(mla_decode_partial_kernel<true>, grid, dim3(NUM_THREADS), SMEM_TOTAL, ctx->stream, tq, tkv, p));
        else
            INF_CUDA(ctx, inf_launch_pdl(mla_decode_partial_kernel<false>, grid, dim3(NUM_THREADS), SMEM_TOTAL, ctx->stream, tq, tkv, p));
    }
#ifdef INF_KPROF
    {
        long long h[576];
        cudaMemcpy(h, d_kprof, sizeof(h), cudaMemcpyDeviceToHost);
        {
            long long e0 = 0, e1 = 0, x0 = 0, x1 = 0; int nc = 0;
            for (int i = 0; i < 256; ++i) {
                if (!h[64 + 2 * i]) continue;
                const long long e = h[64 + 2 * i], x = h[65 + 2 * i];
                if (!nc) { e0 = e1 = e; x0 = x1 = x; }
                e0 = e < e0 ? e : e0; e1 = e > e1 ? e : e1; x0 = x < x0 ? x : x0; x1 = x > x1 ? x : x1; ++nc;
            }
            fprintf(stderr, "KPROF mla_decode %d CTAs: entries spread over %lld ns, first exit %lld ns, last exit %lld ns after the first entry\n", nc, e1 - e0, x0 - e0, x1 - e0);
        }
        fprintf(stderr, "KPROF mla_decode CTA 0 thread 0, ns after entry: set-up %lld, Q in TMEM %lld, last PV retired %lld, partial stored %lld; per page (S ready, max known, PV(j-1) retired, P handed over):", h[0], h[1], h[2], h[3]);
        for (int j = 0; j < 6 && h[4 + j * 4]; ++j) fprintf(stderr, " [%lld %lld %lld %lld]", h[4 + j * 4], h[5 + j * 4], h[6 + j * 4], h[7 + j * 4]);
        fprintf(stderr, "\n");
    }
#endif
    INF_LAUNCH_CHECK(ctx, "mla_decode_partial_kernel");
    dim3 cgrid(heads, tokens * table->batch);
    if (out_dtype == INF_DTYPE_F32)
        INF_CUDA(ctx, inf_launch_pdl(mla_decode_combine_kernel<float>, cgrid, dim3(512), 0, ctx->stream, p.part_acc,
                                     p.part_ml, table->lens, sel_counts, (float*)out, tokens, heads, n_splits, sel_stride));
    else
        INF_CUDA(ctx, inf_launch_pdl(mla_decode_combine_kernel<__half>, cgrid, dim3(512), 0, ctx->stream, p.part_acc,
                                     p.part_ml, table->lens, sel_counts, (__half*)out, tokens, heads, n_splits, sel_stride));
    INF_LAUNCH_CHECK(ctx, "mla_decode_combine_kernel");
    return INF_OK;
}

extern "C" int32_t inf_mla_decode_absorbed(inf_ctx* ctx, const void* q_f16, const inf_mla_pool* pool,
                                           const inf_page_table* table, int32_t tokens, int32_t heads,
                                           int32_t max_len, float scale, void* out, int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
    if (!q_f16 || !pool || !table || !out) return inf_fail(ctx, INF_E_ARG, "mla_decode: null pointer");
    if (!pool->rows) return inf_fail(ctx, INF_E_ARG, "mla_decode: pool has no storage");
    if (pool->latent_dim != LAT || pool->rope_dim != ROPE || pool->page_size != PAGE) return INF_UNSUPPORTED;
    if (tokens <= 0 || heads <= 0 || max_len <= 0) return inf_fail(ctx, INF_E_SHAPE, "mla_decode: sizes must be positive");
    if (!(scale > 0.f)) return inf_fail(ctx, INF_E_CONFIG, "mla_decode: scale must be positive");
    if (out_dtype != INF_DTYPE_F32 && out_dtype != INF_DTYPE_F16)
        return inf_fail(ctx, INF_E_DTYPE, "mla_decode: output dtype must be f32 or f16");
    int rc = inf_validate_table(ctx, table, pool->num_pages, PAGE, tokens, "mla_decode");
    if (rc != INF_OK) return rc;
    if (table->host_lens)
        for (int b = 0; b < table->batch; ++b)
            if (table->host_lens[b] + tokens > max_len)
                return inf_fail(ctx, INF_E_SHAPE, "mla_decode: sequence %d reaches %d rows, beyond max_len %d", b,
                                table->host_lens[b] + tokens, max_len);
    return inf_mla_decode_launch(ctx, q_f16, pool, table, tokens, heads, max_len, scale, out, out_dtype, 0, nullptr,
                                 nullptr, 0);
}

extern "C" int32_t inf_mla_decode_absorbed_selected(inf_ctx* ctx, const void* q_f16, const inf_mla_pool* pool,
                                                    const inf_page_table* table, const int32_t* selected,
                                                    const int32_t* selected_counts, int32_t selected_stride,
                                                    int32_t heads, float scale, void* out, int32_t out_dtype) {
    INF_CHECK_CTX(ctx);
    if (!q_f16 || !pool || !table || !selected || !selected_counts || !out)
        return inf_fail(ctx, INF_E_ARG, "mla_decode_selected: null pointer");
    if (!pool->rows) return inf_fail(ctx, INF_E_ARG, "mla_decode_selected: pool has no storage");
    if (pool->latent_dim != LAT || pool->rope_dim != ROPE || pool->page_size != PAGE) return INF_UNSUPPORTED;
    if (heads <= 0 || selected_stride <= 0)
        return inf_fail(ctx, INF_E_SHAPE, "mla_decode_selected: sizes must be positive");
    if (!(scale > 0.f)) return inf_fail(ctx, INF_E_CONFIG, "mla_decode_selected: scale must be positive");
    if (out_dtype != INF_DTYPE_F32 && out_dtype != INF_DTYPE_F16)
        return inf_fail(ctx, INF_E_DTYPE, "mla_decode_selected: output dtype must be f32 or f16");
    int rc = inf_validate_table(ctx, table, pool->num_pages, PAGE, 1, "mla_decode_selected");
    if (rc != INF_OK) return rc;
    return inf_mla_decode_launch(ctx, q_f16, pool, table, 1, heads, selected_stride, scale, out, out_dtype, 0, selected,
                                 selected_counts, selected_stride);
}

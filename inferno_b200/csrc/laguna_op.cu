// laguna_gated_gqa_f16_attention_device (crates/backend/src/backend.rs:1350) as one C-ABI call, and the GLM
// paged MHA decode (paged_decode_attention_resident_device, backend.rs:1966).
#include <cuda_fp16.h>
#include <math.h>

#include <algorithm>

#include "common.cuh"
#include "ptx.cuh"

int inf_gqa_decode_launch(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                          int q_heads, int max_len, int split_chunk, int sliding_window, const float* gate,
                          float scale, void* out, int out_dtype, void* scratch, size_t scratch_bytes, int len_add,
                          const struct DecodeFp8* fp8, void* const* peer_outs, int n_peers);
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

// The same operator split over the keys, for dims that are multiples of 64 (the GLM layout is 256 / 256): MHA decode
// shares nothing between heads, so it is a pure stream over the head's K and V rows and the only question is how many
// bytes are in flight.  One CTA per (split of the cached keys, head, sequence); eight lanes own one key -- each lane
// KC (VC) 16-byte pieces of its K (V) row, pieces of neighbouring lanes adjacent in memory -- so a warp reads four
// whole rows per load instruction and the dot product closes with three shuffles; the 32 lane groups of a CTA keep
// their own online softmax and merge once at the end.  A second kernel merges the splits and adds the current token,
// which the reference also takes from its f32 buffers, not from the cache (attention_kernels.metal:374-387).
// Threads per CTA and resident CTAs per SM.  Measured on the 64-head, 4 095-key case: 256 x 2 53.2 us, 128 x 4 (128
// registers) 51.1 us, 128 x 3 with every lane group requesting its next key's rows before it works on the current one
// (163 registers) 52.5 us.
#ifndef INF_GLM_THREADS
#define INF_GLM_THREADS 128
#define INF_GLM_CTAS 4
#endif
constexpr int GS_THREADS = INF_GLM_THREADS;
constexpr int GS_GROUPS = GS_THREADS / 8;

template <int KC, int VC>
__global__ void __launch_bounds__(GS_THREADS, INF_GLM_CTAS)
glm_paged_decode_split_kernel(const float* __restrict__ q, const __half* __restrict__ pk, const __half* __restrict__ pv,
                              float* __restrict__ part_acc, float* __restrict__ part_ml, int batch, int heads, int past,
                              int page_size, int keys_per_split, int splits) {
    constexpr int dim = KC * 64, vdim = VC * 64;
    const int split = blockIdx.x, row = blockIdx.y, head = row % heads, b = row / heads;
    const int tid = threadIdx.x, group = tid >> 3, gl = tid & 7;
    const int k_begin = split * keys_per_split, k_end = min(past, k_begin + keys_per_split);
    const float scale = 1.0f / sqrtf((float)dim);
    float qf[KC][8], acc[VC][8];
#pragma unroll
    for (int c = 0; c < KC; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) qf[c][i] = q[(size_t)row * dim + (c * 8 + gl) * 8 + i] * scale;
#pragma unroll
    for (int c = 0; c < VC; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
    float m = NEG_BIG, l = 0.f;
    const unsigned gmask = 0xffu << (tid & 24);  // the eight lanes of this group inside their warp
    const size_t row_base = ((size_t)b * heads + head) * page_size;            // + page * batch * heads * page_size
    const size_t page_stride = (size_t)batch * heads * page_size;
    uint4 kraw[KC], vraw[VC];
    auto request = [&](int key, uint4 (&kr)[KC], uint4 (&vr)[VC]) {
        const int page = key / page_size, off = key - page * page_size;
        const size_t r = (size_t)page * page_stride + row_base + off;
#pragma unroll
        for (int c = 0; c < KC; ++c) kr[c] = __ldg(reinterpret_cast<const uint4*>(pk + r * dim + (c * 8 + gl) * 8));
#pragma unroll
        for (int c = 0; c < VC; ++c) vr[c] = __ldg(reinterpret_cast<const uint4*>(pv + r * vdim + (c * 8 + gl) * 8));
    };
    for (int key = k_begin + group; key < k_end; key += GS_GROUPS) {
        request(key, kraw, vraw);
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < KC; ++c) {
            const __half2* h = reinterpret_cast<const __half2*>(&kraw[c]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                dot = fmaf(qf[c][2 * i], f.x, dot);
                dot = fmaf(qf[c][2 * i + 1], f.y, dot);
            }
        }
        // only the eight lanes of this key's group take part: the four groups of a warp may run different trip counts
        dot += __shfl_xor_sync(gmask, dot, 1);
        dot += __shfl_xor_sync(gmask, dot, 2);
        dot += __shfl_xor_sync(gmask, dot, 4);
        const float mn = fmaxf(m, dot);
        const float rs = l == 0.f ? 0.f : expf(m - mn);
        const float w = expf(dot - mn);
        l = l * rs + w;
        m = mn;
#pragma unroll
        for (int c = 0; c < VC; ++c) {
            const __half2* h = reinterpret_cast<const __half2*>(&vraw[c]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h[i]);
                acc[c][2 * i] = fmaf(acc[c][2 * i], rs, w * f.x);
                acc[c][2 * i + 1] = fmaf(acc[c][2 * i + 1], rs, w * f.y);
            }
        }
    }
    // merge the 32 groups of the CTA, 8 at a time through shared memory
    __shared__ float sm[GS_GROUPS], sl[GS_GROUPS];
    __shared__ float sacc[8][vdim];
    if (gl == 0) {
        sm[group] = m;
        sl[group] = l;
    }
    __syncthreads();
    float M = NEG_BIG;
    for (int g = 0; g < GS_GROUPS; ++g)
        if (sl[g] > 0.f) M = fmaxf(M, sm[g]);
    float L = 0.f;
    for (int g = 0; g < GS_GROUPS; ++g)
        if (sl[g] > 0.f) L += sl[g] * expf(sm[g] - M);
    const float mine = l > 0.f ? expf(m - M) : 0.f;
    float total[(vdim + GS_THREADS - 1) / GS_THREADS];
#pragma unroll
    for (int i = 0; i < (vdim + GS_THREADS - 1) / GS_THREADS; ++i) total[i] = 0.f;
    for (int round = 0; round < GS_GROUPS / 8; ++round) {
        __syncthreads();
        if (group / 8 == round) {
#pragma unroll
            for (int c = 0; c < VC; ++c)
#pragma unroll
                for (int i = 0; i < 8; ++i) sacc[group & 7][(c * 8 + gl) * 8 + i] = acc[c][i] * mine;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < (vdim + GS_THREADS - 1) / GS_THREADS; ++i) {
            const int d = tid + i * GS_THREADS;
            if (d < vdim)
#pragma unroll
                for (int g = 0; g < 8; ++g) total[i] += sacc[g][d];
        }
    }
    const size_t prow = (size_t)row * splits + split;
#pragma unroll
    for (int i = 0; i < (vdim + GS_THREADS - 1) / GS_THREADS; ++i) {
        const int d = tid + i * GS_THREADS;
        if (d < vdim) part_acc[prow * vdim + d] = total[i];
    }
    if (tid == 0) {
        part_ml[prow * 2] = M;
        part_ml[prow * 2 + 1] = L;
    }
}

// The same split with the rows brought in by the copy engine instead of by the threads' own loads: when pages hold a
// multiple of 16 keys, 16 consecutive keys of a head are one contiguous run of K rows and one of V rows, and a producer
// thread keeps a ring of such tiles full with bulk copies (cp.async.bulk) while four consumer warps -- 16 lane groups,
// one key each per tile -- read their slices from shared memory.  The bytes in flight no longer depend on registers.
#ifndef INF_GLM_RING_STAGES
#define INF_GLM_RING_STAGES 4
#define INF_GLM_RING_CTAS 3
#endif
// How many CTAs the ring form launches.  Measured on the 64-head, 4 095-key case (kernel time; four stages, up to
// three CTAs per SM): 2 pieces per head (128 CTAs) 64.4 us, 3 (192) 52.1 us, 4 (256) 46.5-47.1 us, 5 (320) 47.2 us,
// 6 (384) 48.4 us, 7 for most heads (444, every slot filled) 51.0 us, 13 (832, two waves) 50.0 us; at 4 pieces a ring
// of three, five or six stages is within 1 us.  The grid therefore aims at seven CTAs per four SMs.
constexpr int GR_KEYS = 16;
constexpr int GR_STAGES = INF_GLM_RING_STAGES;
constexpr int GR_CONSUMERS = 128;
constexpr int GR_THREADS = GR_CONSUMERS + 32;

template <int KC, int VC>
__global__ void __launch_bounds__(GR_THREADS, INF_GLM_RING_CTAS)
glm_paged_decode_ring_kernel(const float* __restrict__ q, const __half* __restrict__ pk, const __half* __restrict__ pv,
                             float* __restrict__ part_acc, float* __restrict__ part_ml, int batch, int heads, int past,
                             int page_size, int keys_per_split, int splits, int* __restrict__ status) {
    constexpr int dim = KC * 64, vdim = VC * 64;
    constexpr int K_BYTES = GR_KEYS * dim * 2, V_BYTES = GR_KEYS * vdim * 2, STAGE_BYTES = K_BYTES + V_BYTES;
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ uint64_t full[GR_STAGES], empty[GR_STAGES];
    __shared__ float sm[GR_KEYS], sl[GR_KEYS];
    __shared__ float sacc[8][vdim];
    const int split = blockIdx.x, row = blockIdx.y, head = row % heads, b = row / heads;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k_begin = split * keys_per_split, k_end = min(past, k_begin + keys_per_split);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + GR_KEYS - 1) / GR_KEYS : 0;
    if (tid == 0) {
        for (int i = 0; i < GR_STAGES; ++i) {
            inf::mbar_init(&full[i], 1);
            inf::mbar_init(&empty[i], GR_CONSUMERS / 32);
        }
        inf::mbar_fence_init();
    }
    __syncthreads();
    const size_t row_base = ((size_t)b * heads + head) * page_size;  // + page * batch * heads * page_size
    const size_t page_stride = (size_t)batch * heads * page_size;
    float acc[VC][8];
#pragma unroll
    for (int c = 0; c < VC; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
    float m = NEG_BIG, l = 0.f;
    const int group = tid >> 3, gl = tid & 7;
    if (warp == GR_CONSUMERS / 32) {
        // ---- producer: one thread; a 16-key tile never straddles a page (pages hold a multiple of 16 keys and the
        //      splits start at multiples of 16)
        if (lane == 0) {
            for (int t = 0; t < n_tiles; ++t) {
                const int s = t % GR_STAGES;
                if (t >= GR_STAGES && !inf::mbar_wait(&empty[s], ((uint32_t)(t / GR_STAGES - 1)) & 1u)) {
                    atomicOr(status, INF_STATUS_WAIT_TIMEOUT);
                    break;
                }
                const int key0 = k_begin + t * GR_KEYS;
                const int valid = min(GR_KEYS, k_end - key0);
                const int page = key0 / page_size, off = key0 - page * page_size;
                const size_t r = (size_t)page * page_stride + row_base + off;
                uint8_t* dst = ring + s * STAGE_BYTES;
                inf::mbar_arrive_expect_tx(&full[s], (uint32_t)valid * (dim + vdim) * 2);
                inf::bulk_load_1d(dst, pk + r * dim, (uint32_t)valid * dim * 2, &full[s]);
                inf::bulk_load_1d(dst + K_BYTES, pv + r * vdim, (uint32_t)valid * vdim * 2, &full[s]);
            }
        }
    } else {
        const float scale = 1.0f / sqrtf((float)dim);
        float qf[KC][8];
#pragma unroll
        for (int c = 0; c < KC; ++c)
#pragma unroll
            for (int i = 0; i < 8; ++i) qf[c][i] = q[(size_t)row * dim + (c * 8 + gl) * 8 + i] * scale;
        const unsigned gmask = 0xffu << (tid & 24);  // the eight lanes of this group inside their warp
        bool ok = true;
        for (int t = 0; t < n_tiles; ++t) {
            const int s = t % GR_STAGES;
            if (ok && !inf::mbar_wait(&full[s], ((uint32_t)(t / GR_STAGES)) & 1u)) ok = false;
            const int key = k_begin + t * GR_KEYS + group;
            if (ok && key < k_end) {
                const uint8_t* krow = ring + s * STAGE_BYTES + group * (dim * 2) + gl * 16;
                const uint8_t* vrow = ring + s * STAGE_BYTES + K_BYTES + group * (vdim * 2) + gl * 16;
                float dot = 0.f;
#pragma unroll
                for (int c = 0; c < KC; ++c) {
                    const uint4 kraw = *reinterpret_cast<const uint4*>(krow + c * 128);
                    const __half2* h = reinterpret_cast<const __half2*>(&kraw);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __half22float2(h[i]);
                        dot = fmaf(qf[c][2 * i], f.x, dot);
                        dot = fmaf(qf[c][2 * i + 1], f.y, dot);
                    }
                }
                // only the eight lanes of this key's group take part: in the last tile some groups have no key
                dot += __shfl_xor_sync(gmask, dot, 1);
                dot += __shfl_xor_sync(gmask, dot, 2);
                dot += __shfl_xor_sync(gmask, dot, 4);
                const float mn = fmaxf(m, dot);
                const float rs = l == 0.f ? 0.f : expf(m - mn);
                const float w = expf(dot - mn);
                l = l * rs + w;
                m = mn;
#pragma unroll
                for (int c = 0; c < VC; ++c) {
                    const uint4 vraw = *reinterpret_cast<const uint4*>(vrow + c * 128);
                    const __half2* h = reinterpret_cast<const __half2*>(&vraw);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __half22float2(h[i]);
                        acc[c][2 * i] = fmaf(acc[c][2 * i], rs, w * f.x);
                        acc[c][2 * i + 1] = fmaf(acc[c][2 * i + 1], rs, w * f.y);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) inf::mbar_arrive(&empty[s]);  // the warp's four groups have read the tile
        }
        if (!ok && lane == 0) atomicOr(status, INF_STATUS_WAIT_TIMEOUT);
    }
    // merge the 16 groups of the CTA, 8 at a time through shared memory (the producer warp only keeps the barriers company)
    const bool consumer = tid < GR_CONSUMERS;
    if (consumer && gl == 0) {
        sm[group] = m;
        sl[group] = l;
    }
    __syncthreads();
    float M = NEG_BIG;
    for (int g = 0; g < GR_KEYS; ++g)
        if (sl[g] > 0.f) M = fmaxf(M, sm[g]);
    float L = 0.f;
    for (int g = 0; g < GR_KEYS; ++g)
        if (sl[g] > 0.f) L += sl[g] * expf(sm[g] - M);
    const float mine = (consumer && l > 0.f) ? expf(m - M) : 0.f;
    constexpr int PER = (vdim + GR_CONSUMERS - 1) / GR_CONSUMERS;
    float total[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) total[i] = 0.f;
    for (int round = 0; round < GR_KEYS / 8; ++round) {
        __syncthreads();
        if (consumer && group / 8 == round) {
#pragma unroll
            for (int c = 0; c < VC; ++c)
#pragma unroll
                for (int i = 0; i < 8; ++i) sacc[group & 7][(c * 8 + gl) * 8 + i] = acc[c][i] * mine;
        }
        __syncthreads();
        if (consumer) {
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = tid + i * GR_CONSUMERS;
                if (d < vdim)
#pragma unroll
                    for (int g = 0; g < 8; ++g) total[i] += sacc[g][d];
            }
        }
    }
    const size_t prow = (size_t)row * splits + split;
    if (consumer) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = tid + i * GR_CONSUMERS;
            if (d < vdim) part_acc[prow * vdim + d] = total[i];
        }
    }
    if (tid == 0) {
        part_ml[prow * 2] = M;
        part_ml[prow * 2 + 1] = L;
    }
}

// Merge of the splits plus the current token (its key and value in f32).  One CTA of 256 threads per (batch, head).
__global__ void __launch_bounds__(256)
glm_paged_decode_merge_kernel(const float* __restrict__ q, const float* __restrict__ cur_k,
                              const float* __restrict__ cur_v, const float* __restrict__ part_acc,
                              const float* __restrict__ part_ml, float* __restrict__ out, int dim, int vdim, int splits) {
    __shared__ float red[8];
    const int row = blockIdx.x, tid = threadIdx.x;
    float dot = 0.f;
    for (int d = tid; d < dim; d += 256) dot += q[(size_t)row * dim + d] * cur_k[(size_t)row * dim + d];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if ((tid & 31) == 0) red[tid >> 5] = dot;
    __syncthreads();
    const float s_cur = (red[0] + red[1] + red[2] + red[3] + red[4] + red[5] + red[6] + red[7]) / sqrtf((float)dim);
    float M = s_cur;
    for (int s = 0; s < splits; ++s)
        if (part_ml[((size_t)row * splits + s) * 2 + 1] > 0.f) M = fmaxf(M, part_ml[((size_t)row * splits + s) * 2]);
    const float w_cur = expf(s_cur - M);
    float L = w_cur;
    for (int s = 0; s < splits; ++s) {
        const float ls = part_ml[((size_t)row * splits + s) * 2 + 1];
        if (ls > 0.f) L += ls * expf(part_ml[((size_t)row * splits + s) * 2] - M);
    }
    for (int d = tid; d < vdim; d += 256) {
        float a = w_cur * cur_v[(size_t)row * vdim + d];
        for (int s = 0; s < splits; ++s) {
            const float ls = part_ml[((size_t)row * splits + s) * 2 + 1];
            if (ls > 0.f) a += part_acc[((size_t)row * splits + s) * vdim + d] * expf(part_ml[((size_t)row * splits + s) * 2] - M);
        }
        out[(size_t)row * vdim + d] = a / L;
    }
}

template <int KC, int VC>
int launch_glm_split(inf_ctx* ctx, const float* q, const void* pk, const float* cur_k, const void* pv, const float* cur_v,
                     int batch, int heads, int past, int page_size, float* out) {
    const int rows = batch * heads;
    const bool use_ring = page_size % GR_KEYS == 0;
    // the form whose threads load the rows themselves aims at two full waves of the CTAs an SM holds
    int splits = use_ring ? (7 * ctx->sm_count / 4 + rows / 2) / rows : (2 * INF_GLM_CTAS * ctx->sm_count) / rows;
    splits = std::max(1, std::min(splits, (past + 255) / 256));
    const int keys_per_split = ((past + splits - 1) / splits + GS_GROUPS - 1) / GS_GROUPS * GS_GROUPS;
    splits = (past + keys_per_split - 1) / keys_per_split;
    const size_t acc_bytes = (size_t)rows * splits * VC * 64 * sizeof(float);
    int rc = inf_ensure_workspace(ctx, acc_bytes + (size_t)rows * splits * 2 * sizeof(float));
    if (rc != INF_OK) return rc;
    float* part_acc = (float*)ctx->workspace;
    float* part_ml = (float*)((char*)ctx->workspace + acc_bytes);
    if (use_ring) {
        constexpr size_t ring_bytes = (size_t)GR_STAGES * GR_KEYS * (KC + VC) * 64 * 2;
        constexpr uint32_t attr_bit = 1u << (16 + (KC * 4 + VC) % 12);  // (4,4) (3,2) (4,2) (2,2) (1,1): bits 24 18 22 26 21
        if (!(ctx->func_attr_done & attr_bit)) {
            INF_CUDA(ctx, cudaFuncSetAttribute(glm_paged_decode_ring_kernel<KC, VC>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring_bytes));
            ctx->func_attr_done |= attr_bit;
        }
        inf_prof_scope prof(ctx, "glm_paged_decode_split_kernel");
        glm_paged_decode_ring_kernel<KC, VC><<<dim3(splits, rows), GR_THREADS, ring_bytes, ctx->stream>>>(
            q, (const __half*)pk, (const __half*)pv, part_acc, part_ml, batch, heads, past, page_size, keys_per_split, splits,
            ctx->status);
    } else {
        inf_prof_scope prof(ctx, "glm_paged_decode_split_kernel");
        glm_paged_decode_split_kernel<KC, VC><<<dim3(splits, rows), GS_THREADS, 0, ctx->stream>>>(
            q, (const __half*)pk, (const __half*)pv, part_acc, part_ml, batch, heads, past, page_size, keys_per_split, splits);
    }
    INF_LAUNCH_CHECK(ctx, "glm_paged_decode_split_kernel");
    glm_paged_decode_merge_kernel<<<rows, 256, 0, ctx->stream>>>(q, cur_k, cur_v, part_acc, part_ml, out, KC * 64, VC * 64, splits);
    INF_LAUNCH_CHECK(ctx, "glm_paged_decode_merge_kernel");
    return INF_OK;
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
                                     INF_DTYPE_F32, (char*)ctx->workspace + q_bytes, dec_bytes, 1, nullptr, nullptr, 0);
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
    // the key-split form wants dims that are multiples of 64, 16-byte aligned caches and enough keys to split
    if (past_tokens >= 256 && head_dim % 64 == 0 && value_dim % 64 == 0 &&
        !(((uintptr_t)paged_k_f16 | (uintptr_t)paged_v_f16) & 15u)) {
#define GLM_CASE(KC_, VC_)                                                                                      \
    if (head_dim == KC_ * 64 && value_dim == VC_ * 64)                                                          \
        return launch_glm_split<KC_, VC_>(ctx, q, paged_k_f16, cur_k, paged_v_f16, cur_v, batch, heads, past_tokens, \
                                          page_size, out);
        GLM_CASE(4, 4) GLM_CASE(3, 2) GLM_CASE(4, 2) GLM_CASE(2, 2) GLM_CASE(1, 1)
#undef GLM_CASE
    }
    glm_paged_decode_kernel<<<batch * heads, GLM_THREADS, 0, ctx->stream>>>(
        q, (const __half*)paged_k_f16, cur_k, (const __half*)paged_v_f16, cur_v, out, batch, heads, past_tokens,
        page_size, head_dim, value_dim);
    INF_LAUNCH_CHECK(ctx, "glm_paged_decode_kernel");
    return INF_OK;
}

}  // extern "C"

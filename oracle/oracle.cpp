// CPU oracle for the attention hot path -- TEST INFRASTRUCTURE, NOT PRODUCT.
// See oracle.h for the contract.  Scalar f32 arithmetic throughout, in the evaluation
// order of the reference kernels wherever that order is observable.
#include "oracle.h"

#include <math.h>
#include <string.h>

#include <algorithm>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

const float NEG_INF = -3.4028234663852886e+38f;  // kernels/fp8_attention_kernels.metal:9

inline uint32_t f32_bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    return u;
}
inline float bits_f32(uint32_t u) {
    float x;
    memcpy(&x, &u, 4);
    return x;
}

// kernels/fp8_attention_kernels.metal:56-64
inline float softplus(float v) {
    if (v > 20.0f) return v;
    if (v < -20.0f) return expf(v);
    return logf(1.0f + expf(v));
}

struct Online {  // one online-softmax state, f16_attention_kernels.metal:84-90
    float running_max = NEG_INF, running_sum = 0.0f;
    void step(float score, const float* value, float* acc, int dim) {
        float next_max = fmaxf(running_max, score);
        float rescale = running_sum == 0.0f ? 0.0f : expf(running_max - next_max);
        float weight = expf(score - next_max);
        running_sum = running_sum * rescale + weight;
        running_max = next_max;
        for (int d = 0; d < dim; ++d) acc[d] = acc[d] * rescale + weight * value[d];
    }
};

inline float dotf(const float* a, const float* b, int n) {
    float s = 0.0f;
    for (int i = 0; i < n; ++i) s += a[i] * b[i];
    return s;
}

inline uint64_t splitmix64(uint64_t& s) {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
inline uint64_t stream_at(uint64_t seed, uint64_t index) {
    uint64_t s = seed + index * 0x9E3779B97F4A7C15ull;
    return splitmix64(s);
}

}  // namespace

extern "C" {

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Number of OpenMP threads later calls use (a launcher may have exported OMP_NUM_THREADS=1 for its workers).
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

uint16_t orc_f32_to_f16(float x) {
    uint32_t u = f32_bits(x);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t mag = u & 0x7FFFFFFFu;
    if (mag >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (mag > 0x7F800000u ? 0x200u : 0u));
    if (mag >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  // rounds to inf (>= 65520)
    if (mag < 0x33000001u) return (uint16_t)sign;                // below half of the smallest subnormal
    int32_t exp = (int32_t)(mag >> 23) - 127;
    uint32_t man = (mag & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half_exp;
    if (exp < -14) {
        shift = (uint32_t)(13 + (-14 - exp));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(exp + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    uint32_t out;
    if (half_exp == 0)
        out = q;  // subnormal; a carry into bit 10 lands on the smallest normal
    else
        out = ((half_exp - 1) << 10) + q;  // q carries the implicit bit
    return (uint16_t)(sign | out);
}

float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        float v = (float)man * 5.9604644775390625e-8f;  // 2^-24
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

void orc_round_to_f16(const float* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = orc_f16_to_f32(orc_f32_to_f16(in[i]));
}

void orc_fill_normal(float* out, int64_t n, uint64_t seed, float sigma, int round_f16) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint64_t a = stream_at(seed, (uint64_t)(2 * i));
        uint64_t b = stream_at(seed, (uint64_t)(2 * i + 1));
        double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740993.0);  // (0,1)
        double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);
        float v = (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2)) * sigma;
        out[i] = round_f16 ? orc_f16_to_f32(orc_f32_to_f16(v)) : v;
    }
}

void orc_permutation(int32_t* out, int32_t n, uint64_t seed) {
    for (int32_t i = 0; i < n; ++i) out[i] = i;
    uint64_t s = seed;
    for (int32_t i = n - 1; i > 0; --i) {
        uint32_t j = (uint32_t)(splitmix64(s) % (uint64_t)(i + 1));
        std::swap(out[i], out[j]);
    }
}

void orc_uniform_int(int32_t* out, int32_t n, int32_t lo, int32_t hi, uint64_t seed) {
    uint64_t s = seed;
    for (int32_t i = 0; i < n; ++i) out[i] = lo + (int32_t)(splitmix64(s) % (uint64_t)(hi - lo + 1));
}

// crates/config/src/laguna.rs:600-615
void orc_default_inv_freq(float theta, int rotary_dim, float* inv_freq) {
    for (int i = 0; i < rotary_dim / 2; ++i) inv_freq[i] = 1.0f / powf(theta, (float)(2 * i) / (float)rotary_dim);
}

// crates/config/src/laguna.rs:617-667
void orc_yarn_inv_freq(float theta, int rotary_dim, float factor, float original_context, float beta_fast,
                       float beta_slow, float* inv_freq) {
    auto correction = [&](float rotations) {
        return (float)rotary_dim * logf(original_context / (rotations * 2.0f * 3.14159265358979323846f)) /
               (2.0f * logf(theta));
    };
    float low = fmaxf(floorf(correction(beta_fast)), 0.0f);
    float high = fminf(ceilf(correction(beta_slow)), (float)(rotary_dim - 1));
    float ramp_den = low == high ? 0.001f : high - low;
    for (int i = 0; i < rotary_dim / 2; ++i) {
        float pf = powf(theta, (float)(2 * i) / (float)rotary_dim);
        float interpolated = 1.0f / (factor * pf);
        float extrapolated = 1.0f / pf;
        float ramp = fminf(fmaxf(((float)i - low) / ramp_den, 0.0f), 1.0f);
        float ef = 1.0f - ramp;
        inv_freq[i] = interpolated * (1.0f - ef) + extrapolated * ef;
    }
}

// kernels/rope_kernels.metal:167-229 (one head row)
static void norm_rope_row(const float* in, const float* w, const float* inv_freq, float* out, int head_dim,
                          int rotary_dim, float position, float eps, float factor) {
    float inverse_rms = 1.0f;
    if (w) {
        float sumsq = 0.0f;
        for (int d = 0; d < head_dim; ++d) sumsq += in[d] * in[d];
        inverse_rms = 1.0f / sqrtf(sumsq / (float)head_dim + eps);
    }
    int half = rotary_dim / 2;
    for (int d = 0; d < head_dim; ++d) {
        float normalized = w ? in[d] * w[d] * inverse_rms : in[d];
        if (d >= rotary_dim) {
            out[d] = normalized;
            continue;
        }
        int pd = d < half ? d + half : d - half;
        float paired = w ? in[pd] * w[pd] * inverse_rms : in[pd];
        float rotated = d < half ? -paired : paired;
        float angle = position * inv_freq[d % half];
        float c = cosf(angle) * factor, s = sinf(angle) * factor;
        out[d] = normalized * c + rotated * s;
    }
}

void orc_qk_norm_rope_half_split(const float* input, const float* norm_weight, const float* inv_freq, float* output,
                                 int64_t rows, int tokens, int heads, int head_dim, int rotary_dim,
                                 int position_offset, float eps, float attention_factor) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        int token = (int)((row / heads) % tokens);
        norm_rope_row(input + row * head_dim, norm_weight, inv_freq, output + row * head_dim, head_dim, rotary_dim,
                      (float)(position_offset + token), eps, attention_factor);
    }
}

void orc_qk_norm_rope_half_split_pos(const float* input, const float* norm_weight, const float* inv_freq,
                                     float* output, int batch, int tokens, int heads, int head_dim, int rotary_dim,
                                     const int32_t* positions, float eps, float attention_factor) {
    int64_t rows = (int64_t)batch * tokens * heads;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        int token = (int)((row / heads) % tokens);
        int b = (int)(row / ((int64_t)heads * tokens));
        norm_rope_row(input + row * head_dim, norm_weight, inv_freq, output + row * head_dim, head_dim, rotary_dim,
                      (float)(positions[b] + token), eps, attention_factor);
    }
}

// kernels/rope_kernels.metal:5-40
void orc_rope_slice_glm(const float* input, float* output, int batch, int tokens, int heads, int rope_dim,
                        int position_offset, float theta) {
    int pair_count = rope_dim / 2;
    for (int b = 0; b < batch; ++b)
        for (int t = 0; t < tokens; ++t)
            for (int h = 0; h < heads; ++h) {
                int64_t base = (((int64_t)b * tokens + t) * heads + h) * rope_dim;
                for (int p = 0; p < pair_count; ++p) {
                    float inv_freq = 1.0f / powf(theta, (float)p / (float)pair_count);
                    float angle = (float)(position_offset + t) * inv_freq;
                    float c = cosf(angle), s = sinf(angle);
                    float even = input[base + 2 * p], odd = input[base + 2 * p + 1];
                    output[base + 2 * p] = even * c - odd * s;
                    output[base + 2 * p + 1] = even * s + odd * c;
                }
            }
}

// kernels/norm_kernels.metal:52-115
void orc_mla_kv_postprocess(const float* input, const float* norm_weight, float* latent_out, float* rope_out,
                            int64_t rows, int tokens, int latent_dim, int rope_dim, int position_offset, float theta,
                            float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const float* in = input + row * (latent_dim + rope_dim);
        float sumsq = 0.0f;
        for (int d = 0; d < latent_dim; ++d) sumsq += in[d] * in[d];
        float norm_scale = 1.0f / sqrtf(sumsq / (float)latent_dim + eps);
        for (int d = 0; d < latent_dim; ++d) latent_out[row * latent_dim + d] = in[d] * norm_scale * norm_weight[d];
        int position = position_offset + (int)(row % tokens);
        int pair_count = rope_dim / 2;
        for (int d = 0; d < rope_dim; ++d) {
            int pair = d / 2;
            bool even = (d & 1) == 0;
            int partner = even ? d + 1 : d - 1;
            float inv_freq = 1.0f / powf(theta, (float)pair / (float)pair_count);
            float angle = (float)position * inv_freq;
            float value = in[latent_dim + d], pv = in[latent_dim + partner];
            float rotated = even ? -pv : pv;
            rope_out[row * rope_dim + d] = value * cosf(angle) + rotated * sinf(angle);
        }
    }
}

// kernels/f16_attention_kernels.metal:8-145 / :153-316
void orc_gqa_ring_attention(const float* query, const float* cur_key, const float* cur_value, const float* gate,
                            uint16_t* cached_key, uint16_t* cached_value, float* output, int batch, int q_heads,
                            int kv_heads, int head_dim, int q_tokens, int past_tokens, int stored_tokens,
                            int capacity, int sliding_window, int fuse_append) {
    int heads_per_kv = q_heads / kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    int64_t rows = (int64_t)batch * q_tokens * q_heads;
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t row = 0; row < rows; ++row) {
        int qh = (int)(row % q_heads);
        int qt = (int)((row / q_heads) % q_tokens);
        int b = (int)(row / ((int64_t)q_heads * q_tokens));
        int kvh = qh / heads_per_kv;
        int abs_q = past_tokens + qt;
        int visible_start = (sliding_window == 0 || abs_q + 1 <= sliding_window) ? 0 : abs_q + 1 - sliding_window;
        int cached_start = past_tokens - stored_tokens;
        int past_start = std::min(past_tokens, std::max(visible_start, cached_start));
        int past_count = past_tokens - past_start;
        int current_start = visible_start > past_tokens ? visible_start - past_tokens : 0;
        int current_count = qt - current_start + 1;
        int key_count = past_count + current_count;
        const float* q = query + row * head_dim;
        std::vector<float> acc(head_dim, 0.0f), kf(head_dim), vf(head_dim);
        Online st;
        for (int lk = 0; lk < key_count; ++lk) {
            const float *kp, *vp;
            if (lk < past_count) {
                int slot = (past_start + lk) % capacity;
                int64_t idx = (((int64_t)b * capacity + slot) * kv_heads + kvh) * head_dim;
                for (int d = 0; d < head_dim; ++d) {
                    kf[d] = orc_f16_to_f32(cached_key[idx + d]);
                    vf[d] = orc_f16_to_f32(cached_value[idx + d]);
                }
                kp = kf.data();
                vp = vf.data();
            } else {
                int ct = current_start + lk - past_count;
                int64_t idx = (((int64_t)b * q_tokens + ct) * kv_heads + kvh) * head_dim;
                kp = cur_key + idx;
                vp = cur_value + idx;
            }
            st.step(dotf(q, kp, head_dim) * scale, vp, acc.data(), head_dim);
        }
        float g = gate ? softplus(gate[((int64_t)b * q_tokens + qt) * q_heads + qh]) : 1.0f;
        float gain = g / st.running_sum;
        for (int d = 0; d < head_dim; ++d) output[row * head_dim + d] = acc[d] * gain;
    }
    if (fuse_append) {
        for (int b = 0; b < batch; ++b)
            for (int t = 0; t < q_tokens; ++t) {
                int slot = (past_tokens + t) % capacity;
                for (int h = 0; h < kv_heads; ++h) {
                    int64_t src = (((int64_t)b * q_tokens + t) * kv_heads + h) * head_dim;
                    int64_t dst = (((int64_t)b * capacity + slot) * kv_heads + h) * head_dim;
                    for (int d = 0; d < head_dim; ++d) {
                        cached_key[dst + d] = orc_f32_to_f16(cur_key[src + d]);
                        cached_value[dst + d] = orc_f32_to_f16(cur_value[src + d]);
                    }
                }
            }
    }
}

// metal/f16_attention.rs:1079-1187
void orc_test_cpu_gqa(const float* query, const float* key, const float* value, const float* gate, float* output,
                      int tokens, int q_heads, int kv_heads, int head_dim, int sliding_window, int last_only) {
    int heads_per_kv = q_heads / kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    for (int token = last_only ? tokens - 1 : 0; token < tokens; ++token) {
        int first_key = (sliding_window == 0 || token < sliding_window) ? 0 : token + 1 - sliding_window;
        for (int qh = 0; qh < q_heads; ++qh) {
            int kvh = qh / heads_per_kv;
            const float* q = query + ((int64_t)token * q_heads + qh) * head_dim;
            std::vector<float> scores;
            for (int kt = first_key; kt <= token; ++kt)
                scores.push_back(dotf(q, key + ((int64_t)kt * kv_heads + kvh) * head_dim, head_dim) * scale);
            float maximum = -INFINITY;
            for (float s : scores) maximum = fmaxf(maximum, s);
            std::vector<float> weights;
            float denom = 0.0f;
            for (float s : scores) {
                weights.push_back(expf(s - maximum));
                denom += weights.back();
            }
            float gain = gate ? logf(1.0f + expf(gate[(int64_t)token * q_heads + qh])) : 1.0f;
            float* out = output + (last_only ? (int64_t)qh * head_dim : ((int64_t)token * q_heads + qh) * head_dim);
            for (int d = 0; d < head_dim; ++d) {
                float weighted = 0.0f;
                for (size_t o = 0; o < weights.size(); ++o)
                    weighted += weights[o] * value[((int64_t)(first_key + (int)o) * kv_heads + kvh) * head_dim + d];
                out[d] = weighted / denom * gain;
            }
        }
    }
}

// kernels/f16_attention_kernels.metal:325-510
void orc_gqa_ring_decode_segmented(const float* query, const float* cur_key, const float* cur_value,
                                   const float* gate, uint16_t* cached_key, uint16_t* cached_value, float* output,
                                   int batch, int q_heads, int kv_heads, int head_dim, int past_tokens,
                                   int cached_start, int cached_count, int capacity, int segment_tokens) {
    int heads_per_kv = q_heads / kv_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    int key_count = cached_count + 1;
    int segment_count = (key_count + segment_tokens - 1) / segment_tokens;
    std::vector<float> pmax((size_t)batch * segment_count * q_heads), psum(pmax.size()),
        pacc(pmax.size() * head_dim);
    for (int b = 0; b < batch; ++b)
        for (int seg = 0; seg < segment_count; ++seg)
            for (int qh = 0; qh < q_heads; ++qh) {
                int kvh = qh / heads_per_kv;
                int seg_start = seg * segment_tokens;
                int seg_end = std::min(key_count, seg_start + segment_tokens);
                const float* q = query + ((int64_t)b * q_heads + qh) * head_dim;
                std::vector<float> acc(head_dim, 0.0f), kf(head_dim), vf(head_dim);
                Online st;
                for (int lk = seg_start; lk < seg_end; ++lk) {
                    const float *kp, *vp;
                    if (lk < cached_count) {
                        int slot = (cached_start + lk) % capacity;
                        int64_t idx = (((int64_t)b * capacity + slot) * kv_heads + kvh) * head_dim;
                        for (int d = 0; d < head_dim; ++d) {
                            kf[d] = orc_f16_to_f32(cached_key[idx + d]);
                            vf[d] = orc_f16_to_f32(cached_value[idx + d]);
                        }
                        kp = kf.data();
                        vp = vf.data();
                    } else {
                        int64_t idx = ((int64_t)b * kv_heads + kvh) * head_dim;
                        kp = cur_key + idx;
                        vp = cur_value + idx;
                    }
                    st.step(dotf(q, kp, head_dim) * scale, vp, acc.data(), head_dim);
                }
                size_t prow = ((size_t)b * segment_count + seg) * q_heads + qh;
                pmax[prow] = st.running_max;
                psum[prow] = st.running_sum;
                memcpy(&pacc[prow * head_dim], acc.data(), sizeof(float) * head_dim);
            }
    for (int b = 0; b < batch; ++b)
        for (int qh = 0; qh < q_heads; ++qh) {
            float merged_max = NEG_INF, merged_sum = 0.0f;
            std::vector<float> merged(head_dim, 0.0f);
            for (int seg = 0; seg < segment_count; ++seg) {
                size_t prow = ((size_t)b * segment_count + seg) * q_heads + qh;
                float next_max = fmaxf(merged_max, pmax[prow]);
                float merged_scale = merged_sum == 0.0f ? 0.0f : expf(merged_max - next_max);
                float segment_scale = expf(pmax[prow] - next_max);
                merged_sum = merged_sum * merged_scale + psum[prow] * segment_scale;
                for (int d = 0; d < head_dim; ++d)
                    merged[d] = merged[d] * merged_scale + pacc[prow * head_dim + d] * segment_scale;
                merged_max = next_max;
            }
            float g = gate ? softplus(gate[(int64_t)b * q_heads + qh]) : 1.0f;
            float gain = g / merged_sum;
            for (int d = 0; d < head_dim; ++d) output[((int64_t)b * q_heads + qh) * head_dim + d] = merged[d] * gain;
        }
    for (int b = 0; b < batch; ++b)
        for (int h = 0; h < kv_heads; ++h) {
            int slot = past_tokens % capacity;
            int64_t src = ((int64_t)b * kv_heads + h) * head_dim;
            int64_t dst = (((int64_t)b * capacity + slot) * kv_heads + h) * head_dim;
            for (int d = 0; d < head_dim; ++d) {
                cached_key[dst + d] = orc_f32_to_f16(cur_key[src + d]);
                cached_value[dst + d] = orc_f32_to_f16(cur_value[src + d]);
            }
        }
}

static inline int64_t paged_row(const int32_t* page_table, int max_pages, int b, int token, int page_size,
                                int kv_heads, int kvh, int head_dim) {
    int32_t page = page_table[(int64_t)b * max_pages + token / page_size];
    return ((((int64_t)page * kv_heads + kvh) * page_size) + token % page_size) * head_dim;
}

void orc_gqa_paged_attention(const float* query, const float* cur_key, const float* cur_value, const float* gate,
                             uint16_t* k_pool, uint16_t* v_pool, const int32_t* page_table, int max_pages,
                             const int32_t* past_tokens, float* output, int batch, int q_heads, int kv_heads,
                             int head_dim, int page_size, int q_tokens, int sliding_window, int fuse_append,
                             float scale, int threads) {
    int heads_per_kv = q_heads / kv_heads;
    if (scale <= 0.0f) scale = 1.0f / sqrtf((float)head_dim);
    int64_t rows = (int64_t)batch * q_tokens * q_heads;
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : orc_max_threads())
    for (int64_t row = 0; row < rows; ++row) {
        int qh = (int)(row % q_heads);
        int qt = (int)((row / q_heads) % q_tokens);
        int b = (int)(row / ((int64_t)q_heads * q_tokens));
        int kvh = qh / heads_per_kv;
        int past = past_tokens[b];
        int abs_q = past + qt;
        int visible_start = (sliding_window == 0 || abs_q + 1 <= sliding_window) ? 0 : abs_q + 1 - sliding_window;
        int past_start = std::min(past, visible_start);
        int past_count = past - past_start;
        int current_start = visible_start > past ? visible_start - past : 0;
        int current_count = qt - current_start + 1;
        int key_count = past_count + current_count;
        const float* q = query + row * head_dim;
        std::vector<float> acc(head_dim, 0.0f), kf(head_dim), vf(head_dim);
        Online st;
        for (int lk = 0; lk < key_count; ++lk) {
            const float *kp, *vp;
            if (lk < past_count) {
                int64_t idx = paged_row(page_table, max_pages, b, past_start + lk, page_size, kv_heads, kvh, head_dim);
                for (int d = 0; d < head_dim; ++d) {
                    kf[d] = orc_f16_to_f32(k_pool[idx + d]);
                    vf[d] = orc_f16_to_f32(v_pool[idx + d]);
                }
                kp = kf.data();
                vp = vf.data();
            } else {
                int ct = current_start + lk - past_count;
                int64_t idx = (((int64_t)b * q_tokens + ct) * kv_heads + kvh) * head_dim;
                kp = cur_key + idx;
                vp = cur_value + idx;
            }
            st.step(dotf(q, kp, head_dim) * scale, vp, acc.data(), head_dim);
        }
        float g = gate ? softplus(gate[((int64_t)b * q_tokens + qt) * q_heads + qh]) : 1.0f;
        float gain = g / st.running_sum;
        for (int d = 0; d < head_dim; ++d) output[row * head_dim + d] = acc[d] * gain;
    }
    if (fuse_append) {
        for (int b = 0; b < batch; ++b)
            for (int t = 0; t < q_tokens; ++t)
                for (int h = 0; h < kv_heads; ++h) {
                    int64_t src = (((int64_t)b * q_tokens + t) * kv_heads + h) * head_dim;
                    int64_t dst =
                        paged_row(page_table, max_pages, b, past_tokens[b] + t, page_size, kv_heads, h, head_dim);
                    for (int d = 0; d < head_dim; ++d) {
                        k_pool[dst + d] = orc_f32_to_f16(cur_key[src + d]);
                        v_pool[dst + d] = orc_f32_to_f16(cur_value[src + d]);
                    }
                }
    }
}

// ---- FP8 E4M3FN pages -------------------------------------------------------------------------------
// kernels/fp8_attention_kernels.metal:11-27
float orc_fp8_e4m3fn_decode(uint8_t bits) {
    uint32_t sign = bits >> 7, exponent = (bits >> 3) & 0x0fu, mantissa = bits & 0x07u;
    if (exponent == 15u && mantissa == 7u) return 0.0f;
    float magnitude = exponent == 0u ? (float)mantissa * 0.001953125f
                                     : (1.0f + (float)mantissa * 0.125f) * exp2f((float)((int)exponent - 7));
    return sign == 0u ? magnitude : -magnitude;
}

// kernels/fp8_attention_kernels.metal:29-54
uint8_t orc_fp8_e4m3fn_encode(float value) {
    if (std::isnan(value) || value == 0.0f) return 0;
    uint32_t sign = value < 0.0f ? 0x80u : 0u;
    float magnitude = std::min(fabsf(value), 448.0f);
    if (magnitude < 0.015625f) {
        uint32_t mantissa = (uint32_t)nearbyintf(magnitude * 512.0f);
        return (uint8_t)(sign | std::min(mantissa, 8u));
    }
    int unbiased = (int)floorf(log2f(magnitude));
    uint32_t exponent = (uint32_t)(unbiased + 7);
    float normalized = magnitude * exp2f((float)(-unbiased));
    uint32_t mantissa = (uint32_t)nearbyintf((normalized - 1.0f) * 8.0f);
    if (mantissa == 8u) {
        mantissa = 0u;
        exponent += 1u;
    }
    if (exponent > 15u || (exponent == 15u && mantissa > 6u)) {
        exponent = 15u;
        mantissa = 6u;
    }
    return (uint8_t)(sign | (exponent << 3) | mantissa);
}

// kernels/fp8_attention_kernels.metal:70-225 (attention) and :227-263 (append), over pages: cached rows are
// decode(byte) * scale, the current chunk's rows are f32, the append stores encode(x / scale) afterwards.
void orc_gqa_paged_attention_fp8(const float* query, const float* cur_key, const float* cur_value, const float* gate,
                                 uint8_t* k_pool, uint8_t* v_pool, float key_scale, float value_scale,
                                 const int32_t* page_table, int max_pages, const int32_t* past_tokens, float* output,
                                 int batch, int q_heads, int kv_heads, int head_dim, int page_size, int q_tokens,
                                 int sliding_window, int fuse_append, float scale, int threads) {
    int heads_per_kv = q_heads / kv_heads;
    if (scale <= 0.0f) scale = 1.0f / sqrtf((float)head_dim);
    int64_t rows = (int64_t)batch * q_tokens * q_heads;
    (void)threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : orc_max_threads())
    for (int64_t row = 0; row < rows; ++row) {
        int qh = (int)(row % q_heads);
        int qt = (int)((row / q_heads) % q_tokens);
        int b = (int)(row / ((int64_t)q_heads * q_tokens));
        int kvh = qh / heads_per_kv;
        int past = past_tokens[b];
        int abs_q = past + qt;
        int visible_start = (sliding_window == 0 || abs_q + 1 <= sliding_window) ? 0 : abs_q + 1 - sliding_window;
        int past_start = std::min(past, visible_start);
        int past_count = past - past_start;
        int current_start = visible_start > past ? visible_start - past : 0;
        int current_count = qt - current_start + 1;
        int key_count = past_count + current_count;
        const float* q = query + row * head_dim;
        std::vector<float> acc(head_dim, 0.0f), kf(head_dim), vf(head_dim);
        Online st;
        for (int lk = 0; lk < key_count; ++lk) {
            const float *kp, *vp;
            if (lk < past_count) {
                int64_t idx = paged_row(page_table, max_pages, b, past_start + lk, page_size, kv_heads, kvh, head_dim);
                for (int d = 0; d < head_dim; ++d) {
                    kf[d] = orc_fp8_e4m3fn_decode(k_pool[idx + d]) * key_scale;
                    vf[d] = orc_fp8_e4m3fn_decode(v_pool[idx + d]) * value_scale;
                }
                kp = kf.data();
                vp = vf.data();
            } else {
                int ct = current_start + lk - past_count;
                int64_t idx = (((int64_t)b * q_tokens + ct) * kv_heads + kvh) * head_dim;
                kp = cur_key + idx;
                vp = cur_value + idx;
            }
            st.step(dotf(q, kp, head_dim) * scale, vp, acc.data(), head_dim);
        }
        float g = gate ? softplus(gate[((int64_t)b * q_tokens + qt) * q_heads + qh]) : 1.0f;
        float gain = g / st.running_sum;
        for (int d = 0; d < head_dim; ++d) output[row * head_dim + d] = acc[d] * gain;
    }
    if (fuse_append) {
        for (int b = 0; b < batch; ++b)
            for (int t = 0; t < q_tokens; ++t)
                for (int h = 0; h < kv_heads; ++h) {
                    int64_t src = (((int64_t)b * q_tokens + t) * kv_heads + h) * head_dim;
                    int64_t dst =
                        paged_row(page_table, max_pages, b, past_tokens[b] + t, page_size, kv_heads, h, head_dim);
                    for (int d = 0; d < head_dim; ++d) {
                        k_pool[dst + d] = orc_fp8_e4m3fn_encode(cur_key[src + d] / key_scale);
                        v_pool[dst + d] = orc_fp8_e4m3fn_encode(cur_value[src + d] / value_scale);
                    }
                }
    }
}

// kernels/attention_kernels.metal:605-721 (decode: T = 1, include_current flag) and :723-968 (sequence: row t sees
// the selected rows and current rows 0..t): every score, the maximum, the denominator, then the weighted sum.
void orc_selected_attention_f32(const float* q, const float* sel_k, const float* sel_v, const float* cur_k,
                                const float* cur_v, float* out, int batch, int heads, int S, int T, int D, int Dv,
                                int include_current) {
    const float scale = 1.0f / sqrtf((float)D);
    const int64_t rows = (int64_t)batch * heads * T;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const int t = (int)(row % T);
        const int64_t bh = row / T;
        const int visible = S + (include_current ? t + 1 : 0);
        std::vector<float> scores(visible);
        float mx = -3.4028234663852886e+38f;
        for (int key = 0; key < visible; ++key) {
            const float* kr = key < S ? sel_k + (bh * S + key) * D : cur_k + (bh * T + (key - S)) * D;
            scores[key] = dotf(q + row * D, kr, D) * scale;
            mx = std::max(mx, scores[key]);
        }
        float denom = 0.0f;
        for (int key = 0; key < visible; ++key) denom += expf(scores[key] - mx);
        for (int d = 0; d < Dv; ++d) {
            float sum = 0.0f;
            for (int key = 0; key < visible; ++key) {
                const float* vr = key < S ? sel_v + (bh * S + key) * Dv : cur_v + (bh * T + (key - S)) * Dv;
                sum += expf(scores[key] - mx) / denom * vr[d];
            }
            out[row * Dv + d] = sum;
        }
    }
}

void orc_linearize_paged(const uint16_t* pool, const int32_t* page_table, int max_pages, uint16_t* out, int batch,
                         int kv_heads, int tokens, int page_size, int head_dim) {
    for (int b = 0; b < batch; ++b)
        for (int h = 0; h < kv_heads; ++h)
            for (int t = 0; t < tokens; ++t) {
                int64_t src = paged_row(page_table, max_pages, b, t, page_size, kv_heads, h, head_dim);
                int64_t dst = (((int64_t)b * kv_heads + h) * tokens + t) * head_dim;
                memcpy(out + dst, pool + src, sizeof(uint16_t) * head_dim);
            }
}

// kernels/attention_kernels.metal:339-457
void orc_paged_decode_mha_f16(const float* q, const uint16_t* paged_k, const float* cur_k, const uint16_t* paged_v,
                              const float* cur_v, float* output, int batch, int heads, int past_tokens,
                              int page_size, int head_dim, int value_dim) {
    float scale = 1.0f / sqrtf((float)head_dim);
    int key_tokens = past_tokens + 1;
#pragma omp parallel for schedule(dynamic, 1)
    for (int row = 0; row < batch * heads; ++row) {
        int head = row % heads, b = row / heads;
        const float* qr = q + (int64_t)row * head_dim;
        std::vector<float> scores(key_tokens);
        for (int key = 0; key < key_tokens; ++key) {
            float dot = 0.0f;
            if (key < past_tokens) {
                int page = key / page_size, off = key - page * page_size;
                int64_t kb = ((((int64_t)page * batch + b) * heads + head) * page_size + off) * head_dim;
                for (int d = 0; d < head_dim; ++d) dot += qr[d] * orc_f16_to_f32(paged_k[kb + d]);
            } else {
                dot = dotf(qr, cur_k + (int64_t)row * head_dim, head_dim);
            }
            scores[key] = dot * scale;
        }
        float row_max = NEG_INF;
        for (float s : scores) row_max = fmaxf(row_max, s);
        float denom = 0.0f;
        for (float s : scores) denom += expf(s - row_max);
        for (int v = 0; v < value_dim; ++v) {
            float sum = 0.0f;
            for (int key = 0; key < past_tokens; ++key) {
                float p = expf(scores[key] - row_max) / denom;
                int page = key / page_size, off = key - page * page_size;
                int64_t vi = ((((int64_t)page * batch + b) * heads + head) * page_size + off) * value_dim + v;
                sum += p * orc_f16_to_f32(paged_v[vi]);
            }
            sum += expf(scores[past_tokens] - row_max) / denom * cur_v[(int64_t)row * value_dim + v];
            output[(int64_t)row * value_dim + v] = sum;
        }
    }
}

// metal/q2.rs:8506-8538
void orc_q8_0_heads_matvec(const uint8_t* weights, const float* input, float* output, int64_t rows, int heads,
                           int in_features, int out_features) {
    int blocks_per_row = in_features / 32;
    int64_t head_bytes = (int64_t)out_features * blocks_per_row * 34;
    for (int64_t r = 0; r < rows; ++r)
        for (int h = 0; h < heads; ++h) {
            const uint8_t* w = weights + h * head_bytes;
            const float* in = input + (r * heads + h) * in_features;
            for (int o = 0; o < out_features; ++o) {
                float sum = 0.0f;
                for (int blk = 0; blk < blocks_per_row; ++blk) {
                    const uint8_t* block = w + ((int64_t)o * blocks_per_row + blk) * 34;
                    float scale = orc_f16_to_f32((uint16_t)(block[0] | (block[1] << 8)));
                    for (int i = 0; i < 32; ++i) sum += in[blk * 32 + i] * scale * (float)(int8_t)block[2 + i];
                }
                output[(r * heads + h) * out_features + o] = sum;
            }
        }
}

// kernels/attention_kernels.metal:465-603
void orc_mla_absorbed_f32(const float* q_latent, const float* q_rope, const float* paged_latent,
                          const float* cur_latent, const float* paged_rope, const float* cur_rope, float* out_latent,
                          int batch, int heads, int q_tokens, int past_tokens, int page_size, int latent_dim,
                          int rope_dim, int scale_dim) {
    float scale = 1.0f / sqrtf((float)scale_dim);
    int rows = batch * q_tokens * heads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int row = 0; row < rows; ++row) {
        int query = (row / heads) % q_tokens;
        int b = row / (q_tokens * heads);
        int key_tokens = past_tokens + query + 1;
        const float* ql = q_latent + (int64_t)row * latent_dim;
        const float* qr = q_rope + (int64_t)row * rope_dim;
        std::vector<float> scores(key_tokens);
        auto latent_row = [&](int key) -> const float* {
            if (key < past_tokens) {
                int page = key / page_size, off = key - page * page_size;
                return paged_latent + (((int64_t)page * batch + b) * page_size + off) * latent_dim;
            }
            return cur_latent + ((int64_t)b * q_tokens + (key - past_tokens)) * latent_dim;
        };
        auto rope_row = [&](int key) -> const float* {
            if (key < past_tokens) {
                int page = key / page_size, off = key - page * page_size;
                return paged_rope + (((int64_t)page * batch + b) * page_size + off) * rope_dim;
            }
            return cur_rope + ((int64_t)b * q_tokens + (key - past_tokens)) * rope_dim;
        };
        for (int key = 0; key < key_tokens; ++key)
            scores[key] = (dotf(ql, latent_row(key), latent_dim) + dotf(qr, rope_row(key), rope_dim)) * scale;
        float row_max = NEG_INF;
        for (float s : scores) row_max = fmaxf(row_max, s);
        float denom = 0.0f;
        for (float s : scores) denom += expf(s - row_max);
        for (int d = 0; d < latent_dim; ++d) {
            float sum = 0.0f;
            for (int key = 0; key < key_tokens; ++key) sum += expf(scores[key] - row_max) / denom * latent_row(key)[d];
            out_latent[(int64_t)row * latent_dim + d] = sum;
        }
    }
}

void orc_mla_absorbed_paged(const float* q, const float* cur_rows, uint16_t* pool, const int32_t* page_table,
                            int max_pages, const int32_t* past_tokens, float* out, int batch, int heads, int q_tokens,
                            int page_size, int latent_dim, int rope_dim, float scale, int fuse_append, int threads) {
    int row_dim = latent_dim + rope_dim;
    int rows = batch * q_tokens * heads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : orc_max_threads())
    for (int row = 0; row < rows; ++row) {
        int query = (row / heads) % q_tokens;
        int b = row / (q_tokens * heads);
        int past = past_tokens[b];
        int key_tokens = past + query + 1;
        const float* qr = q + (int64_t)row * row_dim;
        std::vector<float> scores(key_tokens), rowf(row_dim);
        auto load_row = [&](int key, float* dst) {
            if (key < past) {
                int32_t page = page_table[(int64_t)b * max_pages + key / page_size];
                const uint16_t* src = pool + ((int64_t)page * page_size + key % page_size) * row_dim;
                for (int d = 0; d < row_dim; ++d) dst[d] = orc_f16_to_f32(src[d]);
            } else {
                memcpy(dst, cur_rows + ((int64_t)b * q_tokens + (key - past)) * row_dim, sizeof(float) * row_dim);
            }
        };
        float row_max = NEG_INF;
        for (int key = 0; key < key_tokens; ++key) {
            load_row(key, rowf.data());
            scores[key] = (dotf(qr, rowf.data(), latent_dim) + dotf(qr + latent_dim, rowf.data() + latent_dim, rope_dim)) * scale;
            row_max = fmaxf(row_max, scores[key]);
        }
        float denom = 0.0f;
        for (float s : scores) denom += expf(s - row_max);
        std::vector<float> acc(latent_dim, 0.0f);
        for (int key = 0; key < key_tokens; ++key) {
            load_row(key, rowf.data());
            float p = expf(scores[key] - row_max) / denom;
            for (int d = 0; d < latent_dim; ++d) acc[d] += p * rowf[d];
        }
        memcpy(out + (int64_t)row * latent_dim, acc.data(), sizeof(float) * latent_dim);
    }
    if (fuse_append) {
        for (int b = 0; b < batch; ++b)
            for (int t = 0; t < q_tokens; ++t) {
                int tok = past_tokens[b] + t;
                int32_t page = page_table[(int64_t)b * max_pages + tok / page_size];
                uint16_t* dst = pool + ((int64_t)page * page_size + tok % page_size) * row_dim;
                const float* src = cur_rows + ((int64_t)b * q_tokens + t) * row_dim;
                for (int d = 0; d < row_dim; ++d) dst[d] = orc_f32_to_f16(src[d]);
            }
    }
}

// kernels/attention_kernels.metal:723-968 with selected_tokens == 0
void orc_causal_mha(const float* q, const float* k_nope, const float* k_rope, const float* v, float* out, int tokens,
                    int heads, int nope_dim, int rope_dim, int v_dim, float scale, const int32_t* rows, int n_rows,
                    int threads) {
    int qk = nope_dim + rope_dim;
    if (!rows) n_rows = tokens;
    int64_t work = (int64_t)n_rows * heads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 0 ? threads : orc_max_threads())
    for (int64_t w = 0; w < work; ++w) {
        int ri = (int)(w / heads), h = (int)(w % heads);
        int t = rows ? rows[ri] : ri;
        const float* qr = q + ((int64_t)t * heads + h) * qk;
        std::vector<float> scores(t + 1);
        float row_max = NEG_INF;
        for (int key = 0; key <= t; ++key) {
            float dot = dotf(qr, k_nope + ((int64_t)key * heads + h) * nope_dim, nope_dim);
            if (rope_dim) dot += dotf(qr + nope_dim, k_rope + (int64_t)key * rope_dim, rope_dim);
            scores[key] = dot * scale;
            row_max = fmaxf(row_max, scores[key]);
        }
        float denom = 0.0f;
        for (int key = 0; key <= t; ++key) denom += expf(scores[key] - row_max);
        std::vector<float> acc(v_dim, 0.0f);
        for (int key = 0; key <= t; ++key) {
            float p = expf(scores[key] - row_max) / denom;
            const float* vr = v + ((int64_t)key * heads + h) * v_dim;
            for (int d = 0; d < v_dim; ++d) acc[d] += p * vr[d];
        }
        memcpy(out + ((int64_t)ri * heads + h) * v_dim, acc.data(), sizeof(float) * v_dim);
    }
}

}  // extern "C"

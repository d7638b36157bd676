/* CPU oracle for the attention hot path -- TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * A scalar restatement of the reference's Metal kernels and of the CPU helpers its
 * own tests compare them with.  Only the test-suite, the smoke check and the
 * benchmark's CPU-baseline leg may link or call this library; the CUDA library
 * never does.  Each function cites the reference source it follows (paths relative
 * to the reference project root).
 *
 * Parity is pinned: tests/test_oracle_pins.py replays the reference's known-answer
 * tests (closed-form inputs, the independent two-pass CPU statements written inside
 * the reference's test modules, and its analytic identities) against these functions.
 *
 * All pointers are host pointers.  fp16 data is carried as uint16_t bit patterns;
 * conversions are IEEE round-to-nearest-even.  Activations are f32 like the
 * reference's operator boundary.
 */
#ifndef INFERNO_ORACLE_H
#define INFERNO_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- fp16 helpers ------------------------------------------------------ */
uint16_t orc_f32_to_f16(float x);
float orc_f16_to_f32(uint16_t h);
void orc_round_to_f16(const float* in, float* out, int64_t n); /* f32 -> f16 -> f32 */

/* ---- deterministic generator shared with the harness ------------------- */
/* splitmix64 counter stream -> Box-Muller N(0, sigma), optionally rounded to fp16 values. */
void orc_fill_normal(float* out, int64_t n, uint64_t seed, float sigma, int round_f16);
/* Fisher-Yates permutation of 0..n-1 driven by the same stream. */
void orc_permutation(int32_t* out, int32_t n, uint64_t seed);
/* Uniform integer in [lo, hi] per element. */
void orc_uniform_int(int32_t* out, int32_t n, int32_t lo, int32_t hi, uint64_t seed);

/* ---- RoPE frequency tables (crates/config/src/laguna.rs:600-667) -------- */
void orc_default_inv_freq(float theta, int rotary_dim, float* inv_freq /* rotary_dim/2 */);
void orc_yarn_inv_freq(float theta, int rotary_dim, float factor, float original_context, float beta_fast,
                       float beta_slow, float* inv_freq);

/* ---- a1: per-head RMSNorm + half-split RoPE ----------------------------- */
/* kernels/rope_kernels.metal:113-229; CPU statement metal/rope.rs:828-875.
 * input/output [rows, head_dim] with rows = batch*tokens*heads; norm_weight may be NULL
 * (then the RMSNorm is skipped entirely).  position = position_offset + token. */
void orc_qk_norm_rope_half_split(const float* input, const float* norm_weight, const float* inv_freq, float* output,
                                 int64_t rows, int tokens, int heads, int head_dim, int rotary_dim,
                                 int position_offset, float eps, float attention_factor);
/* Same with an explicit position per (batch) row group: positions[b] replaces position_offset. */
void orc_qk_norm_rope_half_split_pos(const float* input, const float* norm_weight, const float* inv_freq,
                                     float* output, int batch, int tokens, int heads, int head_dim, int rotary_dim,
                                     const int32_t* positions, float eps, float attention_factor);

/* ---- a2: GLM interleaved-pair RoPE -------------------------------------- */
/* kernels/rope_kernels.metal:5-40; backend.rs:10148-10209; metal/rope.rs:877-912. */
void orc_rope_slice_glm(const float* input, float* output, int batch, int tokens, int heads, int rope_dim,
                        int position_offset, float theta);

/* ---- a3: MLA KV post-process -------------------------------------------- */
/* kernels/norm_kernels.metal:52-115: RMSNorm(latent)*w, interleaved RoPE(rope tail). */
void orc_mla_kv_postprocess(const float* input /* [rows, L+R] */, const float* norm_weight /* [L] */,
                            float* latent_out /* [rows,L] */, float* rope_out /* [rows,R] */, int64_t rows,
                            int tokens, int latent_dim, int rope_dim, int position_offset, float theta, float eps);

/* ---- a4/a5/a7: gated GQA attention over the f16 ring/linear cache ------- */
/* kernels/f16_attention_kernels.metal:8-145 (decode rows) and :153-316 (prefill rows):
 * identical math -- window, cached f16 keys then f32 current-chunk keys, online softmax
 * key by key, softplus(gate)/sum, fused append (RNE f32->f16) at slot abs % capacity.
 * gate may be NULL (gain = 1/sum).  cached_* are [batch, capacity, kv_heads, head_dim]. */
void orc_gqa_ring_attention(const float* query, const float* cur_key, const float* cur_value, const float* gate,
                            uint16_t* cached_key, uint16_t* cached_value, float* output, int batch, int q_heads,
                            int kv_heads, int head_dim, int q_tokens, int past_tokens, int stored_tokens,
                            int capacity, int sliding_window, int fuse_append);

/* Independent two-pass statement from the reference's tests
 * (metal/f16_attention.rs:1079-1187 cpu_decode_gqa / cpu_causal_gqa): all-f32, row `token` only
 * when last_only != 0. */
void orc_test_cpu_gqa(const float* query, const float* key, const float* value, const float* gate, float* output,
                      int tokens, int q_heads, int kv_heads, int head_dim, int sliding_window, int last_only);

/* ---- a6: segmented split-KV decode (partial + merge) --------------------- */
/* kernels/f16_attention_kernels.metal:325-510. */
void orc_gqa_ring_decode_segmented(const float* query, const float* cur_key, const float* cur_value,
                                   const float* gate, uint16_t* cached_key, uint16_t* cached_value, float* output,
                                   int batch, int q_heads, int kv_heads, int head_dim, int past_tokens,
                                   int cached_start, int cached_count, int capacity, int segment_tokens);

/* ---- P + a5/a6/a7 over pages (extension: arbitrary page tables, ragged batch) ---- */
/* Pool layout [num_pages][kv_heads][page_size][head_dim] fp16; logical token n of sequence b lives in
 * page page_table[b*max_pages + n/page_size] at offset n%page_size (crates/cache/src/paged.rs:40-72,
 * kernels/attention_kernels.metal:377-379 generalised from the identity map).
 * Appends the q_tokens current rows at positions past[b]..past[b]+q_tokens-1, then row t attends to
 * keys [max(0, p+1-window), p] with p = past[b]+t: cached rows as fp16, current-chunk rows in f32,
 * exactly like the ring kernel.  output [batch, q_tokens, q_heads, head_dim]. */
void orc_gqa_paged_attention(const float* query, const float* cur_key, const float* cur_value, const float* gate,
                             uint16_t* k_pool, uint16_t* v_pool, const int32_t* page_table, int max_pages,
                             const int32_t* past_tokens, float* output, int batch, int q_heads, int kv_heads,
                             int head_dim, int page_size, int q_tokens, int sliding_window, int fuse_append,
                             float scale /* <=0: 1/sqrt(head_dim) */, int threads);

/* The same over FP8 E4M3FN pages (kernels/fp8_attention_kernels.metal:70-225 attention, :227-263 append; codec
 * :11-54): pools are uint8 [num_pages][kv_heads][page_size][head_dim], a cached value reads decode(byte) * scale,
 * the current chunk's rows are f32, and the append stores encode(x / scale). */
float orc_fp8_e4m3fn_decode(uint8_t bits);
uint8_t orc_fp8_e4m3fn_encode(float value);
void orc_gqa_paged_attention_fp8(const float* query, const float* cur_key, const float* cur_value, const float* gate,
                                 uint8_t* k_pool, uint8_t* v_pool, float key_scale, float value_scale,
                                 const int32_t* page_table, int max_pages, const int32_t* past_tokens, float* output,
                                 int batch, int q_heads, int kv_heads, int head_dim, int page_size, int q_tokens,
                                 int sliding_window, int fuse_append, float scale, int threads);

/* Gather logical rows back out of the pool: out [batch][kv_heads][tokens][head_dim] (layout_kernels.metal:205-232
 * generalised to a page table). */
void orc_linearize_paged(const uint16_t* pool, const int32_t* page_table, int max_pages, uint16_t* out, int batch,
                         int kv_heads, int tokens, int page_size, int head_dim);

/* ---- a8: MHA decode over the GLM paged layout ----------------------------- */
/* kernels/attention_kernels.metal:339-457: cache [page_count, batch, heads, page_size, dim] fp16, identity
 * page order, one f32 current token. */
void orc_paged_decode_mha_f16(const float* q, const uint16_t* paged_k, const float* cur_k, const uint16_t* paged_v,
                              const float* cur_v, float* output, int batch, int heads, int past_tokens,
                              int page_size, int head_dim, int value_dim);

/* ---- a9: absorbed MLA --------------------------------------------------- */
/* Q8_0 per-head matvec (kernels/q2_kernels.metal:3146; CPU statement metal/q2.rs:8506-8538):
 * weights [heads][out_features][in_features/32] blocks of (f16 scale, 32 x int8). */
void orc_q8_0_heads_matvec(const uint8_t* weights, const float* input /* [rows, heads, in] */,
                           float* output /* [rows, heads, out] */, int64_t rows, int heads, int in_features,
                           int out_features);
/* kernels/attention_kernels.metal:465-603, f32 paged cache with identity pages:
 * paged_latent [pages, batch, page_size, L], paged_rope [pages, batch, page_size, R]. */
void orc_mla_absorbed_f32(const float* q_latent, const float* q_rope, const float* paged_latent,
                          const float* cur_latent, const float* paged_rope, const float* cur_rope, float* out_latent,
                          int batch, int heads, int q_tokens, int past_tokens, int page_size, int latent_dim,
                          int rope_dim, int scale_dim);
/* Extension used by the B200 path: fused fp16 rows [num_pages][page_size][L+R] under a page table; the
 * q_tokens current rows (f32, already post-processed) are appended (RNE) at past..past+T-1 and attended in
 * f32, cached rows in fp16.  q [batch, q_tokens, heads, L+R] = q_latent || q_rope.  out [batch,T,heads,L]. */
void orc_mla_absorbed_paged(const float* q, const float* cur_rows /* [batch,T,L+R] */, uint16_t* pool,
                            const int32_t* page_table, int max_pages, const int32_t* past_tokens, float* out,
                            int batch, int heads, int q_tokens, int page_size, int latent_dim, int rope_dim,
                            float scale, int fuse_append, int threads);

/* ---- selected-row attention over expanded heads (DSA), kernels/attention_kernels.metal:605-721 and :723-968 ----
 * q [B,H,T,D]; sel_k [B,H,S,D], sel_v [B,H,S,Dv]; cur_k [B,H,T,D], cur_v [B,H,T,Dv]; row t sees the S selected rows
 * and, when include_current, current rows 0..t.  out [B,H,T,Dv]. */
void orc_selected_attention_f32(const float* q, const float* sel_k, const float* sel_v, const float* cur_k,
                                const float* cur_v, float* out, int batch, int heads, int S, int T, int D, int Dv,
                                int include_current);

/* ---- a10: causal attention over expanded heads (MLA prefill) ------------- */
/* kernels/attention_kernels.metal:723-968 with zero past (backend.rs:8050-8067); K = [k_nope | shared rope
 * tail] as built by combine_rope_tail (kernels/layout_kernels.metal:148-183, rope_head_count == 1).
 * q [T,H,dn+dr], k_nope [T,H,dn], k_rope [T,dr], v [T,H,dv]; computes the rows listed in `rows`
 * (n_rows of them; NULL = all) into out [n_rows,H,dv]. */
void orc_causal_mha(const float* q, const float* k_nope, const float* k_rope, const float* v, float* out, int tokens,
                    int heads, int nope_dim, int rope_dim, int v_dim, float scale, const int32_t* rows, int n_rows,
                    int threads);

int orc_max_threads(void);
void orc_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif

/* inferno_attn.h -- C ABI of the B200 (sm_100a) attention backend.
 *
 * This is the boundary a `CudaBackend` implementation of the reference's
 * `trait Backend` (crates/backend/src/backend.rs:711) binds over FFI for the attention
 * path: fused RoPE + KV-append, paged GQA decode, causal GQA prefill, absorbed-MLA
 * decode and causal MLA prefill.  Plain pointers and sizes only; every pointer named
 * "device" is a CUDA device pointer on the context's GPU.
 *
 * Conventions
 *   - every op returns int32_t: INF_OK (0), INF_UNSUPPORTED (1, the reference's
 *     `Ok(None)`: "this backend has no device path for these arguments",
 *     backend.rs:1054-1056) or a negative INF_E_* mirroring `common::Error`
 *     (crates/common/src/error.rs:7-52).  inf_last_error() returns the message.
 *   - all shape / length / dtype checks run on the host before any launch, like the
 *     reference's validate_execution (crates/backend/src/metal/f16_attention.rs:602-680);
 *     nothing aborts and no kernel traps.
 *   - ops are enqueued on the context's stream and return without synchronising;
 *     dependent ops need no host sync (the guarantee Metal hazard tracking gives the
 *     reference, crates/backend/src/metal/batch.rs:14-17).  inf_flush() waits.
 *   - there is no CPU fallback: without a CUDA device the context cannot be created.
 *   - a context is used from one thread at a time (the reference serialises through a
 *     mutex around its open command buffer, metal/batch.rs:34-55).
 *
 * KV layout in HBM (generalises crates/cache/src/paged.rs:40-72 and the kernel formula
 * kernels/attention_kernels.metal:377-379 from the identity page map to a page table):
 *   GQA pools   K and V: fp16 [num_pages][kv_heads][page_size][head_dim]
 *   MLA pool    fp16 [num_pages][page_size][latent_dim + rope_dim]   (512 + 64)
 *   page table  int32 [batch][max_pages]: logical token n of sequence b lives in page
 *               page_table[b][n / page_size] at slot n % page_size
 */
#ifndef INFERNO_ATTN_H
#define INFERNO_ATTN_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define INF_OK 0
#define INF_UNSUPPORTED 1
#define INF_E_BACKEND (-1)  /* Error::Backend: CUDA failure, device status word set */
#define INF_E_SHAPE (-2)    /* Error::ShapeMismatch */
#define INF_E_CONFIG (-3)   /* Error::Config */
#define INF_E_CACHE (-4)    /* Error::Cache: page table / capacity problems */
#define INF_E_DTYPE (-5)    /* unsupported dtype */
#define INF_E_ARG (-6)      /* null pointer, bad handle */

#define INF_DTYPE_F32 0
#define INF_DTYPE_F16 1

typedef struct inf_ctx inf_ctx;

/* ---- context, memory, ordering ------------------------------------------------ */
/* MetalBackend::new / from_device (backend.rs:2175-2260).  `stream` is a cudaStream_t to
 * enqueue on, or NULL for a stream owned by the context (pass cudaStreamLegacy, (void*)1, to name
 * the default stream). */
int32_t inf_ctx_create(int32_t device_ordinal, void* stream, inf_ctx** out);
int32_t inf_ctx_destroy(inf_ctx* ctx);
/* Re-target the context at another cudaStream_t (NULL is not accepted; (void*)1 names the default stream).
 * Pending work stays on the old stream.  A caller that captures a decode step into a CUDA graph points the
 * context at its capture stream first; the scratch workspace must already be large enough (run the step
 * once before capturing) because growing it allocates, which a capture forbids.  A graph keeps the workspace
 * address it was captured with: when a later, larger call outgrows the workspace the old buffer is kept alive
 * until inf_ctx_destroy, so the graph stays valid (it then shares nothing with the new buffer). */
int32_t inf_ctx_set_stream(inf_ctx* ctx, void* stream);
const char* inf_last_error(inf_ctx* ctx);
/* device_values_supported (backend.rs:1060). */
int32_t inf_device_values_supported(inf_ctx* ctx);
/* device_flush (backend.rs:1066): wait for the stream, then report the device status word
 * (bounded waits that gave up, page ids out of range) as INF_E_BACKEND. */
int32_t inf_flush(inf_ctx* ctx);
/* device_submit (backend.rs:1072): launches are already asynchronous; checks arguments only. */
int32_t inf_submit(inf_ctx* ctx);
/* Diagnostic for the failure path (no counterpart in the reference).  Every wait inside the kernels is bounded: a
 * load that never arrives makes the waiting warps give up after two seconds, the kernel then runs to its normal end
 * and inf_flush reports "bounded wait gave up" (INF_E_BACKEND); the context stays usable.  This call makes the NEXT
 * inf_gqa_decode_paged* launch of the context lose the loads of tile number `tile` (counted from 0) of its first
 * CTA, so that a test can watch that happen.  The affected output rows are undefined. */
int32_t inf_debug_drop_next_load(inf_ctx* ctx, int32_t tile);
/* device_profile_boundary (backend.rs:1080; GPU time per command buffer, metal/batch.rs:161-170):
 * while enabled, every op records a CUDA event pair around its dominant kernel.  inf_profile_read waits
 * for the stream, returns the summed device time and launch count of the kernel called `kernel_name`
 * since the last read, and forgets them. */
int32_t inf_profile_enable(inf_ctx* ctx, int32_t on);
int32_t inf_profile_read(inf_ctx* ctx, const char* kernel_name, double* total_ms, int32_t* launches);
/* device_alloc_f32/f16_tensor (backend.rs:1098/1104), device_upload_f32_tensor (:1086),
 * device_upload_f32_tensor_as_f16 (:1092), device_copy_same_dtype (:1110),
 * device_download_f32_tensor (:1136). */
int32_t inf_alloc(inf_ctx* ctx, size_t bytes, void** device_out);
int32_t inf_free(inf_ctx* ctx, void* device_ptr);
int32_t inf_upload(inf_ctx* ctx, void* device_dst, const void* host_src, size_t bytes);
int32_t inf_upload_f32_as_f16(inf_ctx* ctx, void* device_dst_f16, const float* host_src, size_t count);
int32_t inf_download(inf_ctx* ctx, void* host_dst, const void* device_src, size_t bytes);
int32_t inf_copy(inf_ctx* ctx, void* device_dst, const void* device_src, size_t bytes);
int32_t inf_memset_zero(inf_ctx* ctx, void* device_dst, size_t bytes);

/* ---- descriptors ---------------------------------------------------------------- */
/* DeviceRopeTable (backend.rs:239-244), built by prepare_rope_table (backend.rs:1227):
 * inverse frequencies for the half-split convention plus the factor multiplied into cos/sin. */
typedef struct inf_rope_table {
    const float* inv_freq; /* device, rotary_dim / 2 entries */
    int32_t rotary_dim;    /* 64 or 128 (metal/rope.rs:472-487) */
    float attention_factor;
} inf_rope_table;
int32_t inf_rope_table_create(inf_ctx* ctx, const float* host_inv_freq, int32_t count, int32_t rotary_dim,
                              float attention_factor, inf_rope_table* out);
int32_t inf_rope_table_destroy(inf_ctx* ctx, inf_rope_table* table);

/* The paged replacement of LagunaF16KvCache (backend.rs:297-314): caller-owned pools. */
typedef struct inf_kv_pool {
    void* k; /* device fp16 [num_pages][kv_heads][page_size][head_dim] */
    void* v;
    int32_t num_pages, page_size, kv_heads, head_dim;
} inf_kv_pool;
/* prepare_laguna_f16_kv_cache (backend.rs:1322): allocates and zero-fills both pools. */
int32_t inf_kv_pool_create(inf_ctx* ctx, int32_t num_pages, int32_t page_size, int32_t kv_heads, int32_t head_dim,
                           inf_kv_pool* out);
int32_t inf_kv_pool_destroy(inf_ctx* ctx, inf_kv_pool* pool);

/* The paged replacement of DevicePagedKvView for the MLA latent layout (backend.rs:543-553;
 * latent in view.k, rope tail in view.v, metal/attention.rs:1147-1155): one fused row. */
typedef struct inf_mla_pool {
    void* rows; /* device fp16 [num_pages][page_size][latent_dim + rope_dim] */
    int32_t num_pages, page_size, latent_dim, rope_dim;
} inf_mla_pool;
int32_t inf_mla_pool_create(inf_ctx* ctx, int32_t num_pages, int32_t page_size, int32_t latent_dim,
                            int32_t rope_dim, inf_mla_pool* out);
int32_t inf_mla_pool_destroy(inf_ctx* ctx, inf_mla_pool* pool);

/* Page table of a batch.  `lens` has the meaning each op states.  The host mirrors are
 * optional: when given, every entry a launch can touch is range-checked on the host first
 * (INF_E_CACHE); kernels additionally refuse out-of-range pages and raise the status word. */
typedef struct inf_page_table {
    const int32_t* pages; /* device int32 [batch][max_pages] */
    const int32_t* lens;  /* device int32 [batch] */
    int32_t batch, max_pages;
    const int32_t* host_pages; /* optional host copy of pages */
    const int32_t* host_lens;  /* optional host copy of lens  */
} inf_page_table;

/* ---- host-side page bookkeeping (no device work) --------------------------------------------- */
/* The logical-token -> (physical page, offset) map of the reference's PagedKvCache
 * (crates/cache/src/paged.rs:40-72: token_location, append_prefill :176, append_decode :185,
 * page_stats :135) for many sequences over one shared pool.  Pages come from a free list; the arrays
 * returned by inf_paged_index_arrays are what a caller uploads as inf_page_table.pages / .lens (and may
 * pass as the host mirrors).  Checkpoint / restore is the paged form of checkpoint_laguna_f16_kv_cache /
 * restore_laguna_f16_kv_cache_checkpoint (backend.rs:1336-1348): pages are immutable once full, so a
 * checkpoint is a remembered length and restoring frees the pages mapped since. */
typedef struct inf_paged_index inf_paged_index;
int32_t inf_paged_index_create(int32_t num_pages, int32_t page_size, int32_t max_seqs, int32_t max_pages_per_seq,
                               inf_paged_index** out);
int32_t inf_paged_index_destroy(inf_paged_index* index);
const char* inf_paged_index_last_error(inf_paged_index* index);
int32_t inf_paged_index_append(inf_paged_index* index, int32_t seq, int32_t tokens, int32_t* start_position,
                               int32_t* allocated_pages);
int32_t inf_paged_index_locate(inf_paged_index* index, int32_t seq, int32_t token, int32_t* page, int32_t* offset);
int32_t inf_paged_index_len(inf_paged_index* index, int32_t seq);
int32_t inf_paged_index_page_count(inf_paged_index* index, int32_t seq);
int32_t inf_paged_index_free_pages(inf_paged_index* index);
int32_t inf_paged_index_release(inf_paged_index* index, int32_t seq);
int32_t inf_paged_index_checkpoint(inf_paged_index* index, int32_t seq);
int32_t inf_paged_index_restore(inf_paged_index* index, int32_t seq);
/* The sliding-window ring on pages (reference: a sliding layer's cache is 512 slots, slot = position % capacity,
 * crates/backend/src/metal/f16_attention.rs:120-210; 36 of 48 Laguna layers are sliding).  Pages that lie wholly
 * below first_visible -- the lowest row any future query of the sequence can see, i.e. next position + 1 - window --
 * go back to the free list; logical positions stay, the released page-table slots read -1, and the attention kernels
 * never resolve a page below the window.  A checkpoint older than first_visible forbids the trim (INF_E_CACHE).
 * released_pages (optional) receives the number of pages returned. */
int32_t inf_paged_index_trim(inf_paged_index* index, int32_t seq, int32_t first_visible, int32_t* released_pages);
int32_t inf_paged_index_arrays(inf_paged_index* index, const int32_t** pages, const int32_t** lens,
                               int32_t* max_seqs, int32_t* max_pages);

/* ---- RoPE and KV append ----------------------------------------------------------- */
/* qk_rms_norm_rope_device (backend.rs:1238; kernel qk_rms_norm_half_split_rope_f32_kernel, rope_kernels.metal:113):
 * per-head RMSNorm (weight NULL = no norm) then half-split RoPE of one tensor [batch, tokens, heads, head_dim],
 * f32 in / f32 out; position of a row = position_offset + its token index. */
int32_t inf_qk_rms_norm_rope(inf_ctx* ctx, const float* input, const float* norm_weight, float eps,
                             int32_t position_offset, const inf_rope_table* rope, int32_t batch, int32_t tokens,
                             int32_t heads, int32_t head_dim, float* output);

/* laguna_qk_rms_norm_rope_pair_device (backend.rs:1252; kernel rope_kernels.metal:167):
 * per-head RMSNorm (weight NULL = no norm) then half-split RoPE, f32 in / f32 out.
 * q [batch, tokens, q_heads, head_dim], k [batch, tokens, kv_heads, head_dim]. */
int32_t inf_laguna_qk_rms_norm_rope_pair(inf_ctx* ctx, const float* q, const float* k, const float* q_norm_weight,
                                         const float* k_norm_weight, float eps, int32_t position_offset,
                                         const inf_rope_table* rope, int32_t batch, int32_t tokens, int32_t q_heads,
                                         int32_t kv_heads, int32_t head_dim, float* q_out, float* k_out);

/* Fused RoPE + KV-append: the rope kernel above fused with the cache append of
 * f16_attention_kernels.metal:131-143 / :512-544.  Row t of sequence b sits at position
 * lens[b] + t (lens = tokens already cached).  q/k/v are device f32 or fp16 (in_dtype);
 * q_out receives the roped queries as fp16 [batch, tokens, q_heads, head_dim] (the layout
 * the attention kernels read); K (roped) and V are written RNE-fp16 into their pages.
 * k_roped_f32_out is optional (NULL): the roped keys in f32, as the reference returns them. */
int32_t inf_rope_append_gqa(inf_ctx* ctx, const void* q, const void* k, const void* v, int32_t in_dtype,
                            const float* q_norm_weight, const float* k_norm_weight, float eps,
                            const inf_rope_table* rope, const inf_kv_pool* pool, const inf_page_table* table,
                            int32_t tokens, int32_t q_heads, void* q_out_f16, float* k_roped_f32_out);

/* rope_slice_device (backend.rs:1866; kernel rope_kernels.metal:5): GLM interleaved-pair RoPE,
 * f32 [batch, tokens, heads, rope_dim]. */
int32_t inf_rope_slice(inf_ctx* ctx, const float* input, float* output, int32_t batch, int32_t tokens, int32_t heads,
                       int32_t rope_dim, int32_t position_offset, float theta);

/* mla_kv_postprocess_device (backend.rs:1895; kernel norm_kernels.metal:52) fused with the append
 * the reference does by downloading rows and blitting them into the paged window
 * (crates/runtime/src/lib.rs:3696-3795, 4963-5045).  input f32 [batch, tokens, latent+rope];
 * row t of sequence b is post-processed at position lens[b] + t and stored RNE-fp16 at that
 * logical slot.  latent_out / rope_out (f32, optional) are the reference's two outputs. */
int32_t inf_mla_kv_postprocess_append(inf_ctx* ctx, const float* input, const float* norm_weight, float eps,
                                      float theta, const inf_mla_pool* pool, const inf_page_table* table,
                                      int32_t tokens, float* latent_out, float* rope_out);

/* ---- attention ---------------------------------------------------------------------- */
/* Paged GQA decode, split-KV (kernels f16_attention_kernels.metal:325-510, generalised to pages):
 * q fp16 [batch, q_heads, head_dim]; lens[b] = visible keys including the current token, which
 * has already been appended.  sliding_window 0 = full.  gate (f32 [batch, q_heads], optional)
 * applies softplus(gate) like the reference.  scale <= 0 means 1/sqrt(head_dim).
 * max_len >= max(lens) sizes the grid; split_chunk keys per partial (multiple of 64).
 * out: [batch, q_heads, head_dim] in out_dtype. */
int32_t inf_gqa_decode_paged(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                             int32_t q_heads, int32_t max_len, int32_t split_chunk, int32_t sliding_window,
                             const float* gate, float scale, void* out, int32_t out_dtype);
/* Bytes of scratch inf_gqa_decode_paged needs for these sizes (the context grows its own). */
size_t inf_gqa_decode_workspace_bytes(int32_t batch, int32_t q_heads, int32_t head_dim, int32_t max_len,
                                      int32_t split_chunk);

/* inf_gqa_decode_paged for callers that must not allocate.  (No counterpart in the reference: its
 * arena hands out a fresh partial buffer per call, crates/backend/src/metal/f16_attention.rs:471-478.)
 *
 * inf_gqa_decode_paged keeps the split-KV partials in a workspace that it grows with cudaMalloc when a
 * call is larger than any before it.  A server that has given all free HBM to its KV pool, a decode
 * loop that cannot take the device-wide stall inside cudaMalloc/cudaFree, or a host whose device memory
 * is owned by another allocator can call this variant instead: same arguments, same result, but the
 * partials live in an array of INF_GQA_DECODE_STATIC_SCRATCH_BYTES that is part of the library image
 * (every GPU that loads the library holds it until the process exits), and the call performs no
 * cudaMalloc, cudaFree or other device allocation.
 *
 *   - sizes whose partials (inf_gqa_decode_workspace_bytes) exceed the array are refused with
 *     INF_E_CONFIG and a message naming both numbers; nothing is launched.
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call during set-up, before any stream capture.
 *   - all calls, on every stream and context of the process, share the one array per GPU and it keeps
 *     the previous call's contents (nothing in it needs clearing: each call overwrites what it reads).
 *     Two calls that overlap on the same GPU race on it; keep them on one stream or order them. */
#define INF_GQA_DECODE_STATIC_SCRATCH_BYTES (32u << 20)
int32_t inf_gqa_decode_paged_static(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                    const inf_page_table* table, int32_t q_heads, int32_t max_len,
                                    int32_t split_chunk, int32_t sliding_window, const float* gate, float scale,
                                    void* out, int32_t out_dtype);

/* Causal GQA prefill over pages (kernel f16_attention_kernels.metal:153-316, generalised):
 * q fp16 [batch, tokens, q_heads, head_dim]; lens[b] = keys cached BEFORE this chunk; the chunk's
 * K/V have already been appended at lens[b]..lens[b]+tokens-1.  Row t sees keys
 * [max(0, p+1-window), p], p = lens[b] + t.  out [batch, tokens, q_heads, head_dim]. */
int32_t inf_gqa_prefill_paged(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool, const inf_page_table* table,
                              int32_t tokens, int32_t q_heads, int32_t sliding_window, const float* gate, float scale,
                              void* out, int32_t out_dtype);

/* laguna_gated_gqa_f16_attention_device (backend.rs:1350) as one call: f32 q/k/v (already roped),
 * f32 gate, append then attend.  lens[b] = tokens cached before the call; the caller advances its
 * host counters afterwards, like commit_append (backend.rs:5400).  max_len >= max(lens) + tokens. */
int32_t inf_laguna_gated_gqa_f16_attention(inf_ctx* ctx, const float* q, const float* k, const float* v,
                                           const float* gate, const inf_kv_pool* pool, const inf_page_table* table,
                                           int32_t tokens, int32_t q_heads, int32_t max_len, int32_t sliding_window,
                                           float* out);

/* Absorbed-MLA decode (kernel attention_kernels.metal:465-603; q8_0_absorbed_mla_device backend.rs:1982
 * without its K_b / V_b projections): q fp16 [batch, tokens, heads, latent+rope] = q_latent || q_rope;
 * lens[b] = cached rows BEFORE this call's `tokens` rows, which have already been appended; row t sees
 * rows 0..lens[b]+t.  scale = 1/sqrt(scale_dim).  out [batch, tokens, heads, latent_dim]. */
int32_t inf_mla_decode_absorbed(inf_ctx* ctx, const void* q_f16, const inf_mla_pool* pool,
                                const inf_page_table* table, int32_t tokens, int32_t heads, int32_t max_len,
                                float scale, void* out, int32_t out_dtype);

/* Absorbed-MLA decode over SELECTED cached rows: the attention step of the reference's DSA sparse decode
 * (crates/model/src/attention.rs:2843-2960: the rows chosen by the indexer are copied into a compact cache by
 * selected_kv_for_tokens and attended to with the current token; the expanded-head form of the same step is
 * selected_decode_attention_device, backend.rs:1999, kernel attention_kernels.metal:605).  Here the gather is
 * part of the kernel: selected[b][i], i < selected_counts[b] <= selected_stride, are logical row ids of sequence
 * b (each < lens[b] + 1, the current token's row included by listing it; order free, no duplicates expected);
 * the softmax runs over exactly those rows.  One query token per sequence: q fp16 [batch, 1, heads, 576],
 * out [batch, 1, heads, 512].  Ids outside the visible rows set the context's error status (inf_flush). */
int32_t inf_mla_decode_absorbed_selected(inf_ctx* ctx, const void* q_f16, const inf_mla_pool* pool,
                                         const inf_page_table* table, const int32_t* selected,
                                         const int32_t* selected_counts, int32_t selected_stride, int32_t heads,
                                         float scale, void* out, int32_t out_dtype);

/* The expanded-head forms of the selected-row attention (f32 at the boundary, heads-major layouts as the reference's).
 * inf_selected_decode_attention: selected_decode_attention_device (backend.rs:2001, 7814; kernel
 *   fused_selected_decode_attention_f32_kernel, kernels/attention_kernels.metal:605-721, and its f16-KV twin): q
 *   [batch, heads, 1, head_dim], selected_k [batch, heads, selected_tokens, head_dim], selected_v [.., value_dim] in
 *   selected_dtype (INF_DTYPE_F32 or INF_DTYPE_F16), current_k / current_v f32 [batch, heads, 1, dim]; the softmax
 *   runs over the selected rows plus, when include_current_kv, the current token; scale 1/sqrt(head_dim); out
 *   [batch, heads, 1, value_dim].  selected_tokens == 0 is INF_E_BACKEND like the reference.
 * inf_selected_sequence_attention: selected_sequence_attention_device (backend.rs:2015, 7930; kernel
 *   fused_selected_sequence_attention_f32_kernel, :723-968): causal attention of query_tokens rows (a speculative
 *   batch, or a first prompt chunk with past_tokens == 0) over past_k / past_v [batch, heads, past_tokens, dim] plus
 *   current rows 0..t; all f32; out [batch, heads, query_tokens, value_dim].
 * More than 4096 visible keys (the reference kernel's limit) or dims above 256 return INF_UNSUPPORTED. */
int32_t inf_selected_decode_attention(inf_ctx* ctx, const float* q, const void* selected_k, const void* selected_v,
                                      int32_t selected_dtype, const float* current_k, const float* current_v,
                                      int32_t batch, int32_t heads, int32_t selected_tokens, int32_t head_dim,
                                      int32_t value_dim, int32_t include_current_kv, float* out);
int32_t inf_selected_sequence_attention(inf_ctx* ctx, const float* q, const float* past_k, const float* past_v,
                                        const float* current_k, const float* current_v, int32_t batch, int32_t heads,
                                        int32_t past_tokens, int32_t query_tokens, int32_t head_dim, int32_t value_dim,
                                        float* out);

/* DSA indexer, the step before inf_mla_decode_absorbed_selected.
 * inf_dsa_scores (kernel dsa_scores_f32_kernel, crates/backend/src/metal/kernels/dsa_kernels.metal:137-176):
 * q f32 [batch, heads, head_dim] (already roped), weights f32 [batch, heads], past_keys f32 [batch, past_tokens,
 * head_dim], current_key f32 [batch, head_dim]; scores f32 [batch, past_tokens + 1],
 * score[t] = sum_h weights[h] * max(0, q[h] . key[t] / sqrt(head_dim)).  head_dim % 4 == 0.  fp32 accumulation;
 * for head_dim 128 and heads a multiple of 16 the dot products run on the tensor cores with every input split into
 * two tf32 terms, which keeps a score within 2e-5 of exact arithmetic (the fp32 sum's own rounding).
 * inf_dsa_topk (kernels dsa_topk_block_sort_u32 / dsa_topk_merge_u32, dsa_kernels.metal:211-393): the top_k
 * (<= 2048) token ids of every row of scores [batch, key_tokens], best first, where a precedes b iff
 * score_a > score_b or (score_a == score_b and id_a < id_b); selected uint32 [batch, selected_stride], entries
 * beyond min(top_k, key_tokens) are 0xffffffff.  Scores are expected to be free of NaN. */
int32_t inf_dsa_scores(inf_ctx* ctx, const float* q, const float* weights, const float* past_keys,
                       const float* current_key, int32_t batch, int32_t past_tokens, int32_t heads, int32_t head_dim,
                       float* scores);
int32_t inf_dsa_topk(inf_ctx* ctx, const float* scores, int32_t batch, int32_t key_tokens, int32_t top_k,
                     uint32_t* selected, int32_t selected_stride);

/* DSA indexer preparation (trait methods dsa_index_key_device, backend.rs:2061, and the first half of
 * dsa_decode_topk_device, backend.rs:2074; CPU semantics crates/model/src/indexer.rs:174-203, :397-428, :483-543;
 * Metal kernels dsa_kernels.metal:23-135).  Device pointers, f32.
 *   inf_dsa_index_key: raw_key [batch][tokens][head_dim] -> LayerNorm (weight, bias [head_dim], eps; the reference
 *     uses 1e-6) -> rotary encoding of the first rope_dim values at position position_offset + token with
 *     freq(pair) = 1 / theta^(2 pair / rope_dim): interleaved pairs (2p, 2p+1) in, halves out (p and rope_dim/2 + p).
 *   inf_dsa_query_weights: weights_out [batch][heads] = hidden_states [batch][hidden_size] . weights_proj
 *     [hidden_size][heads] / sqrt(heads); q_out [batch][heads][head_dim] = q_raw under the same rotation at
 *     position_offset.  Their outputs feed inf_dsa_scores.
 * An odd rope_dim or one larger than head_dim is INF_E_CONFIG with the reference's message. */
int32_t inf_dsa_index_key(inf_ctx* ctx, const float* raw_key, const float* weight, const float* bias, int32_t batch,
                          int32_t tokens, int32_t head_dim, int32_t rope_dim, int32_t position_offset, float theta,
                          float eps, float* out);
int32_t inf_dsa_query_weights(inf_ctx* ctx, const float* hidden_states, const float* q_raw, const float* weights_proj,
                              int32_t batch, int32_t hidden_size, int32_t heads, int32_t head_dim, int32_t rope_dim,
                              int32_t position_offset, float theta, float* q_out, float* weights_out);

/* FP8 E4M3FN KV pages: the paged replacement of LagunaFp8KvCache (prepare_laguna_fp8_kv_cache, crates/backend/src/
 * metal/fp8_attention.rs; kernels fp8_attention_kernels.metal:70-263).  Same geometry as inf_kv_pool with one byte
 * per value: stored byte = encode(x / scale), read value = decode(byte) * scale, one scale per tensor.  Pools hold
 * encoder output only: the two NaN codes 0x7f / 0xff (which the encoder never writes and the scalar decode maps to
 * zero) are not looked for by the attention kernel. */
typedef struct inf_kv_pool_fp8 {
    void* k; /* device uint8 [num_pages][kv_heads][page_size][head_dim] */
    void* v;
    int32_t num_pages, page_size, kv_heads, head_dim;
    float key_scale, value_scale;
} inf_kv_pool_fp8;
int32_t inf_kv_pool_fp8_create(inf_ctx* ctx, int32_t num_pages, int32_t page_size, int32_t kv_heads, int32_t head_dim,
                               float key_scale, float value_scale, inf_kv_pool_fp8* out);
int32_t inf_kv_pool_fp8_destroy(inf_ctx* ctx, inf_kv_pool_fp8* pool);

/* inf_rope_append_gqa for FP8 pages (append kernel fp8_attention_kernels.metal:227-263 fused with the RoPE): the
 * roped keys and the values of the call's tokens are stored as encode(x / scale).  Attention reads the current
 * tokens at full precision, not through the cache (fp8_attention_kernels.metal:155-163), so the same rows are
 * also written as fp16 to cur_k_out_f16 / cur_v_out_f16 [batch, tokens, kv_heads, head_dim] (either may be NULL). */
int32_t inf_rope_append_gqa_fp8(inf_ctx* ctx, const void* q, const void* k, const void* v, int32_t in_dtype,
                                const float* q_norm_weight, const float* k_norm_weight, float eps,
                                const inf_rope_table* rope, const inf_kv_pool_fp8* pool, const inf_page_table* table,
                                int32_t tokens, int32_t q_heads, void* q_out_f16, void* cur_k_out_f16,
                                void* cur_v_out_f16);

/* Paged GQA decode over FP8 pages, split-KV: laguna_gated_gqa_fp8_attention_f32_kernel (fp8_attention_kernels.metal:
 * 70-225) for one query token per sequence, generalised to a page table.  lens[b] = rows cached BEFORE the current
 * token; those are read as decode(byte) * scale.  The current token's key (roped) and value are given as fp16
 * [batch, kv_heads, head_dim] and enter the softmax at full precision, as in the reference; whether its FP8 copy
 * has already been appended at slot lens[b] does not matter.  Window, gate, scale, max_len (>= max(lens) + 1),
 * split_chunk and out as inf_gqa_decode_paged.  Halves the bytes a decode step moves. */
int32_t inf_gqa_decode_paged_fp8(inf_ctx* ctx, const void* q_f16, const void* cur_k_f16, const void* cur_v_f16,
                                 const inf_kv_pool_fp8* pool, const inf_page_table* table, int32_t q_heads,
                                 int32_t max_len, int32_t split_chunk, int32_t sliding_window, const float* gate,
                                 float scale, void* out, int32_t out_dtype);

/* FP8 E4M3FN codec of the Laguna safetensors cache (crates/backend/src/metal/kernels/
 * fp8_attention_kernels.metal:11-54 codec, :227-263 append): stored byte = encode(x / scale), read value =
 * decode(byte) * scale, one scale per tensor.  Encode saturates at +-448, maps NaN and 0 to 0x00, rounds ties to
 * even, and below 2^-6 stores multiples of 2^-9; decode maps the two NaN codes to 0.  count values, device
 * pointers.  inf_kv_pool_from_fp8 dequantises whole FP8 K and V page arrays (same geometry as the pool,
 * [num_pages][kv_heads][page_size][head_dim] bytes) into an fp16 pool (what a prefill over an FP8 cache with
 * history reads: it is tensor-bound, so the byte count of its K/V does not set its time). */
int32_t inf_fp8_e4m3fn_encode(inf_ctx* ctx, const float* input, int64_t count, float scale, void* output);
int32_t inf_fp8_e4m3fn_decode(inf_ctx* ctx, const void* input, int64_t count, float scale, float* output);
int32_t inf_kv_pool_from_fp8(inf_ctx* ctx, const void* k_fp8, const void* v_fp8, float key_scale, float value_scale,
                             const inf_kv_pool* pool);

/* Q8Row cold-store codec (crates/cache/src/cold_kv.rs:1624-1703; device decode kernel q8_rows_to_f32_kernel,
 * crates/backend/src/metal/kernels/cast_kernels.metal:31-56).  A row of `dim` values is 4 + dim bytes: the
 * little-endian f32 scale max|x| / 127 (1.0 for an all-zero row), then round(x / scale) as signed bytes clamped to
 * +-127 (ties away from zero).  payload and input / output are device pointers; rows = batch * heads * tokens. */
int32_t inf_q8_rows_encode(inf_ctx* ctx, const float* input, int64_t rows, int32_t dim, void* payload);
int32_t inf_q8_rows_decode(inf_ctx* ctx, const void* payload, int64_t rows, int32_t dim, float* output);
/* Thaw of cold MLA rows into the paged pool (dequantise on load): latent_payload holds batch * tokens Q8Row rows
 * of width pool->latent_dim, rope_payload as many of width pool->rope_dim (the reference keeps the latent and the
 * rope tail as the K and V records of a page); row (b, t) is stored RNE-fp16 at logical slot first_token + t of
 * sequence b.  table->lens is not read; the caller sets the lengths when the range is resident again. */
int32_t inf_mla_pool_thaw_q8_rows(inf_ctx* ctx, const void* latent_payload, const void* rope_payload,
                                  const inf_mla_pool* pool, const inf_page_table* table, int32_t first_token,
                                  int32_t tokens);

/* Per-head Q8_0 matvec (kernel q8_0_packed_heads_matvec_f32_kernel, crates/backend/src/metal/kernels/
 * q2_kernels.metal:3146; host crates/backend/src/metal/q2.rs:2656): weights (device) [heads][out_features]
 * [in_features] in Q8_0 row blocks of 34 bytes (little-endian f16 scale, 32 signed quants); input f32
 * [rows, heads, in_features]; output f32 [rows, heads, out_features].  in_features % 32 == 0. */
int32_t inf_q8_0_packed_heads_matvec(inf_ctx* ctx, const void* weights, const float* input, int32_t rows,
                                     int32_t heads, int32_t in_features, int32_t out_features, float* output);

/* q8_0_absorbed_mla_device (backend.rs:1982, 7695; driver crates/backend/src/metal/device.rs:3501-3585) as one
 * call: q_latent = K_b . q_no_rope, absorbed MLA attention over the paged cache, out = V_b . context.
 * k_b_weights / v_b_weights: device copies of the Q8_0 bytes, [heads][latent][q_no_rope_dim] and
 * [heads][value_dim][latent].  q_no_rope f32 [batch, tokens, heads, q_no_rope_dim], q_rope f32 [batch, tokens,
 * heads, rope].  current_latent f32 [batch, tokens, latent] and current_rope f32 [batch, tokens, rope] are the
 * already post-processed rows of this call's tokens: when given they are stored RNE-fp16 at slots
 * lens[b] .. lens[b]+tokens-1 first; pass both null when inf_mla_kv_postprocess_append has stored them.
 * lens[b] = rows cached before the call; row t sees rows 0 .. lens[b]+t; score scale 1/sqrt(qk_head_dim),
 * qk_head_dim = q_no_rope_dim + rope (checked, as backend.rs:7767).  out f32 [batch, tokens, heads, value_dim]. */
int32_t inf_q8_0_absorbed_mla(inf_ctx* ctx, const void* k_b_weights, const void* v_b_weights, const float* q_no_rope,
                              const float* q_rope, const float* current_latent, const float* current_rope,
                              const inf_mla_pool* pool, const inf_page_table* table, int32_t tokens, int32_t heads,
                              int32_t q_no_rope_dim, int32_t value_dim, int32_t qk_head_dim, int32_t max_len,
                              float* out);

/* Causal attention over expanded heads = the reference's MLA prefill
 * (causal_sequence_attention_device backend.rs:2028; kernel attention_kernels.metal:723).
 * fp16 tensors with element strides: q [tokens][heads][nope+rope], k_nope [tokens][heads][nope],
 * k_rope [tokens][rope] shared by all heads (layout_kernels.metal:166-182), v [tokens][heads][v_dim].
 * *_ts / *_hs are token and head strides in elements (innermost stride 1). */
int32_t inf_mla_prefill_causal(inf_ctx* ctx, const void* q, int64_t q_ts, int64_t q_hs, const void* k_nope,
                               int64_t kn_ts, int64_t kn_hs, const void* k_rope, int64_t kr_ts, const void* v,
                               int64_t v_ts, int64_t v_hs, int32_t tokens, int32_t heads, int32_t nope_dim,
                               int32_t rope_dim, int32_t v_dim, float scale, void* out, int64_t o_ts, int64_t o_hs,
                               int32_t out_dtype);

/* paged_decode_attention_resident_device (backend.rs:1966; kernel attention_kernels.metal:339-457): MHA decode
 * over the GLM expanded layout, fp16 cache [page_count][batch][heads][page_size][dim] in identity page
 * order (page = key / page_size), plus one current token given in f32.  q, cur_k [batch, heads, head_dim],
 * cur_v [batch, heads, value_dim]; out f32 [batch, heads, value_dim].  head_dim and value_dim are
 * multiples of 32 up to 256.  Scale is 1/sqrt(head_dim). */
int32_t inf_paged_decode_attention_resident(inf_ctx* ctx, const float* q, const void* paged_k_f16, const float* cur_k,
                                            const void* paged_v_f16, const float* cur_v, int32_t batch, int32_t heads,
                                            int32_t past_tokens, int32_t page_size, int32_t head_dim,
                                            int32_t value_dim, float* out);

/* paged_kv_contiguous_device (backend.rs:2040; kernel layout_kernels.metal:205): gather logical rows
 * of one pool out of its pages: out fp16 [batch][kv_heads][tokens][head_dim]. */
int32_t inf_linearize_paged(inf_ctx* ctx, const void* pool_f16, const inf_kv_pool* shape,
                            const inf_page_table* table, int32_t tokens, void* out_f16);

/* ---- multi-GPU: the one collective of the path ------------------------------------------------------ */
/* Head-sharded prefill / MLA leaves every rank with [tokens, heads/N, dim]; the output is all-gathered over
 * NCCL (NVLink / NVSwitch) on the context's stream.  (The reference is single-device; no counterpart.)
 * NCCL is loaded at run time (libnccl.so.2, or the path in INFERNO_NCCL_LIB).  Rank 0 creates the id and the
 * host hands its INF_COMM_ID_BYTES bytes to the other ranks by any means; every rank then calls inf_comm_init
 * with its own context.  recv holds nranks * bytes, in rank order. */
#define INF_COMM_ID_BYTES 128
typedef struct inf_comm inf_comm;
int32_t inf_comm_unique_id(inf_ctx* ctx, void* id_out);
int32_t inf_comm_init(inf_ctx* ctx, const void* id, int32_t rank, int32_t nranks, inf_comm** out);
int32_t inf_comm_destroy(inf_comm* comm);
int32_t inf_allgather_heads(inf_comm* comm, const void* send, void* recv, size_t bytes);

/* The all-gather fused into the prefill kernels.  Every rank holds its own copy of the gathered tensor
 * [tokens][all heads][dim]; a rank's kernel stores each finished output tile into its own copy and, with plain
 * stores over NVLink, into the other ranks' copies, so the exchange rides under the attention tile by tile and no
 * collective follows the kernel -- only inf_comm_barrier, after which every rank's copy is complete.  A consumer
 * must not let the next call overwrite a copy a peer may still be reading: alternate two gathered tensors, or put
 * a barrier before the call as well.  (No counterpart in the reference.)
 *   inf_peer_export: INF_PEER_HANDLE_BYTES describing `device_ptr` (any pointer inside a cudaMalloc allocation of this
 *     process) for another process of the same box; the host carries the bytes to the peers by any means.
 *   inf_peer_open / inf_peer_close: map / unmap a peer's export into this process (cudaIpcOpenMemHandle).
 *   inf_comm_barrier: stream-ordered barrier over the communicator's ranks: one small kernel per rank that writes an
 *     arrival flag into every peer's flag array over NVLink and waits, with a time limit, for theirs (the arrays are
 *     exchanged and mapped at inf_comm_init; if that is not possible, a four-byte NCCL all-reduce instead).
 *   inf_mla_prefill_causal_peers / inf_gqa_prefill_paged_peers: the prefill entry points with up to INF_MAX_PEERS
 *     peer outputs; `out` and every peer pointer already point at this rank's first head inside a gathered tensor
 *     whose token stride is o_ts (out_token_stride) elements.
 *   inf_gqa_decode_paged_peers: inf_gqa_decode_paged for a batch sharded by sequence; `out` and every peer pointer
 *     point at this rank's first sequence inside a gathered [all sequences][q_heads][128] output, and the combine
 *     kernel stores each output row into all of them. */
#define INF_MAX_PEERS 7
#define INF_PEER_HANDLE_BYTES 72
int32_t inf_peer_export(inf_ctx* ctx, const void* device_ptr, void* handle_out);
int32_t inf_peer_open(inf_ctx* ctx, const void* handle, void** peer_ptr);
int32_t inf_peer_close(inf_ctx* ctx, void* peer_ptr, const void* handle);
int32_t inf_comm_barrier(inf_comm* comm);
/* 1 when inf_comm_barrier is the peer-flag kernel (every rank could map every other rank's flag array at
 * inf_comm_init), 0 when it falls back to the NCCL all-reduce. */
int32_t inf_comm_barrier_is_p2p(inf_comm* comm);
int32_t inf_mla_prefill_causal_peers(inf_ctx* ctx, const void* q, int64_t q_ts, int64_t q_hs, const void* k_nope,
                                     int64_t kn_ts, int64_t kn_hs, const void* k_rope, int64_t kr_ts, const void* v,
                                     int64_t v_ts, int64_t v_hs, int32_t tokens, int32_t heads, int32_t nope_dim,
                                     int32_t rope_dim, int32_t v_dim, float scale, void* out, int64_t o_ts, int64_t o_hs,
                                     int32_t out_dtype, void* const* peer_outs, int32_t n_peers);
int32_t inf_gqa_prefill_paged_peers(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                    const inf_page_table* table, int32_t tokens, int32_t q_heads, int32_t sliding_window,
                                    const float* gate, float scale, void* out, int32_t out_dtype,
                                    int64_t out_token_stride, void* const* peer_outs, int32_t n_peers);
int32_t inf_gqa_decode_paged_peers(inf_ctx* ctx, const void* q_f16, const inf_kv_pool* pool,
                                   const inf_page_table* table, int32_t q_heads, int32_t max_len, int32_t split_chunk,
                                   int32_t sliding_window, const float* gate, float scale, void* out,
                                   int32_t out_dtype, void* const* peer_outs, int32_t n_peers);

#ifdef __cplusplus
}
#endif
#endif

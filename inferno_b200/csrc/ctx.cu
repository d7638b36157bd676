// Context, memory and ordering entry points of the C ABI, plus pool / rope-table helpers.
#include <cuda_fp16.h>
#include <math.h>
#include <string.h>

#include "common.cuh"

int inf_fail(inf_ctx* ctx, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) ctx->err = buf;
    return code;
}

int inf_ensure_workspace(inf_ctx* ctx, size_t bytes) {
    if (bytes <= ctx->workspace_bytes) return INF_OK;
    // A CUDA graph captured earlier keeps the address it was captured with, so an outgrown workspace is retired,
    // not freed: it lives until the context is destroyed.  Growth is by at least a factor of two, which bounds
    // the retired buffers by the size of the live one.
    size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    if (want < 2 * ctx->workspace_bytes) want = 2 * ctx->workspace_bytes;
    void* fresh = nullptr;
    INF_CUDA(ctx, cudaMalloc(&fresh, want));
    if (ctx->workspace) ctx->retired_workspaces.push_back(ctx->workspace);
    ctx->workspace = fresh;
    ctx->workspace_bytes = want;
    return INF_OK;
}

int inf_make_tmap(inf_ctx* ctx, const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides_bytes,
                  const uint32_t* box, CUtensorMap* out) {
    return inf_make_tmap_typed(ctx, base, rank, dims, strides_bytes, box, out, 2);
}

int inf_make_tmap_typed(inf_ctx* ctx, const void* base, uint32_t rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box, CUtensorMap* out, uint32_t elem_bytes) {
    inf_tmap_key key{};
    key.base = base;
    key.rank = rank | (elem_bytes << 8);  // the element size is part of the identity of a cached descriptor
    for (uint32_t i = 0; i < rank; ++i) {
        key.dims[i] = dims[i];
        key.box[i] = box[i];
        if (i + 1 < rank) key.strides[i] = strides_bytes[i];
    }
    for (auto& kv : ctx->tmaps)
        if (kv.first == key) {
            *out = kv.second;
            return INF_OK;
        }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
        return inf_fail(ctx, INF_E_ARG, "tensor base %p is not 16-byte aligned", base);
    for (uint32_t i = 0; i + 1 < rank; ++i)
        if (strides_bytes[i] % 16 != 0)
            return inf_fail(ctx, INF_E_SHAPE, "tensor stride %llu bytes is not a multiple of 16",
                            (unsigned long long)strides_bytes[i]);
    cuuint64_t gdim[3] = {1, 1, 1};
    cuuint64_t gstr[2] = {0, 0};
    cuuint32_t bx[3] = {1, 1, 1}, es[3] = {1, 1, 1};
    for (uint32_t i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        if (i + 1 < rank) gstr[i] = strides_bytes[i];
    }
    CUtensorMap tm;
    const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = ctx->encode(&tm, dt, rank, const_cast<void*>(base), gdim, gstr, bx, es,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return inf_fail(ctx, INF_E_BACKEND, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (ctx->tmaps.size() >= 64) ctx->tmaps.erase(ctx->tmaps.begin());
    ctx->tmaps.emplace_back(key, tm);
    *out = tm;
    return INF_OK;
}

int inf_validate_table(inf_ctx* ctx, const inf_page_table* t, int num_pages, int page_size, int extra_tokens,
                       const char* what, int window, int query_tokens, bool append_only) {
    if (!t || !t->pages || !t->lens) return inf_fail(ctx, INF_E_ARG, "%s: null page table", what);
    if (t->batch <= 0 || t->max_pages <= 0)
        return inf_fail(ctx, INF_E_SHAPE, "%s: batch %d / max_pages %d must be positive", what, t->batch, t->max_pages);
    if (!t->host_lens) return INF_OK;
    for (int b = 0; b < t->batch; ++b) {
        long long len = (long long)t->host_lens[b] + extra_tokens;
        if (t->host_lens[b] < 0 || len > (long long)t->max_pages * page_size)
            return inf_fail(ctx, INF_E_CACHE, "%s: sequence %d length %lld exceeds page-table capacity %lld", what, b,
                            len, (long long)t->max_pages * page_size);
        if (!t->host_pages) continue;
        int used = (int)((len + page_size - 1) / page_size);
        // with a sliding window the pages wholly below the first query row's lowest visible key are never read and
        // may have been returned to the pool (inf_paged_index_trim): their slots are not checked; an append only
        // touches the pages of its own tokens
        long long lowest = append_only ? t->host_lens[b] : (window > 0 ? len - query_tokens + 1 - window : 0);
        int first = lowest > 0 ? (int)(lowest / page_size) : 0;
        for (int p = first; p < used; ++p) {
            int id = t->host_pages[(size_t)b * t->max_pages + p];
            if (id < 0 || id >= num_pages)
                return inf_fail(ctx, INF_E_CACHE, "%s: sequence %d page slot %d holds page id %d outside [0,%d)", what,
                                b, p, id, num_pages);
        }
    }
    return INF_OK;
}

extern "C" {

int32_t inf_ctx_create(int32_t device_ordinal, void* stream, inf_ctx** out) {
    if (!out) return INF_E_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0 || device_ordinal < 0 || device_ordinal >= count) return INF_E_BACKEND;
    inf_ctx* ctx = new inf_ctx();
    ctx->device = device_ordinal;
    if (cudaSetDevice(device_ordinal) != cudaSuccess) {
        delete ctx;
        return INF_E_BACKEND;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess || prop.major != 10) {
        delete ctx;  // kernels are sm_100a only
        return INF_E_BACKEND;
    }
    ctx->sm_count = prop.multiProcessorCount;
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return INF_E_BACKEND;
        }
        ctx->own_stream = true;
    }
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
        delete ctx;
        return INF_E_BACKEND;
    }
    ctx->encode = (inf_tmap_encode_fn)fn;
    if (cudaMalloc(&ctx->status, 16) != cudaSuccess || cudaMemset(ctx->status, 0, 16) != cudaSuccess ||
        cudaMallocHost(&ctx->host_status, 16) != cudaSuccess) {
        delete ctx;
        return INF_E_BACKEND;
    }
    *out = ctx;
    return INF_OK;
}

int32_t inf_ctx_destroy(inf_ctx* ctx) {
    INF_CHECK_CTX(ctx);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& r : ctx->prof) {
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    if (ctx->workspace) cudaFree(ctx->workspace);
    for (void* w : ctx->retired_workspaces) cudaFree(w);
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->host_status) cudaFreeHost(ctx->host_status);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return INF_OK;
}

int32_t inf_ctx_set_stream(inf_ctx* ctx, void* stream) {
    INF_CHECK_CTX(ctx);
    if (!stream) return inf_fail(ctx, INF_E_ARG, "inf_ctx_set_stream: null stream");
    if (ctx->own_stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
        ctx->own_stream = false;
    }
    ctx->stream = (cudaStream_t)stream;
    return INF_OK;
}

const char* inf_last_error(inf_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int32_t inf_device_values_supported(inf_ctx* ctx) { return ctx ? 1 : 0; }

int32_t inf_flush(inf_ctx* ctx) {
    INF_CHECK_CTX(ctx);
    INF_CUDA(ctx, cudaMemcpyAsync(ctx->host_status, ctx->status, 16, cudaMemcpyDeviceToHost, ctx->stream));
    INF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int s = ctx->host_status[0];
    if (s != 0) {
        INF_CUDA(ctx, cudaMemsetAsync(ctx->status, 0, 16, ctx->stream));
        return inf_fail(ctx, INF_E_BACKEND, "device status word 0x%x:%s%s%s%s", s,
                        (s & INF_STATUS_WAIT_TIMEOUT) ? " bounded wait gave up;" : "",
                        (s & INF_STATUS_BAD_PAGE) ? " page id outside the pool;" : "",
                        (s & INF_STATUS_BAD_LEN) ? " length beyond the page table or max_len;" : "",
                        (s & INF_STATUS_BAD_SMEM) ? " shared-memory base misaligned;" : "");
    }
    return INF_OK;
}

int32_t inf_profile_enable(inf_ctx* ctx, int32_t on) {
    INF_CHECK_CTX(ctx);
    ctx->prof_on = on != 0;
    return INF_OK;
}

int32_t inf_profile_read(inf_ctx* ctx, const char* kernel_name, double* total_ms, int32_t* launches) {
    INF_CHECK_CTX(ctx);
    if (!kernel_name || !total_ms || !launches) return inf_fail(ctx, INF_E_ARG, "inf_profile_read: null pointer");
    INF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    double sum = 0.0;
    int n = 0;
    for (size_t i = 0; i < ctx->prof.size();) {
        if (strcmp(ctx->prof[i].name, kernel_name) == 0) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, ctx->prof[i].a, ctx->prof[i].b) == cudaSuccess) {
                sum += ms;
                ++n;
            }
            cudaEventDestroy(ctx->prof[i].a);
            cudaEventDestroy(ctx->prof[i].b);
            ctx->prof.erase(ctx->prof.begin() + i);
        } else {
            ++i;
        }
    }
    *total_ms = sum;
    *launches = n;
    return INF_OK;
}

int32_t inf_submit(inf_ctx* ctx) {
    INF_CHECK_CTX(ctx);
    return INF_OK;
}

int32_t inf_alloc(inf_ctx* ctx, size_t bytes, void** device_out) {
    INF_CHECK_CTX(ctx);
    if (!device_out) return inf_fail(ctx, INF_E_ARG, "inf_alloc: null output");
    INF_CUDA(ctx, cudaSetDevice(ctx->device));
    INF_CUDA(ctx, cudaMalloc(device_out, bytes ? bytes : 16));
    return INF_OK;
}

int32_t inf_free(inf_ctx* ctx, void* p) {
    INF_CHECK_CTX(ctx);
    if (!p) return INF_OK;
    INF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    INF_CUDA(ctx, cudaFree(p));
    for (size_t i = 0; i < ctx->tmaps.size();)  // descriptors over freed memory must not be reused
        if (ctx->tmaps[i].first.base == p)
            ctx->tmaps.erase(ctx->tmaps.begin() + i);
        else
            ++i;
    return INF_OK;
}

int32_t inf_upload(inf_ctx* ctx, void* dst, const void* src, size_t bytes) {
    INF_CHECK_CTX(ctx);
    if (!dst || !src) return inf_fail(ctx, INF_E_ARG, "inf_upload: null pointer");
    INF_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    INF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the host buffer may be pageable and reused
    return INF_OK;
}

int32_t inf_download(inf_ctx* ctx, void* dst, const void* src, size_t bytes) {
    INF_CHECK_CTX(ctx);
    if (!dst || !src) return inf_fail(ctx, INF_E_ARG, "inf_download: null pointer");
    INF_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    INF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return INF_OK;
}

int32_t inf_copy(inf_ctx* ctx, void* dst, const void* src, size_t bytes) {
    INF_CHECK_CTX(ctx);
    if (!dst || !src) return inf_fail(ctx, INF_E_ARG, "inf_copy: null pointer");
    INF_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return INF_OK;
}

int32_t inf_memset_zero(inf_ctx* ctx, void* dst, size_t bytes) {
    INF_CHECK_CTX(ctx);
    if (!dst) return inf_fail(ctx, INF_E_ARG, "inf_memset_zero: null pointer");
    INF_CUDA(ctx, cudaMemsetAsync(dst, 0, bytes, ctx->stream));
    return INF_OK;
}

__global__ void f32_to_f16_kernel(const float* __restrict__ in, __half* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = __float2half_rn(in[i]);
}

int32_t inf_upload_f32_as_f16(inf_ctx* ctx, void* dst, const float* src, size_t count) {
    INF_CHECK_CTX(ctx);
    if (!dst || !src) return inf_fail(ctx, INF_E_ARG, "inf_upload_f32_as_f16: null pointer");
    int rc = inf_ensure_workspace(ctx, count * sizeof(float));
    if (rc != INF_OK) return rc;
    INF_CUDA(ctx, cudaMemcpyAsync(ctx->workspace, src, count * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    int blocks = (int)((count + 255) / 256);
    if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
    if (blocks < 1) blocks = 1;
    f32_to_f16_kernel<<<blocks, 256, 0, ctx->stream>>>((const float*)ctx->workspace, (__half*)dst, count);
    INF_LAUNCH_CHECK(ctx, "f32_to_f16_kernel");
    INF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return INF_OK;
}

int32_t inf_rope_table_create(inf_ctx* ctx, const float* host_inv_freq, int32_t count, int32_t rotary_dim,
                              float attention_factor, inf_rope_table* out) {
    INF_CHECK_CTX(ctx);
    if (!host_inv_freq || !out) return inf_fail(ctx, INF_E_ARG, "rope table: null pointer");
    // metal/rope.rs:448-487
    if (rotary_dim != 64 && rotary_dim != 128)
        return inf_fail(ctx, INF_E_BACKEND, "Laguna rotary dimension must be 64 or 128, got %d", rotary_dim);
    if (!isfinite(attention_factor) || attention_factor <= 0.0f)
        return inf_fail(ctx, INF_E_BACKEND, "Laguna RoPE attention factor must be positive and finite, got %g",
                        attention_factor);
    if (count != rotary_dim / 2)
        return inf_fail(ctx, INF_E_BACKEND, "Laguna inverse-frequency length must be %d, got %d", rotary_dim / 2,
                        count);
    for (int i = 0; i < count; ++i)
        if (!isfinite(host_inv_freq[i]) || host_inv_freq[i] <= 0.0f)
            return inf_fail(ctx, INF_E_BACKEND, "Laguna inverse frequencies must be positive and finite");
    void* d = nullptr;
    INF_CUDA(ctx, cudaMalloc(&d, count * sizeof(float)));
    INF_CUDA(ctx, cudaMemcpyAsync(d, host_inv_freq, count * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    INF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    out->inv_freq = (const float*)d;
    out->rotary_dim = rotary_dim;
    out->attention_factor = attention_factor;
    return INF_OK;
}

int32_t inf_rope_table_destroy(inf_ctx* ctx, inf_rope_table* t) {
    INF_CHECK_CTX(ctx);
    if (!t) return INF_OK;
    int rc = inf_free(ctx, const_cast<float*>(t->inv_freq));
    t->inv_freq = nullptr;
    return rc;
}

int32_t inf_kv_pool_create(inf_ctx* ctx, int32_t num_pages, int32_t page_size, int32_t kv_heads, int32_t head_dim,
                           inf_kv_pool* out) {
    INF_CHECK_CTX(ctx);
    if (!out) return inf_fail(ctx, INF_E_ARG, "kv pool: null output");
    if (num_pages <= 0 || kv_heads <= 0) return inf_fail(ctx, INF_E_CACHE, "kv pool: sizes must be positive");
    if (page_size <= 0 || page_size % 16 != 0)
        return inf_fail(ctx, INF_E_CACHE, "kv pool: page_size must be a positive multiple of 16, got %d", page_size);
    if (head_dim != 128) return inf_fail(ctx, INF_E_SHAPE, "kv pool: head_dim must be 128, got %d", head_dim);
    size_t bytes = (size_t)num_pages * kv_heads * page_size * head_dim * sizeof(__half);
    void *k = nullptr, *v = nullptr;
    INF_CUDA(ctx, cudaMalloc(&k, bytes));
    cudaError_t e = cudaMalloc(&v, bytes);
    if (e != cudaSuccess) {
        cudaFree(k);
        return inf_fail(ctx, INF_E_BACKEND, "kv pool: cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    INF_CUDA(ctx, cudaMemsetAsync(k, 0, bytes, ctx->stream));
    INF_CUDA(ctx, cudaMemsetAsync(v, 0, bytes, ctx->stream));
    out->k = k;
    out->v = v;
    out->num_pages = num_pages;
    out->page_size = page_size;
    out->kv_heads = kv_heads;
    out->head_dim = head_dim;
    return INF_OK;
}

int32_t inf_kv_pool_destroy(inf_ctx* ctx, inf_kv_pool* pool) {
    INF_CHECK_CTX(ctx);
    if (!pool) return INF_OK;
    int rc = inf_free(ctx, pool->k);
    int rc2 = inf_free(ctx, pool->v);
    pool->k = pool->v = nullptr;
    return rc != INF_OK ? rc : rc2;
}

int32_t inf_kv_pool_fp8_create(inf_ctx* ctx, int32_t num_pages, int32_t page_size, int32_t kv_heads, int32_t head_dim,
                               float key_scale, float value_scale, inf_kv_pool_fp8* out) {
    INF_CHECK_CTX(ctx);
    if (!out) return inf_fail(ctx, INF_E_ARG, "fp8 kv pool: null output");
    if (num_pages <= 0 || kv_heads <= 0) return inf_fail(ctx, INF_E_CACHE, "fp8 kv pool: sizes must be positive");
    if (page_size <= 0 || page_size % 16 != 0)
        return inf_fail(ctx, INF_E_CACHE, "fp8 kv pool: page_size must be a positive multiple of 16, got %d", page_size);
    if (head_dim != 128) return inf_fail(ctx, INF_E_SHAPE, "fp8 kv pool: head_dim must be 128, got %d", head_dim);
    // crates/backend/src/metal/fp8_attention.rs: the scales must be positive and finite
    if (!(key_scale > 0.f) || !(value_scale > 0.f) || !isfinite(key_scale) || !isfinite(value_scale))
        return inf_fail(ctx, INF_E_CONFIG, "fp8 kv pool: scales must be positive and finite");
    size_t bytes = (size_t)num_pages * kv_heads * page_size * head_dim;
    void *k = nullptr, *v = nullptr;
    INF_CUDA(ctx, cudaMalloc(&k, bytes));
    cudaError_t e = cudaMalloc(&v, bytes);
    if (e != cudaSuccess) {
        cudaFree(k);
        return inf_fail(ctx, INF_E_BACKEND, "fp8 kv pool: cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    INF_CUDA(ctx, cudaMemsetAsync(k, 0, bytes, ctx->stream));  // byte 0 decodes to 0.0
    INF_CUDA(ctx, cudaMemsetAsync(v, 0, bytes, ctx->stream));
    *out = inf_kv_pool_fp8{k, v, num_pages, page_size, kv_heads, head_dim, key_scale, value_scale};
    return INF_OK;
}

int32_t inf_kv_pool_fp8_destroy(inf_ctx* ctx, inf_kv_pool_fp8* pool) {
    INF_CHECK_CTX(ctx);
    if (!pool) return INF_OK;
    int rc = inf_free(ctx, pool->k);
    int rc2 = inf_free(ctx, pool->v);
    pool->k = pool->v = nullptr;
    return rc != INF_OK ? rc : rc2;
}

int32_t inf_mla_pool_create(inf_ctx* ctx, int32_t num_pages, int32_t page_size, int32_t latent_dim, int32_t rope_dim,
                            inf_mla_pool* out) {
    INF_CHECK_CTX(ctx);
    if (!out) return inf_fail(ctx, INF_E_ARG, "mla pool: null output");
    if (num_pages <= 0) return inf_fail(ctx, INF_E_CACHE, "mla pool: num_pages must be positive");
    if (page_size != 64) return inf_fail(ctx, INF_E_CACHE, "mla pool: page_size must be 64, got %d", page_size);
    if (latent_dim != 512 || rope_dim != 64)
        return inf_fail(ctx, INF_E_SHAPE, "mla pool: row must be 512 + 64, got %d + %d", latent_dim, rope_dim);
    size_t bytes = (size_t)num_pages * page_size * (latent_dim + rope_dim) * sizeof(__half);
    void* r = nullptr;
    INF_CUDA(ctx, cudaMalloc(&r, bytes));
    INF_CUDA(ctx, cudaMemsetAsync(r, 0, bytes, ctx->stream));
    out->rows = r;
    out->num_pages = num_pages;
    out->page_size = page_size;
    out->latent_dim = latent_dim;
    out->rope_dim = rope_dim;
    return INF_OK;
}

int32_t inf_mla_pool_destroy(inf_ctx* ctx, inf_mla_pool* pool) {
    INF_CHECK_CTX(ctx);
    if (!pool) return INF_OK;
    int rc = inf_free(ctx, pool->rows);
    pool->rows = nullptr;
    return rc;
}

}  // extern "C"

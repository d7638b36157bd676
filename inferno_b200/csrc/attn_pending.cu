// Entry points whose kernels are not built yet answer INF_UNSUPPORTED (the reference's Ok(None)).
#include "common.cuh"
extern "C" {
int32_t inf_laguna_gated_gqa_f16_attention(inf_ctx* ctx, const float*, const float*, const float*, const float*,
                                           const inf_kv_pool*, const inf_page_table*, int32_t, int32_t, int32_t,
                                           int32_t, float*) { INF_CHECK_CTX(ctx); return INF_UNSUPPORTED; }
}

// Host-side plumbing shared by every translation unit of the library: the context
// object behind inf_ctx, error reporting, scratch memory, and TMA descriptor creation.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <vector>

#include "../../include/inferno_attn.h"

// Bits of the device status word (ctx->status[0]); kernels OR them in and keep going safely.
#define INF_STATUS_WAIT_TIMEOUT 1  // a bounded mbarrier wait gave up
#define INF_STATUS_BAD_PAGE 2      // a page id outside the pool was refused
#define INF_STATUS_BAD_LEN 4       // a length that does not fit the page table or the size the launch was given
#define INF_STATUS_BAD_SMEM 8      // the dynamic shared-memory base is not aligned as the tiles need

typedef CUresult (*inf_tmap_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct inf_tmap_key {
    const void* base;
    uint64_t dims[3];
    uint64_t strides[2];
    uint32_t box[3];
    uint32_t rank;
    bool operator==(const inf_tmap_key& o) const {
        if (base != o.base || rank != o.rank) return false;
        for (int i = 0; i < 3; ++i)
            if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
        return strides[0] == o.strides[0] && strides[1] == o.strides[1];
    }
};

struct inf_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int sm_count = 0;
    std::string err;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    std::vector<void*> retired_workspaces;  // outgrown workspaces, kept until destroy: captured graphs may name them
    size_t dsa_scores_smem = 0;  // dynamic shared memory the tensor-core index-score kernel has been allowed so far
    int* status = nullptr;       // device int32[4]
    int* host_status = nullptr;  // pinned int32[4]
    inf_tmap_encode_fn encode = nullptr;
    std::vector<std::pair<inf_tmap_key, CUtensorMap>> tmaps;
    int debug_drop_tile = -1;  // diagnostic: see inf_debug_drop_next_load
    uint32_t func_attr_done = 0;  // one bit per kernel whose dynamic shared-memory limit has been raised
    // optional per-kernel timing (inf_profile_enable): event pairs around named kernels
    bool prof_on = false;
    struct prof_rec {
        const char* name;
        cudaEvent_t a, b;
    };
    std::vector<prof_rec> prof;
};

// Records an event pair around one kernel launch when profiling is on; a no-op otherwise.
struct inf_prof_scope {
    inf_ctx* ctx;
    cudaEvent_t a = nullptr, b = nullptr;
    const char* name;
    inf_prof_scope(inf_ctx* c, const char* n) : ctx(c), name(n) {
        if (ctx->prof_on && cudaEventCreate(&a) == cudaSuccess && cudaEventCreate(&b) == cudaSuccess)
            cudaEventRecord(a, ctx->stream);
    }
    ~inf_prof_scope() {
        if (a && b) {
            cudaEventRecord(b, ctx->stream);
            ctx->prof.push_back({name, a, b});
        }
    }
};

int inf_fail(inf_ctx* ctx, int code, const char* fmt, ...);
// Grows (never shrinks) the context's scratch buffer.  An outgrown buffer is kept until the context is destroyed,
// so work already enqueued -- or a CUDA graph captured earlier -- that names it stays valid.
int inf_ensure_workspace(inf_ctx* ctx, size_t bytes);
// fp16 tiled tensor map with the 128-byte swizzle, rank 2 or 3.  dims/strides innermost first;
// strides in bytes for dims 1..rank-1.
int inf_make_tmap(inf_ctx* ctx, const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides_bytes,
                  const uint32_t* box, CUtensorMap* out);
// The same for elements of elem_bytes bytes (1: bytes, e.g. FP8 pages; 2: fp16); dims and box count elements.
int inf_make_tmap_typed(inf_ctx* ctx, const void* base, uint32_t rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box, CUtensorMap* out, uint32_t elem_bytes);

#define INF_CHECK_CTX(ctx) \
    do {                   \
        if (!(ctx)) return INF_E_ARG; \
    } while (0)

#define INF_CUDA(ctx, call)                                                                              \
    do {                                                                                                 \
        cudaError_t e__ = (call);                                                                        \
        if (e__ != cudaSuccess)                                                                          \
            return inf_fail(ctx, INF_E_BACKEND, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), \
                            __FILE__, __LINE__);                                                         \
    } while (0)

#define INF_LAUNCH_CHECK(ctx, name)                                                                  \
    do {                                                                                             \
        cudaError_t e__ = cudaGetLastError();                                                        \
        if (e__ != cudaSuccess)                                                                      \
            return inf_fail(ctx, INF_E_BACKEND, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

// Programmatic dependent launch for the kernels of one decode step.  A kernel launched through inf_launch_pdl may
// be scheduled while the kernel before it in the stream is still running; it must execute inf_pdl_wait() before
// its first access to global memory (which waits for that kernel to finish and its writes to be visible), so all
// that overlaps is the launch itself and the block set-up.  inf_pdl_release() lets the next kernel of the stream
// be scheduled early in the same way.  Outside such a launch both calls return at once.
#ifdef __CUDACC__
__device__ __forceinline__ void inf_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void inf_pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t inf_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

// Host-side range check of the page-table entries a launch may touch (needs the host mirrors).
// window / query_tokens: with a sliding window, page slots wholly below the lowest key the first of the call's
// query_tokens rows can see are not checked (they may have been trimmed away).  append_only: the call writes its
// extra_tokens rows and reads nothing else, so only their pages are checked.
int inf_validate_table(inf_ctx* ctx, const inf_page_table* t, int num_pages, int page_size, int extra_tokens,
                       const char* what, int window = 0, int query_tokens = 1, bool append_only = false);

// The one collective of the path: an all-gather of the head-sharded attention output over NCCL
// (NVLink 5 / NVSwitch).  NCCL is bound at run time with dlopen, so the library loads on hosts without it
// and single-GPU users never touch it.  The reference has no multi-device path; there is nothing to mirror.
#include <dlfcn.h>
#include <string.h>

#include "common.cuh"

namespace {

typedef struct { char internal[128]; } nccl_unique_id;
typedef void* nccl_comm_t;
typedef int nccl_result_t;

struct NcclApi {
    void* handle = nullptr;
    nccl_result_t (*GetUniqueId)(nccl_unique_id*) = nullptr;
    nccl_result_t (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int) = nullptr;
    nccl_result_t (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
    nccl_result_t (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
    nccl_result_t (*CommDestroy)(nccl_comm_t) = nullptr;
    const char* (*GetErrorString)(nccl_result_t) = nullptr;
    bool tried = false;
};
NcclApi g_nccl;

bool load_nccl(std::string* why) {
    if (g_nccl.tried) {
        if (!g_nccl.handle && why) *why = "NCCL could not be loaded earlier in this process";
        return g_nccl.handle != nullptr;
    }
    g_nccl.tried = true;
    const char* names[] = {getenv("INFERNO_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        if (!n) continue;
        g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.handle) break;
    }
    if (!g_nccl.handle) {
        if (why) *why = std::string("dlopen of libnccl failed: ") + (dlerror() ? dlerror() : "not found");
        return false;
    }
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))dlsym(g_nccl.handle, "ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))dlsym(g_nccl.handle, "ncclCommInitRank");
    g_nccl.AllGather = (decltype(g_nccl.AllGather))dlsym(g_nccl.handle, "ncclAllGather");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))dlsym(g_nccl.handle, "ncclAllReduce");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(g_nccl.handle, "ncclCommDestroy");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(g_nccl.handle, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllGather || !g_nccl.AllReduce || !g_nccl.CommDestroy) {
        if (why) *why = "libnccl lacks a required symbol";
        g_nccl.handle = nullptr;
        return false;
    }
    return true;
}

const char* nccl_err(nccl_result_t r) { return g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "nccl error"; }

}  // namespace

struct inf_comm {
    inf_ctx* ctx;
    nccl_comm_t comm;
    int rank, nranks;
    int* token = nullptr;  // device int the barrier reduces
};

extern "C" {

int32_t inf_comm_unique_id(inf_ctx* ctx, void* id_out) {
    INF_CHECK_CTX(ctx);
    if (!id_out) return inf_fail(ctx, INF_E_ARG, "comm_unique_id: null output");
    std::string why;
    if (!load_nccl(&why)) return inf_fail(ctx, INF_E_BACKEND, "%s", why.c_str());
    nccl_unique_id id;
    nccl_result_t r = g_nccl.GetUniqueId(&id);
    if (r != 0) return inf_fail(ctx, INF_E_BACKEND, "ncclGetUniqueId failed: %s", nccl_err(r));
    memcpy(id_out, &id, sizeof(id));
    return INF_OK;
}

int32_t inf_comm_init(inf_ctx* ctx, const void* id, int32_t rank, int32_t nranks, inf_comm** out) {
    INF_CHECK_CTX(ctx);
    if (!id || !out) return inf_fail(ctx, INF_E_ARG, "comm_init: null pointer");
    *out = nullptr;
    if (nranks <= 0 || rank < 0 || rank >= nranks)
        return inf_fail(ctx, INF_E_CONFIG, "comm_init: rank %d of %d is not valid", rank, nranks);
    std::string why;
    if (!load_nccl(&why)) return inf_fail(ctx, INF_E_BACKEND, "%s", why.c_str());
    INF_CUDA(ctx, cudaSetDevice(ctx->device));
    nccl_unique_id uid;
    memcpy(&uid, id, sizeof(uid));
    nccl_comm_t c = nullptr;
    nccl_result_t r = g_nccl.CommInitRank(&c, nranks, uid, rank);
    if (r != 0) return inf_fail(ctx, INF_E_BACKEND, "ncclCommInitRank failed: %s", nccl_err(r));
    inf_comm* comm = new inf_comm{ctx, c, rank, nranks};
    if (cudaMalloc(&comm->token, sizeof(int)) != cudaSuccess || cudaMemset(comm->token, 0, sizeof(int)) != cudaSuccess) {
        g_nccl.CommDestroy(c);
        delete comm;
        return inf_fail(ctx, INF_E_BACKEND, "comm_init: could not allocate the barrier token");
    }
    *out = comm;
    return INF_OK;
}

int32_t inf_comm_destroy(inf_comm* comm) {
    if (!comm) return INF_OK;
    cudaStreamSynchronize(comm->ctx->stream);
    if (g_nccl.CommDestroy) g_nccl.CommDestroy(comm->comm);
    if (comm->token) cudaFree(comm->token);
    delete comm;
    return INF_OK;
}

int32_t inf_allgather_heads(inf_comm* comm, const void* send, void* recv, size_t bytes) {
    if (!comm) return INF_E_ARG;
    inf_ctx* ctx = comm->ctx;
    if (!send || !recv) return inf_fail(ctx, INF_E_ARG, "allgather_heads: null pointer");
    if (bytes == 0) return INF_OK;
    nccl_result_t r = g_nccl.AllGather(send, recv, bytes, /*ncclInt8*/ 0, comm->comm, ctx->stream);
    if (r != 0) return inf_fail(ctx, INF_E_BACKEND, "ncclAllGather failed: %s", nccl_err(r));
    return INF_OK;
}

int32_t inf_comm_barrier(inf_comm* comm) {
    if (!comm) return INF_E_ARG;
    inf_ctx* ctx = comm->ctx;
    // a four-byte all-reduce on the context's stream: when it has run on a rank, every rank's earlier work on its own
    // stream -- kernels that stored into this rank's memory included -- has finished
    nccl_result_t r = g_nccl.AllReduce(comm->token, comm->token, 1, /*ncclInt32*/ 2, /*ncclMax*/ 2, comm->comm, ctx->stream);
    if (r != 0) return inf_fail(ctx, INF_E_BACKEND, "ncclAllReduce (barrier) failed: %s", nccl_err(r));
    return INF_OK;
}

int32_t inf_peer_export(inf_ctx* ctx, const void* device_ptr, void* handle_out) {
    INF_CHECK_CTX(ctx);
    if (!device_ptr || !handle_out) return inf_fail(ctx, INF_E_ARG, "peer_export: null pointer");
    // the handle names the whole allocation the pointer lies in; the offset inside it travels with the handle
    CUdeviceptr base = 0;
    size_t size = 0;
    typedef CUresult (*range_fn)(CUdeviceptr*, size_t*, CUdeviceptr);
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn)
        return inf_fail(ctx, INF_E_BACKEND, "peer_export: cuMemGetAddressRange is not available");
    if (((range_fn)fn)(&base, &size, (CUdeviceptr)device_ptr) != CUDA_SUCCESS)
        return inf_fail(ctx, INF_E_ARG, "peer_export: %p is not a device allocation", device_ptr);
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, (void*)base);
    if (e != cudaSuccess) return inf_fail(ctx, INF_E_BACKEND, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle_out, &h, 64);
    const uint64_t offset = (uint64_t)((CUdeviceptr)device_ptr - base);
    memcpy((char*)handle_out + 64, &offset, 8);
    return INF_OK;
}

int32_t inf_peer_open(inf_ctx* ctx, const void* handle, void** peer_ptr) {
    INF_CHECK_CTX(ctx);
    if (!handle || !peer_ptr) return inf_fail(ctx, INF_E_ARG, "peer_open: null pointer");
    *peer_ptr = nullptr;
    INF_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    uint64_t offset = 0;
    memcpy(&offset, (const char*)handle + 64, 8);
    void* base = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return inf_fail(ctx, INF_E_BACKEND, "cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
    *peer_ptr = (char*)base + offset;
    return INF_OK;
}

int32_t inf_peer_close(inf_ctx* ctx, void* peer_ptr, const void* handle) {
    INF_CHECK_CTX(ctx);
    if (!peer_ptr || !handle) return INF_OK;
    uint64_t offset = 0;
    memcpy(&offset, (const char*)handle + 64, 8);
    INF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    INF_CUDA(ctx, cudaIpcCloseMemHandle((char*)peer_ptr - offset));
    return INF_OK;
}

}  // extern "C"

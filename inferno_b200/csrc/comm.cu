// The one collective of the path: an all-gather of the head-sharded attention output over NCCL
// (NVLink 5 / NVSwitch).  NCCL is bound at run time with dlopen, so the library loads on hosts without it
// and single-GPU users never touch it.  The reference has no multi-device path; there is nothing to mirror.
#include <dlfcn.h>
#include <string.h>

#include <vector>

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

constexpr int FLAG_SLOTS = 64;   // [0, 32): arrival values written by the peers; [32]: this rank's epoch
constexpr int EPOCH_SLOT = 32;
constexpr int MAX_RANKS = INF_MAX_PEERS + 1;

struct PeerFlags {
    int* of[MAX_RANKS];  // every rank's flag array as mapped into this process (own entry: the local array)
};

struct inf_comm {
    inf_ctx* ctx;
    nccl_comm_t comm;
    int rank, nranks;
    int* token = nullptr;  // device int the NCCL form of the barrier reduces
    int* flags = nullptr;  // this rank's flag array (FLAG_SLOTS ints), written by the peers' barrier kernels
    PeerFlags peers = {};
    bool p2p = false;      // the peers' flag arrays are mapped: the barrier is one small kernel, no NCCL call
};

// One CTA, one thread per rank.  Thread r tells rank r "I have arrived at barrier number e" with a store into r's
// flag array over NVLink and waits until r has said the same here.  Everything this rank's stream ran before the
// barrier -- kernels that stored into the peers' memory included -- has completed before this kernel starts, and the
// system-wide fence orders those stores before the flag.  The wait is bounded: a rank that never arrives turns into
// the status word's time-out bit, not into a hung GPU.  Each rank's kernel runs on its own GPU.
__global__ void comm_barrier_kernel(int* mine, PeerFlags peers, int rank, int world, int* status) {
    __shared__ int e_s;
    const int r = threadIdx.x;
    // launched as a programmatic dependent: resident while the kernel before it drains, and past this point only when
    // that kernel has completed and its stores (into the peers' memory too) have been performed
    inf_pdl_wait();
    if (r == 0) e_s = mine[EPOCH_SLOT] + 1;
    __syncthreads();
    const int e = e_s;
    if (r < world && r != rank) {
        __threadfence_system();
        volatile int* there = peers.of[r] + rank;
        *there = e;
        volatile int* here = mine + r;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        while (*here < e) {
            __nanosleep(32);
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 2000000000ull) {
                atomicOr(status, INF_STATUS_WAIT_TIMEOUT);
                break;
            }
        }
        // what the peers stored before their flags already lies in this GPU's memory; the kernels after this one start
        // with cold L1 caches, so a device-scope fence is all that is left to do
        __threadfence();
    }
    __syncthreads();
    if (r == 0) mine[EPOCH_SLOT] = e;
}

static int peer_export_impl(inf_ctx* ctx, const void* device_ptr, void* handle_out);
static int peer_open_impl(inf_ctx* ctx, const void* handle, void** peer_ptr);

// Exchange the flag arrays' handles over NCCL itself and map them.  Any failure leaves the NCCL barrier in place.
void setup_p2p_barrier(inf_comm* c) {
    inf_ctx* ctx = c->ctx;
    if (c->nranks > MAX_RANKS || c->nranks < 2) return;
    if (cudaMalloc(&c->flags, FLAG_SLOTS * sizeof(int)) != cudaSuccess) return;
    cudaMemset(c->flags, 0, FLAG_SLOTS * sizeof(int));
    char mine[INF_PEER_HANDLE_BYTES];
    if (peer_export_impl(ctx, c->flags, mine) != INF_OK) return;
    char *d_send = nullptr, *d_recv = nullptr;
    if (cudaMalloc(&d_send, INF_PEER_HANDLE_BYTES) != cudaSuccess ||
        cudaMalloc(&d_recv, (size_t)INF_PEER_HANDLE_BYTES * c->nranks) != cudaSuccess)
        return;
    std::vector<char> all((size_t)INF_PEER_HANDLE_BYTES * c->nranks);
    bool ok = cudaMemcpy(d_send, mine, INF_PEER_HANDLE_BYTES, cudaMemcpyHostToDevice) == cudaSuccess &&
              g_nccl.AllGather(d_send, d_recv, INF_PEER_HANDLE_BYTES, /*ncclInt8*/ 0, c->comm, ctx->stream) == 0 &&
              cudaStreamSynchronize(ctx->stream) == cudaSuccess &&
              cudaMemcpy(all.data(), d_recv, all.size(), cudaMemcpyDeviceToHost) == cudaSuccess;
    cudaFree(d_send);
    cudaFree(d_recv);
    if (!ok) return;
    int mapped = 0;
    for (int r = 0; r < c->nranks; ++r) {
        if (r == c->rank) {
            c->peers.of[r] = c->flags;
            continue;
        }
        void* p = nullptr;
        if (peer_open_impl(ctx, all.data() + (size_t)r * INF_PEER_HANDLE_BYTES, &p) == INF_OK) {
            c->peers.of[r] = (int*)p;
            ++mapped;
        }
    }
    // every rank must come to the same decision: agree through one more reduction (min over ranks)
    int* d_ok = c->token;
    int mine_ok = mapped == c->nranks - 1 ? 1 : 0, all_ok = 0;
    if (cudaMemcpy(d_ok, &mine_ok, sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess &&
        g_nccl.AllReduce(d_ok, d_ok, 1, /*ncclInt32*/ 2, /*ncclMin*/ 3, c->comm, ctx->stream) == 0 &&
        cudaStreamSynchronize(ctx->stream) == cudaSuccess &&
        cudaMemcpy(&all_ok, d_ok, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess)
        c->p2p = all_ok == 1;
    cudaMemset(c->token, 0, sizeof(int));
}

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
    setup_p2p_barrier(comm);
    *out = comm;
    return INF_OK;
}

int32_t inf_comm_destroy(inf_comm* comm) {
    if (!comm) return INF_OK;
    cudaStreamSynchronize(comm->ctx->stream);
    if (g_nccl.CommDestroy) g_nccl.CommDestroy(comm->comm);
    if (comm->token) cudaFree(comm->token);
    for (int r = 0; r < comm->nranks && r < MAX_RANKS; ++r)
        if (r != comm->rank && comm->peers.of[r]) cudaIpcCloseMemHandle(comm->peers.of[r]);
    if (comm->flags) cudaFree(comm->flags);
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

int32_t inf_comm_barrier_is_p2p(inf_comm* comm) { return comm && comm->p2p ? 1 : 0; }

int32_t inf_comm_barrier(inf_comm* comm) {
    if (!comm) return INF_E_ARG;
    inf_ctx* ctx = comm->ctx;
    if (comm->p2p) {
        INF_CUDA(ctx, inf_launch_pdl(comm_barrier_kernel, dim3(1), dim3(32), 0, ctx->stream, comm->flags, comm->peers,
                                     comm->rank, comm->nranks, ctx->status));
        INF_LAUNCH_CHECK(ctx, "comm_barrier_kernel");
        return INF_OK;
    }
    // otherwise a four-byte all-reduce on the context's stream: when it has run on a rank, every rank's earlier work on its own
    // stream -- kernels that stored into this rank's memory included -- has finished
    nccl_result_t r = g_nccl.AllReduce(comm->token, comm->token, 1, /*ncclInt32*/ 2, /*ncclMax*/ 2, comm->comm, ctx->stream);
    if (r != 0) return inf_fail(ctx, INF_E_BACKEND, "ncclAllReduce (barrier) failed: %s", nccl_err(r));
    return INF_OK;
}

int32_t inf_peer_export(inf_ctx* ctx, const void* device_ptr, void* handle_out) {
    INF_CHECK_CTX(ctx);
    return peer_export_impl(ctx, device_ptr, handle_out);
}

int32_t inf_peer_open(inf_ctx* ctx, const void* handle, void** peer_ptr) {
    INF_CHECK_CTX(ctx);
    return peer_open_impl(ctx, handle, peer_ptr);
}

}  // extern "C"

static int peer_export_impl(inf_ctx* ctx, const void* device_ptr, void* handle_out) {
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

static int peer_open_impl(inf_ctx* ctx, const void* handle, void** peer_ptr) {
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

extern "C" {

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

// NCCL plumbing behind the C ABI: the same entry-point names as the reference's runtime-
// compiled shims (minit/nccl/library.py:41-58, minit/nccl/kernel.py:47-57), but libnccl is
// opened with dlopen() so this library carries no link-time dependency on it, and every call
// returns a status instead of throwing.
#include <dlfcn.h>
#include <string.h>
#include <cuda_runtime.h>
#include <mutex>
#include "../../include/minit_b200.h"

namespace {

// Minimal mirror of the NCCL declarations used here (stable public ABI of nccl.h).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclInt32 = 2, ncclFloat16 = 6, ncclFloat32 = 7, ncclBfloat16 = 9 };
enum { ncclSum = 0 };

struct Api {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
};
Api g_api;
std::mutex g_mu;

int load_locked(const char* path) {
    if (g_api.handle) return MT_OK;
    void* h = dlopen(path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return MT_ERR_NCCL;
    Api a;
    a.handle = h;
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
    a.Broadcast = reinterpret_cast<decltype(a.Broadcast)>(dlsym(h, "ncclBroadcast"));
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllGather || !a.AllReduce || !a.Broadcast) {
        dlclose(h);
        return MT_ERR_NCCL;
    }
    g_api = a;
    return MT_OK;
}

int ensure_loaded() {
    std::lock_guard<std::mutex> lk(g_mu);
    return load_locked(nullptr);
}

int nccl_dtype(int dtype) {
    switch (dtype) {
        case MT_F16: return ncclFloat16;
        case MT_BF16: return ncclBfloat16;
        case 2: return ncclFloat32;
        case 3: return ncclInt32;
    }
    return -1;
}

}  // namespace

extern "C" {

int mt_nccl_load(const char* path) {
    std::lock_guard<std::mutex> lk(g_mu);
    return load_locked(path);
}

size_t nccl_unique_id_size(void) { return sizeof(ncclUniqueId); }

int nccl_create_unique_id(char* bytes) {
    if (!bytes) return MT_ERR_NULL;
    int rc = ensure_loaded();
    if (rc != MT_OK) return rc;
    ncclUniqueId id;
    if (g_api.GetUniqueId(&id) != 0) return MT_ERR_NCCL;
    memcpy(bytes, &id, sizeof(id));
    return MT_OK;
}

int nccl_init_rank(int nr_ranks, int rank, const char* bytes, int device, void** comm_out) {
    if (!bytes || !comm_out) return MT_ERR_NULL;
    if (nr_ranks < 1 || rank < 0 || rank >= nr_ranks) return MT_ERR_SHAPE;
    int rc = ensure_loaded();
    if (rc != MT_OK) return rc;
    if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    ncclUniqueId id;
    memcpy(&id, bytes, sizeof(id));
    ncclComm_t comm = nullptr;
    if (g_api.CommInitRank(&comm, nr_ranks, id, rank) != 0) return MT_ERR_NCCL;
    *comm_out = comm;
    return MT_OK;
}

int nccl_destroy(void* comm) {
    if (!comm) return MT_ERR_NULL;
    int rc = ensure_loaded();
    if (rc != MT_OK) return rc;
    return g_api.CommDestroy(static_cast<ncclComm_t>(comm)) == 0 ? MT_OK : MT_ERR_NCCL;
}

int nccl_all_gather(void* stream, void* comm, const void* sendbuff, void* recvbuff, size_t count, int dtype) {
    if (!comm || !sendbuff || !recvbuff) return MT_ERR_NULL;
    const int dt = nccl_dtype(dtype);
    if (dt < 0) return MT_ERR_DTYPE;
    int rc = ensure_loaded();
    if (rc != MT_OK) return rc;
    return g_api.AllGather(sendbuff, recvbuff, count, dt, static_cast<ncclComm_t>(comm), static_cast<cudaStream_t>(stream)) == 0 ? MT_OK : MT_ERR_NCCL;
}

int nccl_all_reduce(void* stream, void* comm, const void* sendbuff, void* recvbuff, size_t count, int dtype) {
    if (!comm || !sendbuff || !recvbuff) return MT_ERR_NULL;
    const int dt = nccl_dtype(dtype);
    if (dt < 0) return MT_ERR_DTYPE;
    int rc = ensure_loaded();
    if (rc != MT_OK) return rc;
    return g_api.AllReduce(sendbuff, recvbuff, count, dt, ncclSum, static_cast<ncclComm_t>(comm), static_cast<cudaStream_t>(stream)) == 0 ? MT_OK : MT_ERR_NCCL;
}

int nccl_broadcast(void* stream, void* comm, const void* sendbuff, void* recvbuff, size_t count, int dtype, int root) {
    if (!comm || !sendbuff || !recvbuff) return MT_ERR_NULL;
    const int dt = nccl_dtype(dtype);
    if (dt < 0) return MT_ERR_DTYPE;
    int rc = ensure_loaded();
    if (rc != MT_OK) return rc;
    return g_api.Broadcast(sendbuff, recvbuff, count, dt, root, static_cast<ncclComm_t>(comm), static_cast<cudaStream_t>(stream)) == 0 ? MT_OK : MT_ERR_NCCL;
}

}  // extern "C"

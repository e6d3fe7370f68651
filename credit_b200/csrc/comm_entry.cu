// The path's only collective behind the C ABI: the all-reduce of LayerNorm backward's dgamma/dbeta
// when the rows are sharded over the GPUs of a node (one process per GPU). The reference is
// single-device (device 0 is hard-coded, src/workloads/layernorm_backward.cu:443), so these entry
// points have no reference counterpart; they let a host that does not use torch.distributed finish
// the sharded call with NCCL on the same stream as the kernels, in place on the [2, cols] buffer
// the finishing kernel writes.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, which resolves to a copy the process has
// already loaded, e.g. PyTorch's, or to the system one): the library has no link-time dependency
// on it and every other entry point works where NCCL is absent.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <mutex>

#include "../../include/credit_b200.h"
#include "error_state.h"

namespace {

using credit::report_error;

// The few NCCL types and constants this file needs (public ABI of NCCL 2.x).
struct NcclUniqueId {
    char internal[128];
};
static_assert(sizeof(NcclUniqueId) == CREDIT_COMM_ID_BYTES, "credit_comm ids are NCCL unique ids");
using NcclComm = void*;
constexpr int kNcclSuccess = 0, kNcclFloat32 = 7, kNcclSum = 0;

struct NcclApi {
    bool tried = false;
    void* handle = nullptr;
    int (*get_unique_id)(NcclUniqueId*) = nullptr;
    int (*comm_init_rank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*comm_destroy)(NcclComm) = nullptr;
    int (*all_reduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*error_string)(int) = nullptr;
};
NcclApi g_nccl;
std::mutex g_nccl_mutex;

int load_nccl(NcclApi** out) {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (!g_nccl.tried) {
        g_nccl.tried = true;
        g_nccl.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.handle != nullptr) {
            g_nccl.get_unique_id = reinterpret_cast<decltype(g_nccl.get_unique_id)>(dlsym(g_nccl.handle, "ncclGetUniqueId"));
            g_nccl.comm_init_rank = reinterpret_cast<decltype(g_nccl.comm_init_rank)>(dlsym(g_nccl.handle, "ncclCommInitRank"));
            g_nccl.comm_destroy = reinterpret_cast<decltype(g_nccl.comm_destroy)>(dlsym(g_nccl.handle, "ncclCommDestroy"));
            g_nccl.all_reduce = reinterpret_cast<decltype(g_nccl.all_reduce)>(dlsym(g_nccl.handle, "ncclAllReduce"));
            g_nccl.error_string = reinterpret_cast<decltype(g_nccl.error_string)>(dlsym(g_nccl.handle, "ncclGetErrorString"));
        }
    }
    if (g_nccl.handle == nullptr || g_nccl.get_unique_id == nullptr || g_nccl.comm_init_rank == nullptr ||
        g_nccl.comm_destroy == nullptr || g_nccl.all_reduce == nullptr)
        return report_error(CREDIT_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded: %s",
                            g_nccl.handle == nullptr ? dlerror() : "a symbol is missing");
    *out = &g_nccl;
    return CREDIT_OK;
}

int nccl_fail(const NcclApi& api, int code, const char* what) {
    return report_error(CREDIT_ERR_CUDA, "%s: NCCL error %d (%s)", what, code,
                        api.error_string != nullptr ? api.error_string(code) : "?");
}

}  // namespace

struct credit_comm {
    NcclComm nccl = nullptr;
    int world_size = 0;
    int rank = 0;
    int device = 0;
};

extern "C" {

int credit_comm_get_unique_id(void* id_out) {
    if (id_out == nullptr) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "id_out is NULL");
    NcclApi* api = nullptr;
    int rc = load_nccl(&api);
    if (rc != CREDIT_OK) return rc;
    NcclUniqueId id;
    const int code = api->get_unique_id(&id);
    if (code != kNcclSuccess) return nccl_fail(*api, code, "ncclGetUniqueId");
    std::memcpy(id_out, &id, sizeof(id));
    return CREDIT_OK;
}

int credit_comm_init_rank(credit_comm** comm_out, int world_size, int rank, const void* id) {
    if (comm_out == nullptr || id == nullptr) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "comm_out and id must not be NULL");
    if (world_size < 1 || rank < 0 || rank >= world_size)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "rank %d outside a world of %d", rank, world_size);
    NcclApi* api = nullptr;
    int rc = load_nccl(&api);
    if (rc != CREDIT_OK) return rc;
    NcclUniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    credit_comm* comm = new credit_comm();
    comm->world_size = world_size;
    comm->rank = rank;
    cudaError_t err = cudaGetDevice(&comm->device);
    if (err != cudaSuccess) {
        delete comm;
        return report_error(CREDIT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(err));
    }
    const int code = api->comm_init_rank(&comm->nccl, world_size, uid, rank);
    if (code != kNcclSuccess) {
        delete comm;
        return nccl_fail(*api, code, "ncclCommInitRank");
    }
    *comm_out = comm;
    return CREDIT_OK;
}

int credit_comm_destroy(credit_comm* comm) {
    if (comm == nullptr) return CREDIT_OK;
    NcclApi* api = nullptr;
    int rc = load_nccl(&api);
    if (rc == CREDIT_OK && comm->nccl != nullptr) {
        const int code = api->comm_destroy(comm->nccl);
        if (code != kNcclSuccess) rc = nccl_fail(*api, code, "ncclCommDestroy");
    }
    delete comm;
    return rc;
}

int credit_layernorm_bwd_allreduce(credit_comm* comm, float* dgamma_dbeta, int64_t cols, void* stream) {
    if (comm == nullptr || comm->nccl == nullptr) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "comm is NULL");
    if (dgamma_dbeta == nullptr || cols < 1 || cols > (1ll << 30))
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "dgamma_dbeta must be a [2, cols] buffer, cols in [1, 2^30]");
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return report_error(CREDIT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(err));
    if (device != comm->device)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "the communicator belongs to device %d, the current device is %d",
                            comm->device, device);
    if (comm->world_size == 1) return CREDIT_OK;   // nothing to add
    NcclApi* api = nullptr;
    int rc = load_nccl(&api);
    if (rc != CREDIT_OK) return rc;
    const int code = api->all_reduce(dgamma_dbeta, dgamma_dbeta, static_cast<size_t>(2 * cols), kNcclFloat32, kNcclSum,
                                     comm->nccl, static_cast<cudaStream_t>(stream));
    if (code != kNcclSuccess) return nccl_fail(*api, code, "ncclAllReduce");
    return CREDIT_OK;
}

}  // extern "C"

// NCCL behind plain C functions, for the vocabulary-sharded mode's one exchange.
//
// The library is not linked against NCCL: libnccl.so.2 is opened when the first
// communicator is asked for (a process that already holds one -- PyTorch's -- shares it),
// so a host that never uses more than one GPU needs no NCCL at all.  Communicators are
// created non-blocking and every call that may wait on another rank is polled against a
// deadline; when the deadline passes the communicator is aborted, which also ends a
// collective kernel that spins on the GPU for a rank that never came.  The reference does
// the same on its TCP fabric: a fixed deadline on the slices' partials turns a missing one
// into FG_ERR_LIMIT (src/runtime.c:2379-2435).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "fg_kernels.h"

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int *) = nullptr;
};

NcclApi api;

double now_ms() {
    timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return 1e3 * (double)t.tv_sec + 1e-6 * (double)t.tv_nsec;
}

void nap() {
    timespec t = {0, 50 * 1000};  // 50 us
    nanosleep(&t, nullptr);
}

template <typename F>
bool bind(F &slot, const char *name) {
    slot = reinterpret_cast<F>(dlsym(api.handle, name));
    return slot != nullptr;
}

// Waits until the communicator's pending call has gone through, or the deadline passes.
int settle(ncclComm_t comm, ncclResult_t first, double deadline) {
    ncclResult_t state = first;
    while (state == ncclInProgress) {
        if (now_ms() > deadline) return FGK_NCCL_TIMEOUT;
        nap();
        if (api.CommGetAsyncError(comm, &state) != ncclSuccess) return FGK_NCCL_FAILED;
    }
    return state == ncclSuccess ? 0 : FGK_NCCL_FAILED;
}

}  // namespace

extern "C" int fgk_nccl_load(void) {
    if (api.handle) return 0;
    const char *named = getenv("FG_NCCL_LIBRARY");
    void *handle = dlopen(named && *named ? named : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!handle) return FGK_NCCL_MISSING;
    api.handle = handle;
    const bool ok = bind(api.GetUniqueId, "ncclGetUniqueId") &&
                    bind(api.CommInitRankConfig, "ncclCommInitRankConfig") &&
                    bind(api.CommGetAsyncError, "ncclCommGetAsyncError") &&
                    bind(api.AllGather, "ncclAllGather") && bind(api.CommDestroy, "ncclCommDestroy") &&
                    bind(api.CommAbort, "ncclCommAbort") && bind(api.GetErrorString, "ncclGetErrorString") &&
                    bind(api.GetVersion, "ncclGetVersion");
    if (!ok) {
        dlclose(handle);
        api = NcclApi();
        return FGK_NCCL_MISSING;
    }
    return 0;
}

extern "C" int fgk_nccl_version(void) {
    int version = 0;
    if (fgk_nccl_load() != 0 || api.GetVersion(&version) != ncclSuccess) return 0;
    return version;
}

extern "C" int fgk_nccl_unique_id(void *id128) {
    static_assert(sizeof(ncclUniqueId) == FGK_NCCL_ID_BYTES, "unique id size");
    const int loaded = fgk_nccl_load();
    if (loaded) return loaded;
    return api.GetUniqueId(static_cast<ncclUniqueId *>(id128)) == ncclSuccess ? 0 : FGK_NCCL_FAILED;
}

extern "C" int fgk_nccl_create(void **comm_out, uint32_t ranks, uint32_t rank, const void *id128,
                               uint32_t timeout_ms) {
    const int loaded = fgk_nccl_load();
    if (loaded) return loaded;
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 0;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t comm = nullptr;
    const double deadline = now_ms() + timeout_ms;
    ncclResult_t first = api.CommInitRankConfig(&comm, (int)ranks, id, (int)rank, &config);
    if (first != ncclSuccess && first != ncclInProgress) return FGK_NCCL_FAILED;
    const int settled = settle(comm, first, deadline);
    if (settled != 0) {
        if (comm) api.CommAbort(comm);
        return settled;
    }
    *comm_out = comm;
    return 0;
}

extern "C" int fgk_nccl_all_gather(void *comm, const void *send, void *receive, size_t bytes_per_rank,
                                   void *stream, uint32_t timeout_ms) {
    ncclComm_t c = static_cast<ncclComm_t>(comm);
    const double deadline = now_ms() + timeout_ms;
    const ncclResult_t first =
        api.AllGather(send, receive, bytes_per_rank, ncclChar, c, static_cast<cudaStream_t>(stream));
    if (first != ncclSuccess && first != ncclInProgress) return FGK_NCCL_FAILED;
    return settle(c, first, deadline);
}

extern "C" void fgk_nccl_abort(void *comm) {
    if (comm && api.handle) api.CommAbort(static_cast<ncclComm_t>(comm));
}

extern "C" void fgk_nccl_destroy(void *comm) {
    if (comm && api.handle) api.CommDestroy(static_cast<ncclComm_t>(comm));
}

// Waits for the stream like cudaStreamSynchronize, but gives up at the deadline.
// Returns 0, a cudaError_t, or FGK_NCCL_TIMEOUT.
extern "C" int fgk_stream_wait_deadline(void *stream, uint32_t timeout_ms) {
    const double deadline = now_ms() + timeout_ms;
    for (;;) {
        const cudaError_t state = cudaStreamQuery(static_cast<cudaStream_t>(stream));
        if (state == cudaSuccess) return 0;
        if (state != cudaErrorNotReady) return (int)state;
        if (now_ms() > deadline) return FGK_NCCL_TIMEOUT;
        nap();
    }
}

extern "C" int fgk_ipc_handle(void *device_pointer, void *handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == FGK_IPC_HANDLE_BYTES, "IPC handle size");
    return (int)cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle64), device_pointer);
}

extern "C" int fgk_ipc_open(const void *handle64, void **device_pointer) {
    cudaIpcMemHandle_t handle;
    memcpy(&handle, handle64, sizeof(handle));
    return (int)cudaIpcOpenMemHandle(device_pointer, handle, cudaIpcMemLazyEnablePeerAccess);
}

extern "C" int fgk_ipc_close(void *device_pointer) { return (int)cudaIpcCloseMemHandle(device_pointer); }

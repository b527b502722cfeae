// Plumbing for the mailboxes of sharded runs: device allocation and CUDA IPC handles (the only entry points of the library
// that allocate).  The exchange itself lives in the norm kernel that consumes the summed vector (pi_dense.cu).
#include "pi_common.cuh"
#include <cstring>

using namespace pi;

extern "C" {
#pragma GCC visibility push(default)

int pi_device_malloc(void ** ptr, size_t bytes) {
    PI_REQUIRE(ptr && bytes > 0, "device_malloc: bad arguments");
    PI_CUDA(cudaMalloc(ptr, bytes));
    PI_CUDA(cudaMemset(*ptr, 0, bytes));
    return PI_OK;
}
int pi_device_free(void * ptr) { PI_CUDA(cudaFree(ptr)); return PI_OK; }

int pi_ipc_export(void * ptr, void * host_handle64) {
    PI_REQUIRE(ptr && host_handle64, "ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    PI_CUDA(cudaIpcGetMemHandle((cudaIpcMemHandle_t *)host_handle64, ptr));
    return PI_OK;
}
int pi_ipc_import(const void * host_handle64, void ** ptr) {
    PI_REQUIRE(ptr && host_handle64, "ipc_import: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, host_handle64, sizeof h);
    PI_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return PI_OK;
}
int pi_ipc_close(void * ptr) { PI_CUDA(cudaIpcCloseMemHandle(ptr)); return PI_OK; }

#pragma GCC visibility pop
}

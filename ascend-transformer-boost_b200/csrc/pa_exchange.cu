// Peer-memory plumbing of the sharded decode step: device buffers that the other processes of the
// node map through CUDA IPC.  With kv heads sharded over the GPUs, every rank's attention kernel
// stores its output rows straight into the gathered output buffer of every rank (plain stores to
// peer-mapped memory over NVLink) and the last CTA of the kernel publishes / awaits per-rank
// completion flags kept in such a buffer (see pa_exchange.cuh).
#include <cuda_runtime.h>
#include <cstring>
#include "../../include/atb_b200.h"

extern "C" {

int atb_b200_peer_buffer_create(uint64_t bytes, void **local_ptr, uint8_t handle[64])
{
    if (local_ptr == nullptr || handle == nullptr || bytes == 0) {
        return 1;
    }
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        return 26; // ERROR_OUT_OF_DEVICE_MEMORY
    }
    if (cudaMemset(p, 0, bytes) != cudaSuccess) {
        cudaFree(p);
        return 4;
    }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaFree(p);
        return 4;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    std::memcpy(handle, &h, 64);
    *local_ptr = p;
    return 0;
}

int atb_b200_peer_buffer_open(const uint8_t handle[64], void **peer_ptr)
{
    if (handle == nullptr || peer_ptr == nullptr) {
        return 1;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    return cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : 4;
}

int atb_b200_peer_buffer_close(void *peer_ptr) { return cudaIpcCloseMemHandle(peer_ptr) == cudaSuccess ? 0 : 4; }

int atb_b200_peer_buffer_destroy(void *local_ptr) { return cudaFree(local_ptr) == cudaSuccess ? 0 : 4; }

} // extern "C"

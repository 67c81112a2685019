// Exchange buffers of the tensor-parallel layer: allocation and CUDA IPC mapping between the
// one-process-per-GPU ranks of a node.  Set-up calls (not on the decode path); the kernels that
// use the buffers are in linear_stream.cu.
#include <cstring>

#include "common.cuh"

using namespace alloyb;

extern "C" size_t alloyb_tp_buffer_bytes(int max_n) {
    if (max_n <= 0) return 0;
    return 8448 + static_cast<size_t>(2) * 8 * max_n * sizeof(float);
}

extern "C" int alloyb_tp_alloc(size_t bytes, void** out) {
    if (!out || bytes == 0) return ALLOYB_E_NULL;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        set_cuda_error(e);
        return ALLOYB_E_CUDA;
    }
    *out = p;
    return ALLOYB_OK;
}

extern "C" int alloyb_tp_free(void* p) {
    if (!p) return ALLOYB_OK;
    const cudaError_t e = cudaFree(p);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

extern "C" int alloyb_tp_ipc_export(void* p, void* handle64) {
    if (!p || !handle64) return ALLOYB_E_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    const cudaError_t e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

extern "C" int alloyb_tp_ipc_import(const void* handle64, void** out) {
    if (!handle64 || !out) return ALLOYB_E_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    *out = p;
    return ALLOYB_OK;
}

extern "C" int alloyb_tp_ipc_close(void* p) {
    if (!p) return ALLOYB_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(p);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

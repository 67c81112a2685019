// Library-level entry points: version, error text, device check.
#include "common.cuh"

namespace alloyb {

static thread_local int g_last_cuda_error = 0;

void set_cuda_error(cudaError_t e) { g_last_cuda_error = static_cast<int>(e); }

int check_launch() {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_cuda_error(e);
        return ALLOYB_E_CUDA;
    }
    return ALLOYB_OK;
}

}  // namespace alloyb

extern "C" int alloyb_version(void) { return 1; }

extern "C" const char* alloyb_error_string(int code) {
    switch (code) {
        case ALLOYB_OK: return "ok";
        case ALLOYB_E_SHAPE: return "unsupported shape or size";
        case ALLOYB_E_ALIGN: return "pointer or row pitch misaligned";
        case ALLOYB_E_DTYPE: return "unsupported element type";
        case ALLOYB_E_NULL: return "null pointer";
        case ALLOYB_E_CUDA: return "CUDA runtime error";
        case ALLOYB_E_WORKSPACE: return "workspace too small";
        case ALLOYB_E_DEVICE: return "device-side bounded wait ran out";
        case ALLOYB_E_LIMIT: return "size exceeds a fixed maximum";
        default: return "unknown error";
    }
}

extern "C" int alloyb_last_cuda_error(void) { return alloyb::g_last_cuda_error; }

extern "C" int alloyb_device_supported(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
    return major == 10;
}

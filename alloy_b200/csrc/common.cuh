// Shared device/host helpers of the alloy_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/alloy_b200.h"

namespace alloyb {

constexpr int ALLOYB_NOT_TAKEN = 1;    // a fast path declined the shape: nothing was launched, take the general one


constexpr int QK_K = 256;
constexpr int Q4K_BYTES = 144;
constexpr int Q6K_BYTES = 210;
constexpr int Q8_BLOCK = 32;
constexpr int KV_BLOCK_BYTES = 34;   // fp16 scale + 32 int8 codes
constexpr int PAGE_TOKENS = 16;

// ---- per-thread error bookkeeping (host) --------------------------------------------------
void set_cuda_error(cudaError_t e);
int check_launch();   // cudaGetLastError -> ALLOYB_OK / ALLOYB_E_CUDA

// ---- element load/store by storage type ---------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float half_bits_to_f32(uint32_t bits16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

// Q4_K: 6-bit scale and min of sub-block g from the 12 packed bytes (as three words).
// Bytes 0-3: low six bits = scales 0-3, top two = high bits of scales 4-7;
// bytes 4-7: same for mins; bytes 8-11: low nibble = scales 4-7 low, high nibble = mins 4-7 low.
__device__ __forceinline__ void q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int g,
                                              int& sc, int& mn) {
    const int sh = (g & 3) * 8;
    const uint32_t a = (s0 >> sh) & 0xffu;
    const uint32_t b = (s1 >> sh) & 0xffu;
    if (g < 4) {
        sc = a & 63;
        mn = b & 63;
    } else {
        const uint32_t c = (s2 >> sh) & 0xffu;
        sc = (c & 15) | ((a >> 6) << 4);
        mn = (c >> 4) | ((b >> 6) << 4);
    }
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue early / wait for the previous kernel's memory to be visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Launch with programmatic stream serialization allowed: the kernel may begin while its
// predecessor in the stream is still running, and touches that predecessor's data only after
// pdl_wait().  Every kernel of the library calls pdl_launch_dependents() on entry, so a chain
// of small kernels overlaps each one's launch and prologue with the tail of the one before.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace alloyb

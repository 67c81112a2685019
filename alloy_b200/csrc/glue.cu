// Small element-wise / reduction ops of the decode step: RMSNorm, RoPE, SiLU*up, argmax.
#include "common.cuh"

namespace alloyb {

template <typename T>
__global__ void __launch_bounds__(256) rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                       T* __restrict__ y, int K, float eps) {
    __shared__ float red[8];
    const int row = blockIdx.x;
    const T* xr = x + static_cast<int64_t>(row) * K;
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < K; i += 256) {
        const float v = to_f32<T>(xr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float r = rsqrtf(tot / static_cast<float>(K) + eps);
    T* yr = y + static_cast<int64_t>(row) * K;
    for (int i = threadIdx.x; i < K; i += 256) {
        const T normed = from_f32<T>(to_f32<T>(xr[i]) * r);          // narrow before the weight
        yr[i] = from_f32<T>(to_f32<T>(w[i]) * to_f32<T>(normed));
    }
}

// One thread per (row, j < D/2): rows = B*H of q then B*KV_H of k.
template <typename T>
__global__ void rope_kernel(T* __restrict__ q, T* __restrict__ k, const int32_t* __restrict__ pos,
                            int pos_count, const float* __restrict__ inv_freq, int B, int H, int KV_H,
                            int D) {
    const int half = D / 2;
    const int64_t total = static_cast<int64_t>(B) * (H + KV_H) * half;
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= total) return;
    pdl_wait();
    const int j = static_cast<int>(i % half);
    const int64_t row = i / half;
    const int b = static_cast<int>(row / (H + KV_H));
    const int hh = static_cast<int>(row % (H + KV_H));
    T* base = (hh < H) ? q + (static_cast<int64_t>(b) * H + hh) * D
                       : k + (static_cast<int64_t>(b) * KV_H + (hh - H)) * D;
    const float angle = static_cast<float>(pos[pos_count == 1 ? 0 : b]) * inv_freq[j];
    float s, c;
    sincosf(angle, &s, &c);
    const float x1 = to_f32<T>(base[j]);
    const float x2 = to_f32<T>(base[j + half]);
    base[j] = from_f32<T>(x1 * c - x2 * s);
    base[j + half] = from_f32<T>(x2 * c + x1 * s);
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ y,
                                int64_t n) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    pdl_wait();
    const float gv = to_f32<T>(g[i]);
    y[i] = from_f32<T>(gv / (1.0f + expf(-gv)) * to_f32<T>(u[i]));
}

template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ logits,
                                                      int64_t* __restrict__ out, int N) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const T* row = logits + static_cast<int64_t>(blockIdx.x) * N;
    pdl_wait();
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float v = to_f32<T>(row[i]);
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? bv[threadIdx.x] : -INFINITY;
        idx = threadIdx.x < nw ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = idx;
    }
}

}  // namespace alloyb

using namespace alloyb;

extern "C" int alloyb_rms_norm(const void* x, const void* weight, void* y, int M, int K, float eps,
                               int dtype, void* stream) {
    if (!x || !weight || !y) return ALLOYB_E_NULL;
    if (M < 0 || K <= 0) return ALLOYB_E_SHAPE;
    if (M == 0) return ALLOYB_OK;
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case ALLOYB_F16:
            rms_norm_kernel<__half><<<M, 256, 0, st>>>(static_cast<const __half*>(x),
                                                       static_cast<const __half*>(weight),
                                                       static_cast<__half*>(y), K, eps);
            break;
        case ALLOYB_BF16:
            rms_norm_kernel<__nv_bfloat16><<<M, 256, 0, st>>>(
                static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight),
                static_cast<__nv_bfloat16*>(y), K, eps);
            break;
        case ALLOYB_F32:
            rms_norm_kernel<float><<<M, 256, 0, st>>>(static_cast<const float*>(x),
                                                      static_cast<const float*>(weight),
                                                      static_cast<float*>(y), K, eps);
            break;
        default: return ALLOYB_E_DTYPE;
    }
    return check_launch();
}

extern "C" int alloyb_rope_inplace(void* q, void* k, const int32_t* pos, int pos_count,
                                   const float* inv_freq, int B, int H, int KV_H, int D, int dtype,
                                   void* stream) {
    if (!q || !k || !pos || !inv_freq) return ALLOYB_E_NULL;
    if (B <= 0 || H <= 0 || KV_H < 0 || D <= 0 || D % 2) return ALLOYB_E_SHAPE;
    if (pos_count != 1 && pos_count != B) return ALLOYB_E_SHAPE;
    const int64_t total = static_cast<int64_t>(B) * (H + KV_H) * (D / 2);
    const int blocks = static_cast<int>((total + 255) / 256);
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case ALLOYB_F16:
            rope_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<__half*>(q), static_cast<__half*>(k),
                                                        pos, pos_count, inv_freq, B, H, KV_H, D);
            break;
        case ALLOYB_BF16:
            rope_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
                static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), pos, pos_count,
                inv_freq, B, H, KV_H, D);
            break;
        case ALLOYB_F32:
            rope_kernel<float><<<blocks, 256, 0, st>>>(static_cast<float*>(q), static_cast<float*>(k),
                                                       pos, pos_count, inv_freq, B, H, KV_H, D);
            break;
        default: return ALLOYB_E_DTYPE;
    }
    return check_launch();
}

extern "C" int alloyb_silu_mul(const void* gate, const void* up, void* y, int64_t n, int dtype,
                               void* stream) {
    if (!gate || !up || !y) return ALLOYB_E_NULL;
    if (n < 0) return ALLOYB_E_SHAPE;
    if (n == 0) return ALLOYB_OK;
    const int64_t blocks = (n + 255) / 256;
    if (blocks > 0x7fffffff) return ALLOYB_E_SHAPE;
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case ALLOYB_F16:
            silu_mul_kernel<__half><<<static_cast<int>(blocks), 256, 0, st>>>(
                static_cast<const __half*>(gate), static_cast<const __half*>(up),
                static_cast<__half*>(y), n);
            break;
        case ALLOYB_BF16:
            silu_mul_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
                static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
                static_cast<__nv_bfloat16*>(y), n);
            break;
        case ALLOYB_F32:
            silu_mul_kernel<float><<<static_cast<int>(blocks), 256, 0, st>>>(
                static_cast<const float*>(gate), static_cast<const float*>(up),
                static_cast<float*>(y), n);
            break;
        default: return ALLOYB_E_DTYPE;
    }
    return check_launch();
}

extern "C" int alloyb_argmax(const void* logits, int64_t* out_ids, int M, int N, int dtype,
                             void* stream) {
    if (!logits || !out_ids) return ALLOYB_E_NULL;
    if (M < 0 || N <= 0) return ALLOYB_E_SHAPE;
    if (M == 0) return ALLOYB_OK;
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case ALLOYB_F16:
            argmax_kernel<__half><<<M, 1024, 0, st>>>(static_cast<const __half*>(logits), out_ids, N);
            break;
        case ALLOYB_BF16:
            argmax_kernel<__nv_bfloat16><<<M, 1024, 0, st>>>(
                static_cast<const __nv_bfloat16*>(logits), out_ids, N);
            break;
        case ALLOYB_F32:
            argmax_kernel<float><<<M, 1024, 0, st>>>(static_cast<const float*>(logits), out_ids, N);
            break;
        default: return ALLOYB_E_DTYPE;
    }
    return check_launch();
}

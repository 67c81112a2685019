// Small element-wise / reduction ops of the decode step: RMSNorm, RoPE, SiLU*up, argmax.
#include "common.cuh"

namespace alloyb {

// One CTA per row.  fp32 sum of squares; x * r is narrowed to T before the weight multiplies it
// (the reference's rounding points, metal/std/norm.py:58-73).  VEC: 16-byte loads of a row that
// is 16-byte aligned with K a multiple of 8 (2-byte types), the row kept in registers between
// the two passes when it fits (K <= 8 * blockDim).
template <typename T, bool VEC>
__global__ void __launch_bounds__(1024) rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                        T* __restrict__ y, int K, float eps) {
    pdl_launch_dependents();
    __shared__ float red[32];
    const int row = blockIdx.x;
    const T* xr = x + static_cast<int64_t>(row) * K;
    T* yr = y + static_cast<int64_t>(row) * K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    pdl_wait();
    float ss = 0.f;
    uint4 keep = make_uint4(0u, 0u, 0u, 0u);
    if (VEC) {
        for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
            if (i == static_cast<int>(threadIdx.x) * 8) keep = v;
            const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = to_f32<T>(e[j]);
                ss = fmaf(f, f, ss);
            }
        }
    } else {
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            const float v = to_f32<T>(xr[i]);
            ss = fmaf(v, v, ss);
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < nw; ++i) tot += red[i];
    const float r = rsqrtf(tot / static_cast<float>(K) + eps);
    if (VEC) {
        for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8) {
            const uint4 v = (i == static_cast<int>(threadIdx.x) * 8) ? keep : *reinterpret_cast<const uint4*>(xr + i);
            const uint4 wv = *reinterpret_cast<const uint4*>(w + i);
            const T* e = reinterpret_cast<const T*>(&v);
            const T* we = reinterpret_cast<const T*>(&wv);
            uint4 o;
            T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const T normed = from_f32<T>(to_f32<T>(e[j]) * r);      // narrow before the weight
                oe[j] = from_f32<T>(to_f32<T>(we[j]) * to_f32<T>(normed));
            }
            *reinterpret_cast<uint4*>(yr + i) = o;
        }
    } else {
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            const T normed = from_f32<T>(to_f32<T>(xr[i]) * r);          // narrow before the weight
            yr[i] = from_f32<T>(to_f32<T>(w[i]) * to_f32<T>(normed));
        }
    }
}

template <typename T>
static cudaError_t launch_rms_norm(const void* x, const void* w, void* y, int M, int K, float eps, cudaStream_t st) {
    const bool vec = sizeof(T) == 2 && K % 8 == 0 &&
                     (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) % 16 == 0;
    if (vec) {
        int threads = (K / 8 + 31) / 32 * 32;
        if (threads > 1024) threads = 1024;
        return launch_pdl(rms_norm_kernel<T, true>, dim3(M), dim3(threads), 0, st, static_cast<const T*>(x),
                          static_cast<const T*>(w), static_cast<T*>(y), K, eps);
    }
    return launch_pdl(rms_norm_kernel<T, false>, dim3(M), dim3(256), 0, st, static_cast<const T*>(x),
                      static_cast<const T*>(w), static_cast<T*>(y), K, eps);
}

// One thread per (row, j < D/2): rows = B*H of q then B*KV_H of k.
template <typename T>
__global__ void rope_kernel(T* __restrict__ q, T* __restrict__ k, const int32_t* __restrict__ pos,
                            int pos_count, const float* __restrict__ inv_freq, int B, int H, int KV_H,
                            int D) {
    pdl_launch_dependents();
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
    // two rounded products and one rounded sum, never a fused multiply-add: the same fp32 sequence
    // as the element-wise reference (and as the fused RoPE + append kernel)
    base[j] = from_f32<T>(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
    base[j + half] = from_f32<T>(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)));
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ y,
                                int64_t n) {
    pdl_launch_dependents();
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    pdl_wait();
    const float gv = to_f32<T>(g[i]);
    y[i] = from_f32<T>(gv / (1.0f + expf(-gv)) * to_f32<T>(u[i]));
}

// The same, eight 16-bit elements per thread (16-byte loads and stores): the large activations of a prefill
// chunk are bound by bandwidth, which one element per thread does not reach.
template <typename T>
__global__ void silu_mul_vec8_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ y, int64_t n8) {
    pdl_launch_dependents();
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n8) return;
    pdl_wait();
    const uint4 gv = __ldg(reinterpret_cast<const uint4*>(g) + i), uv = __ldg(reinterpret_cast<const uint4*>(u) + i);
    const T* gh = reinterpret_cast<const T*>(&gv);
    const T* uh = reinterpret_cast<const T*>(&uv);
    uint4 out;
    T* oh = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float x = to_f32<T>(gh[e]);
        oh[e] = from_f32<T>(x / (1.0f + expf(-x)) * to_f32<T>(uh[e]));
    }
    reinterpret_cast<uint4*>(y)[i] = out;
}

// Greedy argmax of one row by a cluster of eight CTAs: every CTA scans an eighth of the row, the
// eight (value, index) candidates meet in CTA 0 through distributed shared memory.  Ties go to
// the smallest index.
constexpr int ARGMAX_CLUSTER = 8;

__device__ __forceinline__ void argmax_take(float& best, int& idx, float ov, int oi) {
    if (ov > best || (ov == best && oi < idx)) {
        best = ov;
        idx = oi;
    }
}

template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ logits, int64_t* __restrict__ out, int N) {
    pdl_launch_dependents();
    __shared__ float bv[32];
    __shared__ int bi[32];
    __shared__ float c_val;
    __shared__ int c_idx;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const T* row = logits + static_cast<int64_t>(blockIdx.y) * N;
    const int chunk = (N + ARGMAX_CLUSTER - 1) / ARGMAX_CLUSTER;
    const int lo = static_cast<int>(rank) * chunk;
    const int hi = lo + chunk < N ? lo + chunk : N;
    pdl_wait();
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_take(best, idx, to_f32<T>(row[i]), i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_take(best, idx, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? bv[threadIdx.x] : -INFINITY;
        idx = threadIdx.x < nw ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            argmax_take(best, idx, ov, oi);
        }
        if (threadIdx.x == 0) {
            c_val = best;
            c_idx = idx;
        }
    }
    // every CTA's candidate is written; CTA 0 reads all eight through the cluster's shared window
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank == 0 && threadIdx.x < 32) {
        best = -INFINITY;
        idx = 0x7fffffff;
        if (threadIdx.x < ARGMAX_CLUSTER) {
            uint32_t va, ia;
            const uint32_t lv = static_cast<uint32_t>(__cvta_generic_to_shared(&c_val));
            const uint32_t li = static_cast<uint32_t>(__cvta_generic_to_shared(&c_idx));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(va) : "r"(lv), "r"(threadIdx.x));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ia) : "r"(li), "r"(threadIdx.x));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(best) : "r"(va));
            asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(idx) : "r"(ia));
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            argmax_take(best, idx, ov, oi);
        }
        if (threadIdx.x == 0) out[blockIdx.y] = idx;
    }
    // nobody leaves while CTA 0 may still read its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <typename T>
static cudaError_t launch_argmax(const void* logits, int64_t* out, int M, int N, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ARGMAX_CLUSTER, M);
    cfg.blockDim = dim3(1024);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ARGMAX_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, argmax_kernel<T>, static_cast<const T*>(logits), out, N);
}

}  // namespace alloyb

using namespace alloyb;

extern "C" int alloyb_rms_norm(const void* x, const void* weight, void* y, int M, int K, float eps,
                               int dtype, void* stream) {
    if (!x || !weight || !y) return ALLOYB_E_NULL;
    if (M < 0 || K <= 0) return ALLOYB_E_SHAPE;
    if (M == 0) return ALLOYB_OK;
    cudaStream_t st = as_stream(stream);
    cudaError_t e;
    switch (dtype) {
        case ALLOYB_F16: e = launch_rms_norm<__half>(x, weight, y, M, K, eps, st); break;
        case ALLOYB_BF16: e = launch_rms_norm<__nv_bfloat16>(x, weight, y, M, K, eps, st); break;
        case ALLOYB_F32: e = launch_rms_norm<float>(x, weight, y, M, K, eps, st); break;
        default: return ALLOYB_E_DTYPE;
    }
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
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
            launch_pdl(rope_kernel<__half>, dim3(blocks), dim3(256), 0, st, static_cast<__half*>(q), static_cast<__half*>(k),
                                                        pos, pos_count, inv_freq, B, H, KV_H, D);
            break;
        case ALLOYB_BF16:
            launch_pdl(rope_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st, 
                static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), pos, pos_count,
                inv_freq, B, H, KV_H, D);
            break;
        case ALLOYB_F32:
            launch_pdl(rope_kernel<float>, dim3(blocks), dim3(256), 0, st, static_cast<float*>(q), static_cast<float*>(k),
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
    if (dtype != ALLOYB_F32 && n % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
        const int64_t n8 = n / 8;
        const dim3 grid(static_cast<unsigned int>((n8 + 255) / 256));
        if (dtype == ALLOYB_F16)
            launch_pdl(silu_mul_vec8_kernel<__half>, grid, dim3(256), 0, st, static_cast<const __half*>(gate),
                       static_cast<const __half*>(up), static_cast<__half*>(y), n8);
        else if (dtype == ALLOYB_BF16)
            launch_pdl(silu_mul_vec8_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, static_cast<const __nv_bfloat16*>(gate),
                       static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(y), n8);
        else
            return ALLOYB_E_DTYPE;
        return check_launch();
    }
    switch (dtype) {
        case ALLOYB_F16:
            launch_pdl(silu_mul_kernel<__half>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, 
                static_cast<const __half*>(gate), static_cast<const __half*>(up),
                static_cast<__half*>(y), n);
            break;
        case ALLOYB_BF16:
            launch_pdl(silu_mul_kernel<__nv_bfloat16>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, 
                static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
                static_cast<__nv_bfloat16*>(y), n);
            break;
        case ALLOYB_F32:
            launch_pdl(silu_mul_kernel<float>, dim3(static_cast<int>(blocks)), dim3(256), 0, st, 
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
    cudaError_t e;
    switch (dtype) {
        case ALLOYB_F16: e = launch_argmax<__half>(logits, out_ids, M, N, st); break;
        case ALLOYB_BF16: e = launch_argmax<__nv_bfloat16>(logits, out_ids, M, N, st); break;
        case ALLOYB_F32: e = launch_argmax<float>(logits, out_ids, M, N, st); break;
        default: return ALLOYB_E_DTYPE;
    }
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return check_launch();
}

// Formats and ops adjacent to the Q4_K / Q6_K path that share its row decoders:
//   * Q5_0 in the reference's normalised three-buffer form (server/gguf/quant.py:414-490):
//     qweight (N, K/2) u8, byte k/2 = element k (low nibble) | element k+1 (high nibble);
//     qhigh (N, K/2) u8, bit 0 / bit 4 of byte k/2 = fifth bit of element k / k+1;
//     scales (N, K/32) fp16.  w = scale * ((nibble | fifth << 4) - 16).
//   * routed mixture-of-experts (torch/custom_ops.py:59-66; kernels metal/std/moe.py:31-228): top-k
//     router over raw logits with a softmax over the winners, gathered Q4_K gate/up GEMV with SiLU,
//     gathered Q6_K down GEMV with the routing-weighted sum over the slots.
// These are CUDA-core kernels (one warp per output row): the formats are not part of the Q4_K_M
// mixes the tensor-core kernels are built for.
#include "linear_rows.cuh"

namespace alloyb {
namespace q5 {

constexpr int ROWS_WARPS = 8;
constexpr int MT = 4;

// One warp per weight row; a lane takes whole 32-element blocks (16 + 16 packed bytes, one scale).
template <typename XT>
__global__ void __launch_bounds__(ROWS_WARPS * 32)
q5_0_rows_kernel(const XT* __restrict__ x, int M, int K, int N, const uint8_t* __restrict__ qw,
                 const uint8_t* __restrict__ qh, const __half* __restrict__ scales, XT* __restrict__ y) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * ROWS_WARPS + warp;
    if (row >= N) return;
    const int nblk = K / 32;
    const uint8_t* wr = qw + static_cast<int64_t>(row) * (K / 2);
    const uint8_t* hr = qh + static_cast<int64_t>(row) * (K / 2);
    const __half* sr = scales + static_cast<int64_t>(row) * nblk;
    pdl_wait();
    for (int m0 = 0; m0 < M; m0 += MT) {
        float acc[MT];
#pragma unroll
        for (int t = 0; t < MT; ++t) acc[t] = 0.f;
        for (int b = lane; b < nblk; b += 32) {
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + b * 16));
            const uint4 hv = __ldg(reinterpret_cast<const uint4*>(hr + b * 16));
            const float s = __half2float(__ldg(sr + b));
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, hw[4] = {hv.x, hv.y, hv.z, hv.w};
            float q[32];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t wb = (ww[i >> 2] >> (8 * (i & 3))) & 0xffu;
                const uint32_t hb = (hw[i >> 2] >> (8 * (i & 3))) & 0xffu;
                q[2 * i] = static_cast<float>(static_cast<int>((wb & 15u) | ((hb & 1u) << 4)) - 16);
                q[2 * i + 1] = static_cast<float>(static_cast<int>((wb >> 4) | (((hb >> 4) & 1u) << 4)) - 16);
            }
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                if (m0 + t < M) {
                    const XT* xr = x + static_cast<int64_t>(m0 + t) * K + b * 32;
                    float a = 0.f;
#pragma unroll
                    for (int e = 0; e < 32; ++e) a = fmaf(to_f32<XT>(xr[e]), q[e], a);
                    acc[t] = fmaf(s, a, acc[t]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            const float v = warp_sum(acc[t]);
            if (lane == 0 && m0 + t < M) y[static_cast<int64_t>(m0 + t) * N + row] = from_f32<XT>(v);
        }
    }
}

template <typename OT>
__global__ void q5_0_dequant_kernel(const uint8_t* __restrict__ qw, const uint8_t* __restrict__ qh,
                                    const __half* __restrict__ scales, const int64_t* __restrict__ ids,
                                    OT* __restrict__ out, int64_t n_rows, int64_t table_rows, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = n_rows * static_cast<int64_t>(K);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / K;
        const int c = static_cast<int>(i - r * K);
        const int64_t src = ids ? ids[r] : r;
        float w = 0.f;
        if (src >= 0 && src < table_rows) {
            const uint32_t wb = qw[src * (K / 2) + c / 2], hb = qh[src * (K / 2) + c / 2];
            const int sh = (c & 1) * 4;
            const int q = static_cast<int>(((wb >> sh) & 15u) | (((hb >> sh) & 1u) << 4)) - 16;
            w = __fmul_rn(__half2float(scales[src * (K / 32) + c / 32]), static_cast<float>(q));
        }
        out[i] = from_f32<OT>(w);
    }
}

// ---- routed experts ---------------------------------------------------------------------------

// One warp per token: the top_k largest logits in descending order (lowest index on ties) and the
// softmax over just those (metal/std/moe.py:31-80).
__global__ void moe_router_kernel(const float* __restrict__ logits, int* __restrict__ idx_out,
                                  float* __restrict__ w_out, int T, int E, int top_k) {
    pdl_launch_dependents();
    extern __shared__ float sl[];
    const int t = blockIdx.x, lane = threadIdx.x;
    pdl_wait();
    for (int e = lane; e < E; e += 32) sl[e] = logits[static_cast<int64_t>(t) * E + e];
    __syncwarp();
    float m0 = 0.f, sum = 0.f;
    float vals[32];
    for (int k = 0; k < top_k; ++k) {
        float best = -3.0e38f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = sl[e];
            if (v > best) { best = v; bi = e; }          // ascending e per lane: first maximum kept
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (k == 0) m0 = best;
        if (k < 32) vals[k] = best;
        if (lane == 0) {
            idx_out[t * top_k + k] = bi;
            sl[bi] = -3.0e38f;
        }
        __syncwarp();
    }
    for (int k = 0; k < top_k; ++k) sum += expf(vals[k] - m0);
    if (lane == 0)
        for (int k = 0; k < top_k; ++k) w_out[t * top_k + k] = expf(vals[k] - m0) / sum;
}

// One warp per (token-slot, intermediate channel): h = silu(x . gate_row) * (x . up_row) in fp32,
// gate row e*2I + c, up row e*2I + I + c of the fused (E, 2I, K/256*144) block tensor.
template <typename XT>
__global__ void __launch_bounds__(ROWS_WARPS * 32)
moe_gate_up_kernel(const XT* __restrict__ x, const uint8_t* __restrict__ gate_up, const int* __restrict__ routing,
                   float* __restrict__ h_out, int K, int I, int top_k, int num_experts) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ts = blockIdx.y, c = blockIdx.x * ROWS_WARPS + warp;
    if (c >= I) return;
    pdl_wait();
    const int e = routing[ts];
    float v = 0.f;
    if (e >= 0 && e < num_experts) {
        const int64_t rb = static_cast<int64_t>(K / QK_K) * Q4K_BYTES;
        const uint8_t* grow = gate_up + (static_cast<int64_t>(e) * 2 * I + c) * rb;
        const uint8_t* urow = grow + static_cast<int64_t>(I) * rb;
        const XT* xr = x + static_cast<int64_t>(ts / top_k) * K;
        float ag[1] = {0.f}, au[1] = {0.f};
        row_dot_q4k<XT, 1>(grow, xr, K, K, 1, ag);
        row_dot_q4k<XT, 1>(urow, xr, K, K, 1, au);
        const float g = warp_sum(ag[0]), u = warp_sum(au[0]);
        v = act_silu(g) * u;
    }
    if (lane == 0) h_out[static_cast<int64_t>(ts) * I + c] = v;
}

// One warp per (token, hidden channel): y = sum over the slots of w_slot * (down[e_slot] row . h_slot).
__global__ void __launch_bounds__(ROWS_WARPS * 32)
moe_down_kernel(const float* __restrict__ h_in, const uint8_t* __restrict__ down, const int* __restrict__ routing,
                const float* __restrict__ weights, float* __restrict__ y, int H, int I, int top_k, int num_experts) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y, j = blockIdx.x * ROWS_WARPS + warp;
    if (j >= H) return;
    pdl_wait();
    const int64_t rb = static_cast<int64_t>(I / QK_K) * Q6K_BYTES;
    float acc = 0.f;
    for (int s = 0; s < top_k; ++s) {
        const int ts = t * top_k + s;
        const int e = routing[ts];
        if (e < 0 || e >= num_experts) continue;
        float a[1] = {0.f};
        row_dot_q6k<float, 1>(down + (static_cast<int64_t>(e) * H + j) * rb, h_in + static_cast<int64_t>(ts) * I, I, I, 1, a);
        acc = fmaf(weights[ts], a[0], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[static_cast<int64_t>(t) * H + j] = acc;
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace q5
}  // namespace alloyb

using namespace alloyb;

extern "C" int alloyb_q5_0_mm(const void* x, const void* qweight, const void* qhigh, const void* scales, void* y,
                              int M, int N, int K, int dtype, void* stream) {
    if (!x || !qweight || !qhigh || !scales || !y) return ALLOYB_E_NULL;
    if (M < 0 || N <= 0 || K <= 0 || K % 32) return ALLOYB_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(qweight) | reinterpret_cast<uintptr_t>(qhigh)) % 16) return ALLOYB_E_ALIGN;
    if (M == 0) return ALLOYB_OK;
    const int blocks = (N + q5::ROWS_WARPS - 1) / q5::ROWS_WARPS;
    cudaStream_t st = as_stream(stream);
    const uint8_t* w8 = static_cast<const uint8_t*>(qweight);
    const uint8_t* h8 = static_cast<const uint8_t*>(qhigh);
    const __half* sc = static_cast<const __half*>(scales);
    switch (dtype) {
        case ALLOYB_F16:
            launch_pdl(q5::q5_0_rows_kernel<__half>, dim3(blocks), dim3(q5::ROWS_WARPS * 32), 0, st,
                       static_cast<const __half*>(x), M, K, N, w8, h8, sc, static_cast<__half*>(y));
            break;
        case ALLOYB_BF16:
            launch_pdl(q5::q5_0_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(q5::ROWS_WARPS * 32), 0, st,
                       static_cast<const __nv_bfloat16*>(x), M, K, N, w8, h8, sc, static_cast<__nv_bfloat16*>(y));
            break;
        case ALLOYB_F32:
            launch_pdl(q5::q5_0_rows_kernel<float>, dim3(blocks), dim3(q5::ROWS_WARPS * 32), 0, st,
                       static_cast<const float*>(x), M, K, N, w8, h8, sc, static_cast<float*>(y));
            break;
        default:
            return ALLOYB_E_DTYPE;
    }
    return check_launch();
}

extern "C" int alloyb_dequant_q5_0(const void* qweight, const void* qhigh, const void* scales, const int64_t* ids,
                                   void* out, int64_t n_rows, int64_t table_rows, int K, int out_dtype,
                                   void* stream) {
    if (!qweight || !qhigh || !scales || !out) return ALLOYB_E_NULL;
    if (n_rows < 0 || table_rows <= 0 || K <= 0 || K % 32) return ALLOYB_E_SHAPE;
    if (n_rows == 0) return ALLOYB_OK;
    const int64_t total = n_rows * static_cast<int64_t>(K);
    const int64_t want = (total + 255) / 256;
    const int blocks = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
    cudaStream_t st = as_stream(stream);
    const uint8_t* w8 = static_cast<const uint8_t*>(qweight);
    const uint8_t* h8 = static_cast<const uint8_t*>(qhigh);
    const __half* sc = static_cast<const __half*>(scales);
    switch (out_dtype) {
        case ALLOYB_F32:
            launch_pdl(q5::q5_0_dequant_kernel<float>, dim3(blocks), dim3(256), 0, st, w8, h8, sc, ids,
                       static_cast<float*>(out), n_rows, table_rows, K);
            break;
        case ALLOYB_F16:
            launch_pdl(q5::q5_0_dequant_kernel<__half>, dim3(blocks), dim3(256), 0, st, w8, h8, sc, ids,
                       static_cast<__half*>(out), n_rows, table_rows, K);
            break;
        case ALLOYB_BF16:
            launch_pdl(q5::q5_0_dequant_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st, w8, h8, sc, ids,
                       static_cast<__nv_bfloat16*>(out), n_rows, table_rows, K);
            break;
        default:
            return ALLOYB_E_DTYPE;
    }
    return check_launch();
}

extern "C" size_t alloyb_moe_workspace_bytes(int T, int top_k, int moe_intermediate) {
    if (T <= 0 || top_k <= 0 || moe_intermediate <= 0) return 0;
    const size_t slots = static_cast<size_t>(T) * top_k;
    return 2 * q5::align256(slots * 4) + q5::align256(slots * moe_intermediate * 4);
}

extern "C" int alloyb_moe_routed(const void* hidden, int hidden_dtype, const float* router_logits,
                                 const void* gate_up_blocks, const void* down_qweight, float* out, int T, int H,
                                 int num_experts, int top_k, int moe_intermediate, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    if (!hidden || !router_logits || !gate_up_blocks || !down_qweight || !out || !workspace) return ALLOYB_E_NULL;
    if (T < 0 || H <= 0 || H % QK_K || moe_intermediate <= 0 || moe_intermediate % QK_K) return ALLOYB_E_SHAPE;
    if (num_experts <= 0 || num_experts > 8192 || top_k <= 0 || top_k > 32 || top_k > num_experts) return ALLOYB_E_SHAPE;
    if (reinterpret_cast<uintptr_t>(workspace) % 256) return ALLOYB_E_ALIGN;
    if ((reinterpret_cast<uintptr_t>(gate_up_blocks) % 4) || (reinterpret_cast<uintptr_t>(down_qweight) % 2))
        return ALLOYB_E_ALIGN;
    if (T == 0) return ALLOYB_OK;
    if (workspace_bytes < alloyb_moe_workspace_bytes(T, top_k, moe_intermediate)) return ALLOYB_E_WORKSPACE;
    const size_t slots = static_cast<size_t>(T) * top_k;
    if (slots > 65535) return ALLOYB_E_LIMIT;            // the slot index is a grid y coordinate
    char* ws = static_cast<char*>(workspace);
    int* idx = reinterpret_cast<int*>(ws);
    float* wts = reinterpret_cast<float*>(ws + q5::align256(slots * 4));
    float* h = reinterpret_cast<float*>(ws + 2 * q5::align256(slots * 4));
    cudaStream_t st = as_stream(stream);
    const int I = moe_intermediate;
    launch_pdl(q5::moe_router_kernel, dim3(T), dim3(32), static_cast<size_t>(num_experts) * 4, st, router_logits, idx,
               wts, T, num_experts, top_k);
    int rc = check_launch();
    if (rc != ALLOYB_OK) return rc;
    const dim3 g1((I + q5::ROWS_WARPS - 1) / q5::ROWS_WARPS, static_cast<unsigned>(slots));
    const uint8_t* gu = static_cast<const uint8_t*>(gate_up_blocks);
    switch (hidden_dtype) {
        case ALLOYB_F16:
            launch_pdl(q5::moe_gate_up_kernel<__half>, g1, dim3(q5::ROWS_WARPS * 32), 0, st,
                       static_cast<const __half*>(hidden), gu, static_cast<const int*>(idx), h, H, I, top_k, num_experts);
            break;
        case ALLOYB_BF16:
            launch_pdl(q5::moe_gate_up_kernel<__nv_bfloat16>, g1, dim3(q5::ROWS_WARPS * 32), 0, st,
                       static_cast<const __nv_bfloat16*>(hidden), gu, static_cast<const int*>(idx), h, H, I, top_k,
                       num_experts);
            break;
        case ALLOYB_F32:
            launch_pdl(q5::moe_gate_up_kernel<float>, g1, dim3(q5::ROWS_WARPS * 32), 0, st,
                       static_cast<const float*>(hidden), gu, static_cast<const int*>(idx), h, H, I, top_k, num_experts);
            break;
        default:
            return ALLOYB_E_DTYPE;
    }
    rc = check_launch();
    if (rc != ALLOYB_OK) return rc;
    const dim3 g2((H + q5::ROWS_WARPS - 1) / q5::ROWS_WARPS, T);
    launch_pdl(q5::moe_down_kernel, g2, dim3(q5::ROWS_WARPS * 32), 0, st, static_cast<const float*>(h),
               static_cast<const uint8_t*>(down_qweight), static_cast<const int*>(idx), static_cast<const float*>(wts), out,
               H, I, top_k, num_experts);
    return check_launch();
}

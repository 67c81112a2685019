// Warp-per-output-row dequant dot products on the CUDA cores.
//
// This is the shape-agnostic member of the quantised-linear family: any M, any
// K that is a whole number of blocks, any activation type, rows that are only
// 2-byte aligned (Q6_K).  The tensor-core GEMV (linear_mma.cu) and the tcgen05
// GEMM take the shapes they are built for; everything else lands here.
//
// One warp owns one weight row and MT activation rows at a time.  Per block the
// lanes split the packed bytes into 32 equal word-sized pieces, so every global
// load instruction of a warp covers one contiguous run of the row.
#pragma once
#include "common.cuh"

namespace alloyb {

// acc[t] += sum over this lane's share of row `w` against x rows m0..m0+MT-1.
template <typename XT, int MT>
__device__ __forceinline__ void row_dot_q4k(const uint8_t* __restrict__ w, const XT* __restrict__ x,
                                            int64_t ldx, int K, int m_left, float (&acc)[MT]) {
    const int lane = threadIdx.x & 31;
    const int gp = lane >> 3;             // sub-block pair 0..3
    const int l0 = (lane & 7) * 4;        // first of 4 elements inside the 32-wide sub-block
    const int nb = K / QK_K;
    for (int b = 0; b < nb; ++b) {
        const uint8_t* blk = w + static_cast<int64_t>(b) * Q4K_BYTES;
        const uint32_t* bw = reinterpret_cast<const uint32_t*>(blk);
        const uint32_t hdr = __ldg(bw);
        const uint32_t s0 = __ldg(bw + 1), s1 = __ldg(bw + 2), s2 = __ldg(bw + 3);
        const uint32_t qw = __ldg(bw + 4 + lane);
        const float d = half_bits_to_f32(hdr & 0xffffu);
        const float dmin = half_bits_to_f32(hdr >> 16);
        int sc_lo, mn_lo, sc_hi, mn_hi;
        q4k_scale_min(s0, s1, s2, 2 * gp, sc_lo, mn_lo);
        q4k_scale_min(s0, s1, s2, 2 * gp + 1, sc_hi, mn_hi);
        const float dl = d * static_cast<float>(sc_lo), dh = d * static_cast<float>(sc_hi);
        const float ml = dmin * static_cast<float>(mn_lo), mh = dmin * static_cast<float>(mn_hi);
        const int kbase = b * QK_K + gp * 64 + l0;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            if (t < m_left) {
                const XT* xr = x + t * ldx + kbase;
                float sl = 0.f, sh = 0.f, xl = 0.f, xh = 0.f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float a = to_f32<XT>(xr[e]);
                    const float c = to_f32<XT>(xr[32 + e]);
                    const uint32_t byte = (qw >> (8 * e)) & 0xffu;
                    sl = fmaf(a, static_cast<float>(byte & 15u), sl);
                    sh = fmaf(c, static_cast<float>(byte >> 4), sh);
                    xl += a;
                    xh += c;
                }
                acc[t] += dl * sl + dh * sh - ml * xl - mh * xh;
            }
        }
    }
}

template <typename XT, int MT>
__device__ __forceinline__ void row_dot_q6k(const uint8_t* __restrict__ w, const XT* __restrict__ x,
                                            int64_t ldx, int K, int m_left, float (&acc)[MT]) {
    const int lane = threadIdx.x & 31;
    const int h = lane >> 4;              // which 128-element half of the block
    const int lq = (lane & 15) * 2;       // first of 2 positions inside each 32-wide sub-block
    const int nb = K / QK_K;
    for (int b = 0; b < nb; ++b) {
        const uint8_t* blk = w + static_cast<int64_t>(b) * Q6K_BYTES;
        const uint16_t* b16 = reinterpret_cast<const uint16_t*>(blk);   // rows are 2-byte aligned
        const uint32_t qla = __ldg(b16 + (h * 64 + lq) / 2);
        const uint32_t qlb = __ldg(b16 + (h * 64 + 32 + lq) / 2);
        const uint32_t qh = __ldg(b16 + (128 + h * 32 + lq) / 2);
        const float d = half_bits_to_f32(__ldg(b16 + 104));
        const int8_t* sc8 = reinterpret_cast<const int8_t*>(blk + 192) + h * 8 + (lq >> 4);
        float wv[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float ds = d * static_cast<float>(__ldg(sc8 + 2 * j));
            const uint32_t qlw = (j & 1) ? qlb : qla;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t byte = (qlw >> (8 * e)) & 0xffu;
                const uint32_t nib = (j >= 2) ? (byte >> 4) : (byte & 15u);
                const uint32_t hi = (qh >> (8 * e + 2 * j)) & 3u;
                wv[j][e] = ds * static_cast<float>(static_cast<int>(nib | (hi << 4)) - 32);
            }
        }
        const int kbase = b * QK_K + h * 128 + lq;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            if (t < m_left) {
                const XT* xr = x + t * ldx + kbase;
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s = fmaf(to_f32<XT>(xr[j * 32]), wv[j][0], s);
                    s = fmaf(to_f32<XT>(xr[j * 32 + 1]), wv[j][1], s);
                }
                acc[t] += s;
            }
        }
    }
}

template <typename XT, int MT>
__device__ __forceinline__ void row_dot_q8_0(const int8_t* __restrict__ w,
                                             const __half* __restrict__ scales,
                                             const XT* __restrict__ x, int64_t ldx, int K,
                                             int m_left, float (&acc)[MT]) {
    const int lane = threadIdx.x & 31;
    for (int k0 = lane * 4; k0 < K; k0 += 128) {
        const uint32_t qw = __ldg(reinterpret_cast<const uint32_t*>(w + k0));
        const float s = __half2float(__ldg(scales + k0 / Q8_BLOCK));
#pragma unroll
        for (int t = 0; t < MT; ++t) {
            if (t < m_left) {
                const XT* xr = x + t * ldx + k0;
                float a = 0.f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int q = static_cast<int8_t>((qw >> (8 * e)) & 0xffu);
                    a = fmaf(to_f32<XT>(xr[e]), static_cast<float>(q), a);
                }
                acc[t] = fmaf(s, a, acc[t]);
            }
        }
    }
}

__device__ __forceinline__ float act_silu(float g) { return g / (1.0f + __expf(-g)); }
__device__ __forceinline__ float act_gelu_tanh(float g) {
    return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

}  // namespace alloyb

// Q8_0 dequant-GEMV for 1..4 tokens per pass (more tokens: more passes), plain and gate/up fused.
//
// Weights arrive in the reference's normalised pair (server/gguf/quant.py:497-521): int8 codes
// (N, K) and fp16 scales (N, K/32), w = scale * code; 1.0625 bytes per weight, so the kernel is a
// pure streaming problem like the Q4_K / Q6_K GEMVs, and follows the reference kernel's plan
// (metal/std/quant.py:61-273: split K over the lanes, several rows per SIMD group):
//
//   * a CTA stages the tokens in shared memory once; a warp owns four consecutive weight rows (two
//     of each matrix for a gate/up pair) and the 32 lanes split K: per step a lane takes 16 codes of
//     every row (one 128-bit load per row, all inside one 32-element block, so one scale per row)
//     against 16 activations it converts to fp32 once and reuses for the rows; the loads of the
//     next step are issued before the current one is computed, which keeps ~64 KB in flight per SM;
//   * int8 -> fp32 without the conversion pipe: the byte goes into the mantissa of 2^23 (one PRMT),
//     minus 2^23 + 128 (one FADD, exact); products accumulate in fp32 per block and the block's
//     scale multiplies the partial sum -- the factored form the reference uses;
//   * rows are reduced with warp shuffles; the gate/up variant keeps both sums and applies the
//     activation in the epilogue (metal/std/quant.py:358-695).
#include "linear.cuh"
#include "linear_rows.cuh"

namespace alloyb {
namespace q8 {

constexpr int WARPS = 8;
constexpr int ROWS = 4;              // row loads per warp and step: 4 rows, or 2 rows of gate + 2 of up
constexpr int MT = 4;                // tokens per pass

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// the four int8 codes of a word as floats
__device__ __forceinline__ void codes4(uint32_t w, float (&c)[4]) {
    const uint32_t u = w ^ 0x80808080u;                           // code + 128, unsigned
    constexpr uint32_t MAGIC = 0x4B000000u;                       // 2^23: the byte lands in the mantissa
    c[0] = __uint_as_float(prmt(u, MAGIC, 0x7650u)) - 8388736.0f;
    c[1] = __uint_as_float(prmt(u, MAGIC, 0x7651u)) - 8388736.0f;
    c[2] = __uint_as_float(prmt(u, MAGIC, 0x7652u)) - 8388736.0f;
    c[3] = __uint_as_float(prmt(u, MAGIC, 0x7653u)) - 8388736.0f;
}

struct Params {
    const void* x;                   // (M, K) activations
    int M, K, N;
    const int8_t* w[2];              // [gate | up] or [w | -]
    const __half* s[2];
    void* y;                         // (M, N)
    int64_t ldy;
    const void* residual;            // plain only
    int act;
};

// MTOK: tokens per pass (1: the decode case, light enough on registers for two CTAs per SM; 4)
template <typename XT, bool GATED, int MTOK>
__global__ void __launch_bounds__(WARPS * 32, MTOK == 1 ? 2 : 1) q8_gemv_kernel(const Params P) {
    constexpr int MT = MTOK;
    pdl_launch_dependents();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    XT* xs = reinterpret_cast<XT*>(smem_raw);                     // [M][K]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NM = GATED ? 2 : 1, R = ROWS / NM;
    const int row0 = (blockIdx.x * WARPS + warp) * R;
    const int K = P.K, M = P.M, nblk = K / Q8_BLOCK;
    pdl_wait();
    for (int i = threadIdx.x * 8; i < M * K; i += WARPS * 32 * 8)
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(xs) + static_cast<size_t>(i) * sizeof(XT)) =
            *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(P.x) + static_cast<size_t>(i) * sizeof(XT));
    if (sizeof(XT) == 4)                                          // fp32: the second half of each 8-element group
        for (int i = threadIdx.x * 8 + 4; i < M * K; i += WARPS * 32 * 8)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(xs) + static_cast<size_t>(i) * 4) =
                *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(P.x) + static_cast<size_t>(i) * 4);
    __syncthreads();
    if (row0 >= P.N) return;
    float acc[NM][R][MT];
#pragma unroll
    for (int a = 0; a < NM; ++a)
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[a][r][m] = 0.f;
    const int8_t* wrow[NM][R];
    const __half* srow[NM][R];
#pragma unroll
    for (int a = 0; a < NM; ++a)
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = min(row0 + r, P.N - 1);               // tail rows re-read the last row
            wrow[a][r] = P.w[a] + static_cast<int64_t>(row) * K;
            srow[a][r] = P.s[a] + static_cast<int64_t>(row) * nblk;
        }
    uint4 cw[NM][R], nw[NM][R];
    float sc[NM][R], ns[NM][R];
    auto load = [&](int k0, uint4 (&c)[NM][R], float (&s)[NM][R]) {
#pragma unroll
        for (int a = 0; a < NM; ++a)
#pragma unroll
            for (int r = 0; r < R; ++r) {
                c[a][r] = __ldg(reinterpret_cast<const uint4*>(wrow[a][r] + k0));
                s[a][r] = __half2float(__ldg(srow[a][r] + k0 / Q8_BLOCK));
            }
    };
    load(lane * 16, cw, sc);
    for (int k0 = lane * 16; k0 < K; k0 += 32 * 16) {
        const bool more = k0 + 32 * 16 < K;
        if (more) load(k0 + 32 * 16, nw, ns);                     // in flight while this step is computed
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m >= M) break;
            float xf[16];
            const XT* xr = xs + static_cast<size_t>(m) * K + k0;
#pragma unroll
            for (int e = 0; e < 16; ++e) xf[e] = to_f32<XT>(xr[e]);
#pragma unroll
            for (int a = 0; a < NM; ++a)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t wv[4] = {cw[a][r].x, cw[a][r].y, cw[a][r].z, cw[a][r].w};
                    float part = 0.f;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float c[4];
                        codes4(wv[q], c);
#pragma unroll
                        for (int e = 0; e < 4; ++e) part = fmaf(xf[4 * q + e], c[e], part);
                    }
                    acc[a][r][m] = fmaf(sc[a][r], part, acc[a][r][m]);
                }
        }
        if (more) {
#pragma unroll
            for (int a = 0; a < NM; ++a)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    cw[a][r] = nw[a][r];
                    sc[a][r] = ns[a][r];
                }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m >= M) break;
            const float v = warp_sum(acc[0][r][m]);
            const float u = GATED ? warp_sum(acc[NM - 1][r][m]) : 0.f;
            if (lane == 0 && row0 + r < P.N) {
                const int64_t o = static_cast<int64_t>(m) * P.ldy + row0 + r;
                XT* y = static_cast<XT*>(P.y);
                if (GATED) {
                    const float a = (P.act == ALLOYB_ACT_SILU) ? act_silu(v) : act_gelu_tanh(v);
                    y[o] = from_f32<XT>(a * u);
                } else {
                    XT out = from_f32<XT>(v);
                    if (P.residual) out = from_f32<XT>(to_f32<XT>(static_cast<const XT*>(P.residual)[o]) + to_f32<XT>(out));
                    y[o] = out;
                }
            }
        }
}

template <typename XT, bool GATED, int MTOK>
static int launch_m(const Params& P, cudaStream_t st) {
    static bool configured[64] = {};
    auto kern = q8_gemv_kernel<XT, GATED, MTOK>;
    const size_t smem = static_cast<size_t>(P.M) * P.K * sizeof(XT);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
        configured[dev] = true;
    }
    constexpr int rows_per_cta = WARPS * ROWS / (GATED ? 2 : 1);
    const int blocks = (P.N + rows_per_cta - 1) / rows_per_cta;
    const cudaError_t e = launch_pdl(kern, dim3(blocks), dim3(WARPS * 32), smem, st, P);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return check_launch();
}

template <typename XT, bool GATED>
static int launch(const Params& P, cudaStream_t st) {
    return P.M == 1 ? launch_m<XT, GATED, 1>(P, st) : launch_m<XT, GATED, MT>(P, st);
}

}  // namespace q8

// M tokens against one or two (gate/up) Q8_0 matrices; NOT_TAKEN when the shape or alignment is
// outside the kernel (the row kernels then serve it).  More than four tokens run as passes of four.
int try_q8_gemv(const void* x, int M, int K, int dtype, const void* w0, const void* s0, const void* w1, const void* s1,
                void* y, int N, int64_t ldy, const void* residual, bool gated, int act, cudaStream_t st) {
    if (M < 1 || M >= 64 || K % 512 || N < 1) return ALLOYB_NOT_TAKEN;
    const size_t esz = dtype == ALLOYB_F32 ? 4 : 2;
    if (static_cast<size_t>(q8::MT) * K * esz > 190 * 1024) return ALLOYB_NOT_TAKEN;
    if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(w0) % 16 || (gated && reinterpret_cast<uintptr_t>(w1) % 16))
        return ALLOYB_NOT_TAKEN;
    for (int m0 = 0; m0 < M; m0 += q8::MT) {
        q8::Params P;
        P.x = static_cast<const uint8_t*>(x) + static_cast<size_t>(m0) * K * esz;
        P.M = M - m0 < q8::MT ? M - m0 : q8::MT;
        P.K = K;
        P.N = N;
        P.w[0] = static_cast<const int8_t*>(w0);
        P.s[0] = static_cast<const __half*>(s0);
        P.w[1] = static_cast<const int8_t*>(gated ? w1 : w0);
        P.s[1] = static_cast<const __half*>(gated ? s1 : s0);
        P.y = static_cast<uint8_t*>(y) + static_cast<size_t>(m0) * ldy * esz;
        P.ldy = ldy;
        P.residual = residual ? static_cast<const uint8_t*>(residual) + static_cast<size_t>(m0) * ldy * esz : nullptr;
        P.act = act;
        int rc;
        if (dtype == ALLOYB_F16) rc = gated ? q8::launch<__half, true>(P, st) : q8::launch<__half, false>(P, st);
        else if (dtype == ALLOYB_BF16) rc = gated ? q8::launch<__nv_bfloat16, true>(P, st) : q8::launch<__nv_bfloat16, false>(P, st);
        else if (dtype == ALLOYB_F32) rc = gated ? q8::launch<float, true>(P, st) : q8::launch<float, false>(P, st);
        else return ALLOYB_E_DTYPE;
        if (rc != ALLOYB_OK) return rc;
    }
    return ALLOYB_OK;
}

}  // namespace alloyb

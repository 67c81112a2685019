// Bit-exact row dequantisers (embedding gather + test hook) for Q4_K / Q6_K / Q8_0.
//
// Each thread decodes one element with the element-wise formulas of the GGUF
// block formats.  All products (d*sc*nib, dmin*m, d*sc8*q, scale*q) are exact
// in fp32, so the only rounding is the Q4_K subtract; FMA contraction is
// avoided there so the result is the rounded difference of the two exact
// products whatever the compiler does.
#include "common.cuh"

namespace alloyb {

__device__ __forceinline__ float decode_q4k(const uint8_t* __restrict__ blk, int p) {
    const int g = p >> 5, l = p & 31;
    const float d = half_bits_to_f32(blk[0] | (blk[1] << 8));
    const float dmin = half_bits_to_f32(blk[2] | (blk[3] << 8));
    const uint8_t* s = blk + 4;
    int sc, mn;
    if (g < 4) {
        sc = s[g] & 63;
        mn = s[g + 4] & 63;
    } else {
        sc = (s[g + 4] & 15) | ((s[g - 4] >> 6) << 4);
        mn = (s[g + 4] >> 4) | ((s[g] >> 6) << 4);
    }
    const int byte = blk[16 + (g >> 1) * 32 + l];
    const int nib = (g & 1) ? (byte >> 4) : (byte & 15);
    const float a = __fmul_rn(__fmul_rn(d, static_cast<float>(sc)), static_cast<float>(nib));
    const float b = __fmul_rn(dmin, static_cast<float>(mn));
    return __fsub_rn(a, b);
}

__device__ __forceinline__ float decode_q6k(const uint8_t* __restrict__ blk, int p) {
    const int g = p >> 5, l = p & 31;
    const int qlb = blk[(g >> 2) * 64 + (g & 1) * 32 + l];
    const int nib = ((g & 3) >= 2) ? (qlb >> 4) : (qlb & 15);
    const int hi = (blk[128 + (g >> 2) * 32 + l] >> ((g & 3) * 2)) & 3;
    const int q = (nib | (hi << 4)) - 32;
    const int sc = static_cast<int8_t>(blk[192 + (p >> 4)]);
    const float d = half_bits_to_f32(blk[208] | (blk[209] << 8));
    return __fmul_rn(__fmul_rn(d, static_cast<float>(sc)), static_cast<float>(q));
}

template <int FMT, typename OT>
__global__ void dequant_rows_kernel(const uint8_t* __restrict__ data, const __half* __restrict__ scales,
                                    const int64_t* __restrict__ ids, OT* __restrict__ out,
                                    int64_t n_rows, int64_t table_rows, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = n_rows * static_cast<int64_t>(K);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / K;
        const int c = static_cast<int>(i - r * K);
        int64_t src = ids ? ids[r] : r;
        float w = 0.f;
        if (src >= 0 && src < table_rows) {   // out-of-range ids decode to 0 instead of faulting
            if (FMT == ALLOYB_Q4_K) {
                const uint8_t* blk = data + src * (static_cast<int64_t>(K / QK_K) * Q4K_BYTES) +
                                     static_cast<int64_t>(c / QK_K) * Q4K_BYTES;
                w = decode_q4k(blk, c % QK_K);
            } else if (FMT == ALLOYB_Q6_K) {
                const uint8_t* blk = data + src * (static_cast<int64_t>(K / QK_K) * Q6K_BYTES) +
                                     static_cast<int64_t>(c / QK_K) * Q6K_BYTES;
                w = decode_q6k(blk, c % QK_K);
            } else {
                const int8_t q = reinterpret_cast<const int8_t*>(data)[src * K + c];
                const float s = __half2float(scales[src * (K / Q8_BLOCK) + c / Q8_BLOCK]);
                w = __fmul_rn(s, static_cast<float>(q));
            }
        }
        out[i] = from_f32<OT>(w);
    }
}

template <int FMT>
static int launch_dequant(const void* data, const void* scales, const int64_t* ids, void* out,
                          int64_t n_rows, int64_t table_rows, int K, int out_dtype, void* stream) {
    if (!data || !out) return ALLOYB_E_NULL;
    if (n_rows < 0 || table_rows <= 0 || K <= 0) return ALLOYB_E_SHAPE;
    if (K % (FMT == ALLOYB_Q8_0 ? Q8_BLOCK : QK_K) != 0) return ALLOYB_E_SHAPE;
    if (FMT == ALLOYB_Q8_0 && !scales) return ALLOYB_E_NULL;
    if (n_rows == 0) return ALLOYB_OK;
    const int64_t total = n_rows * static_cast<int64_t>(K);
    const int threads = 256;
    const int64_t want = (total + threads - 1) / threads;
    const int blocks = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
    cudaStream_t st = as_stream(stream);
    const uint8_t* d8 = static_cast<const uint8_t*>(data);
    const __half* sc = static_cast<const __half*>(scales);
    switch (out_dtype) {
        case ALLOYB_F32:
            launch_pdl(dequant_rows_kernel<FMT, float>, dim3(blocks), dim3(threads), 0, st, 
                d8, sc, ids, static_cast<float*>(out), n_rows, table_rows, K);
            break;
        case ALLOYB_F16:
            launch_pdl(dequant_rows_kernel<FMT, __half>, dim3(blocks), dim3(threads), 0, st, 
                d8, sc, ids, static_cast<__half*>(out), n_rows, table_rows, K);
            break;
        case ALLOYB_BF16:
            launch_pdl(dequant_rows_kernel<FMT, __nv_bfloat16>, dim3(blocks), dim3(threads), 0, st, 
                d8, sc, ids, static_cast<__nv_bfloat16*>(out), n_rows, table_rows, K);
            break;
        default:
            return ALLOYB_E_DTYPE;
    }
    return check_launch();
}

}  // namespace alloyb

using namespace alloyb;

extern "C" int alloyb_dequant_q4k(const void* blocks, const int64_t* ids, void* out, int64_t n_rows,
                                  int64_t table_rows, int K, int out_dtype, void* stream) {
    return launch_dequant<ALLOYB_Q4_K>(blocks, nullptr, ids, out, n_rows, table_rows, K, out_dtype,
                                       stream);
}
extern "C" int alloyb_dequant_q6k(const void* blocks, const int64_t* ids, void* out, int64_t n_rows,
                                  int64_t table_rows, int K, int out_dtype, void* stream) {
    return launch_dequant<ALLOYB_Q6_K>(blocks, nullptr, ids, out, n_rows, table_rows, K, out_dtype,
                                       stream);
}
extern "C" int alloyb_dequant_q8_0(const void* qweight, const void* scales, const int64_t* ids,
                                   void* out, int64_t n_rows, int64_t table_rows, int K,
                                   int out_dtype, void* stream) {
    return launch_dequant<ALLOYB_Q8_0>(qweight, scales, ids, out, n_rows, table_rows, K, out_dtype,
                                       stream);
}

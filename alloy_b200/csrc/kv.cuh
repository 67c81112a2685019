// KV cache layouts shared by the append and attention kernels.
#pragma once
#include "common.cuh"

namespace alloyb {

// Byte offset of one token row (D/32 blocks of 34 bytes) inside the paged pool
// (num_pages, 2, KV_H, 16, D/32*34).
__host__ __device__ __forceinline__ int64_t paged_row_offset(int64_t page, int kv, int h, int tok,
                                                             int KV_H, int D) {
    const int64_t row_bytes = static_cast<int64_t>(D / 32) * KV_BLOCK_BYTES;
    return (((page * 2 + kv) * KV_H + h) * PAGE_TOKENS + tok) * row_bytes;
}

// Device pointers of one cache in any of the three layouts.
struct KVPtrs {
    void* k0;
    void* k1;
    void* v0;
    void* v1;
    int S_max;          // split / f16: positions per (batch, head); paged: max_pages * 16
    int max_pages;      // paged only
    int64_t num_pages;  // paged only
};

// Status bits the kernels OR into the caller's status word instead of faulting.
enum { KV_STATUS_POS_RANGE = 1, KV_STATUS_PAGE_RANGE = 2 };

#ifdef __CUDACC__
// q8_0 quantisation of one 32-element block, all in fp32 with IEEE division and no contraction, so codes
// and scales are bit-identical to the NumPy statement in the reference's test
// (tests/kernels/test_kv_quant.py:19-30):
//   m = max|x|; scale = fp16(m / 127); inv = m > 0 ? 127 / m : 0;
//   code = int8(sign(x*inv) * floor(|x*inv| + 0.5))
struct Q8Block {
    int code;
    __half scale;
};

// All 32 lanes of a warp hold one element each of the same block.
__device__ __forceinline__ Q8Block quantize_block_q8(float x) {
    const float m = warp_max(fabsf(x));
    const float inv = (m > 0.f) ? __fdiv_rn(127.0f, m) : 0.f;
    const float q = __fmul_rn(x, inv);
    const float mag = floorf(__fadd_rn(fabsf(q), 0.5f));
    Q8Block r;
    r.code = static_cast<int>(copysignf(mag, q));
    r.scale = __float2half_rn(__fdiv_rn(m, 127.0f));
    return r;
}

// One 32-element block of a new K (which = 0) or V (1) row at position p, one element per lane, into
// the cache of any layout (q8 layouts quantise it).
template <int LAYOUT>
__device__ __forceinline__ void store_kv_block(const KVPtrs& kv, int which, int b, int h, int p, int blk, int lane,
                                               __half xin, int KV_H, int D, int* status) {
    const int nblk = D / 32;
    if (LAYOUT == ALLOYB_KV_F16) {
        __half* cache = static_cast<__half*>(which ? kv.v0 : kv.k0);
        cache[((static_cast<int64_t>(b) * KV_H + h) * kv.S_max + p) * D + blk * 32 + lane] = xin;
        return;
    }
    const Q8Block qb = quantize_block_q8(__half2float(xin));
    if (LAYOUT == ALLOYB_KV_Q8_SPLIT) {
        const int64_t row = (static_cast<int64_t>(b) * KV_H + h) * kv.S_max + p;
        static_cast<int8_t*>(which ? kv.v0 : kv.k0)[row * D + blk * 32 + lane] = static_cast<int8_t>(qb.code);
        if (lane == 0) static_cast<__half*>(which ? kv.v1 : kv.k1)[row * nblk + blk] = qb.scale;
    } else {
        const int32_t* table = static_cast<const int32_t*>(kv.k1);
        const int64_t page = table[static_cast<int64_t>(b) * kv.max_pages + p / PAGE_TOKENS];
        if (page < 0 || page >= kv.num_pages) {
            if (lane == 0 && status) atomicOr(status, KV_STATUS_PAGE_RANGE);
            return;
        }
        uint8_t* dst = static_cast<uint8_t*>(kv.k0) + paged_row_offset(page, which, h, p % PAGE_TOKENS, KV_H, D) +
                       blk * KV_BLOCK_BYTES;
        if (lane == 0) *reinterpret_cast<__half*>(dst) = qb.scale;
        reinterpret_cast<int8_t*>(dst + 2)[lane] = static_cast<int8_t>(qb.code);
    }
}

#endif

// Store one new token per sequence at pos[b] (pos_count == 1: pos[0] for all).
int launch_kv_append(int layout, const void* new_k, const void* new_v, int64_t sb, int64_t sh,
                     const KVPtrs& kv, const int32_t* pos, int pos_count, int B, int KV_H, int D,
                     int* status, cudaStream_t st);

// Tensor-core decode attention (head_dim 128, <= 8 query heads per KV head); see attn_mma.cu.
// `fuse` (optional): RoPE of q and of the new K row and the append of the new K / V rows happen inside
// the kernel (fp16 q, 16-byte aligned); q itself is left untouched in memory.
struct AttnFuse {
    const float* inv_freq;      // D / 2 rotation frequencies
    const __half* new_k;        // (B, KV_H, D) rows, strides below (elements)
    const __half* new_v;
    int64_t new_bs, new_hs;
};
int launch_attn_mma(int layout, const void* q, int64_t q_bs, int64_t q_hs, int q_dtype, const KVPtrs& kv,
                    const int32_t* pos, int pos_count, void* out, int B, int H, int KV_H, float scale_log2,
                    int splits, float* part_o, float* part_lse, unsigned int* counters, int* status,
                    cudaStream_t st, const AttnFuse* fuse = nullptr);
int attn_mma_device_error(int clear);

}  // namespace alloyb

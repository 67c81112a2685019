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

// Store one new token per sequence at pos[b] (pos_count == 1: pos[0] for all).
int launch_kv_append(int layout, const void* new_k, const void* new_v, int64_t sb, int64_t sh,
                     const KVPtrs& kv, const int32_t* pos, int pos_count, int B, int KV_H, int D,
                     int* status, cudaStream_t st);

// Tensor-core decode attention (head_dim 128, <= 8 query heads per KV head); see attn_mma.cu.
int launch_attn_mma(int layout, const void* q, int64_t q_bs, int64_t q_hs, int q_dtype, const KVPtrs& kv,
                    const int32_t* pos, int pos_count, void* out, int B, int H, int KV_H, float scale_log2,
                    int splits, float* part_o, float* part_lse, unsigned int* counters, int* status,
                    cudaStream_t st);
int attn_mma_device_error(int clear);

}  // namespace alloyb

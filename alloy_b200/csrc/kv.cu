// q8_0 KV cache: quantise-on-append (split tensors and paged 34-byte blocks) and dequantise.
//
// Arithmetic per 32-element block of one token/head, all in fp32 with IEEE
// division and no contraction, so codes and scales are bit-identical to the
// NumPy statement in the reference's test (tests/kernels/test_kv_quant.py:19-30):
//   m = max|x|; scale = fp16(m / 127); inv = m > 0 ? 127 / m : 0;
//   code = int8(sign(x*inv) * floor(|x*inv| + 0.5))
#include "kv.cuh"

namespace alloyb {

// Range quantise into the split layout; one warp per (b, h, token, block).
__global__ void kv_quantize_range_kernel(const __half* __restrict__ src, int64_t sb, int64_t sh,
                                         int64_t stok, int8_t* __restrict__ codes,
                                         __half* __restrict__ scales, int B, int KV_H, int S_max,
                                         int D, int start, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int nblk = D / 32;
    const int64_t warps_total = static_cast<int64_t>(B) * KV_H * n_tokens * nblk;
    const int64_t wid = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (wid >= warps_total) return;
    int64_t r = wid;
    const int blk = static_cast<int>(r % nblk); r /= nblk;
    const int t = static_cast<int>(r % n_tokens); r /= n_tokens;
    const int h = static_cast<int>(r % KV_H); r /= KV_H;
    const int b = static_cast<int>(r);
    const float x = __half2float(src[b * sb + h * sh + t * stok + blk * 32 + lane]);
    const Q8Block qb = quantize_block_q8(x);
    const int64_t row = (static_cast<int64_t>(b) * KV_H + h) * S_max + (start + t);
    codes[row * D + blk * 32 + lane] = static_cast<int8_t>(qb.code);
    if (lane == 0) scales[row * nblk + blk] = qb.scale;
}

// One new token per sequence, any layout; one warp per (b, h, K|V, block).
template <int LAYOUT>
__global__ void kv_append_kernel(const __half* __restrict__ new_k, const __half* __restrict__ new_v,
                                 int64_t sb, int64_t sh, KVPtrs kv, const int32_t* __restrict__ pos,
                                 int pos_count, int B, int KV_H, int D, int* __restrict__ status) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int nblk = D / 32;
    const int64_t warps_total = static_cast<int64_t>(B) * KV_H * nblk * 2;
    const int64_t wid = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (wid >= warps_total) return;
    pdl_wait();
    int64_t r = wid;
    const int which = static_cast<int>(r & 1); r >>= 1;
    const int blk = static_cast<int>(r % nblk); r /= nblk;
    const int h = static_cast<int>(r % KV_H); r /= KV_H;
    const int b = static_cast<int>(r);
    const int p = pos[pos_count == 1 ? 0 : b];
    if (p < 0 || p >= kv.S_max) {
        if (lane == 0 && status) atomicOr(status, KV_STATUS_POS_RANGE);
        return;
    }
    const __half xin = (which ? new_v : new_k)[b * sb + h * sh + blk * 32 + lane];
    store_kv_block<LAYOUT>(kv, which, b, h, p, blk, lane, xin, KV_H, D, status);
}

__global__ void kv_dequant_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales,
                                  __half* __restrict__ out, int64_t rows_total, int S_max, int D,
                                  int end) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = rows_total * D;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = i / D;
        if (static_cast<int>(row % S_max) >= end) continue;
        const int c = static_cast<int>(i - row * D);
        const float s = __half2float(scales[row * (D / 32) + c / 32]);
        out[i] = __float2half_rn(__fmul_rn(static_cast<float>(codes[i]), s));
    }
}

// RoPE (rotate-half) of the new token's q (in place) and k, and the append of k / v to the cache, in
// one launch.  A warp owns 32 rotation pairs (j, j + D/2) of one head, i.e. two whole 32-element
// blocks, so the rotated K row is quantised without leaving the warp.  Same arithmetic and
// rounding points as rope_inplace followed by the append: fp32 rotation, fp16 result, q8 of that.
template <int LAYOUT>
__global__ void rope_kv_append_kernel(__half* __restrict__ q, const __half* __restrict__ new_k,
                                      const __half* __restrict__ new_v, int64_t sb, int64_t sh, KVPtrs kv,
                                      const int32_t* __restrict__ pos, int pos_count,
                                      const float* __restrict__ inv_freq, int B, int H, int KV_H, int D,
                                      int* __restrict__ status) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int npair = D / 64, nblk = D / 32;          // pair-warps per head, blocks per row
    const int64_t wq = static_cast<int64_t>(B) * H * npair, wk = static_cast<int64_t>(B) * KV_H * npair,
                  wv = static_cast<int64_t>(B) * KV_H * nblk;
    int64_t wid = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (wid >= wq + wk + wv) return;
    pdl_wait();
    if (wid < wq + wk) {
        const bool is_q = wid < wq;
        if (!is_q) wid -= wq;
        const int heads = is_q ? H : KV_H;
        const int ph = static_cast<int>(wid % npair);
        const int hh = static_cast<int>((wid / npair) % heads);
        const int b = static_cast<int>(wid / npair / heads);
        const int p = pos[pos_count == 1 ? 0 : b];
        const int j = 32 * ph + lane, half = D / 2;
        const float angle = static_cast<float>(p) * inv_freq[j];
        float sn, cs;
        sincosf(angle, &sn, &cs);
        if (is_q) {
            __half* base = q + (static_cast<int64_t>(b) * H + hh) * D;
            const float x1 = __half2float(base[j]), x2 = __half2float(base[j + half]);
            base[j] = __float2half_rn(__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn)));
            base[j + half] = __float2half_rn(__fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn)));
            return;
        }
        if (p < 0 || p >= kv.S_max) {
            if (lane == 0 && status) atomicOr(status, KV_STATUS_POS_RANGE);
            return;
        }
        const __half* base = new_k + b * sb + hh * sh;
        const float x1 = __half2float(base[j]), x2 = __half2float(base[j + half]);
        store_kv_block<LAYOUT>(kv, 0, b, hh, p, ph, lane,
                               __float2half_rn(__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn))), KV_H, D, status);
        store_kv_block<LAYOUT>(kv, 0, b, hh, p, ph + npair, lane,
                               __float2half_rn(__fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn))), KV_H, D, status);
        return;
    }
    wid -= wq + wk;
    const int blk = static_cast<int>(wid % nblk);
    const int h = static_cast<int>((wid / nblk) % KV_H);
    const int b = static_cast<int>(wid / nblk / KV_H);
    const int p = pos[pos_count == 1 ? 0 : b];
    if (p < 0 || p >= kv.S_max) return;                // reported by the K warps
    store_kv_block<LAYOUT>(kv, 1, b, h, p, blk, lane, new_v[b * sb + h * sh + blk * 32 + lane], KV_H, D, status);
}

// n_tokens new rows per (sequence, kv head) into the cache at [start_b, start_b + n_tokens), any
// layout (the prefill / verify write; the q8 layouts quantise the rows exactly as the append does):
// one warp per (b, h, token, K|V, 32-element block).
template <int LAYOUT>
__global__ void kv_write_range_kernel(const __half* __restrict__ new_k, const __half* __restrict__ new_v, int64_t sb,
                                      int64_t sh, int64_t stok, KVPtrs kv, const int32_t* __restrict__ start,
                                      int start_count, int B, int KV_H, int D, int n_tokens, int* __restrict__ status) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int nblk = D / 32;
    const int64_t warps_total = static_cast<int64_t>(B) * KV_H * n_tokens * nblk * 2;
    const int64_t wid = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (wid >= warps_total) return;
    pdl_wait();
    int64_t r = wid;
    const int which = static_cast<int>(r & 1); r >>= 1;
    const int blk = static_cast<int>(r % nblk); r /= nblk;
    const int t = static_cast<int>(r % n_tokens); r /= n_tokens;
    const int h = static_cast<int>(r % KV_H); r /= KV_H;
    const int b = static_cast<int>(r);
    const int p = start[start_count == 1 ? 0 : b] + t;
    if (p < 0 || p >= kv.S_max) {
        if (lane == 0 && status) atomicOr(status, KV_STATUS_POS_RANGE);
        return;
    }
    const __half xin = (which ? new_v : new_k)[b * sb + h * sh + t * stok + blk * 32 + lane];
    store_kv_block<LAYOUT>(kv, which, b, h, p, blk, lane, xin, KV_H, D, status);
}

int launch_kv_write_range(int layout, const void* new_k, const void* new_v, int64_t sb, int64_t sh, int64_t stok,
                          const KVPtrs& kv, const int32_t* start, int start_count, int B, int KV_H, int D,
                          int n_tokens, int* status, cudaStream_t st) {
    const __half* nk = static_cast<const __half*>(new_k);
    const __half* nv = static_cast<const __half*>(new_v);
    const int64_t warps = static_cast<int64_t>(B) * KV_H * n_tokens * (D / 32) * 2;
    const int64_t blocks64 = (warps * 32 + 255) / 256;
    if (blocks64 > 0x7fffffff) return ALLOYB_E_SHAPE;
    const int blocks = static_cast<int>(blocks64);
    switch (layout) {
        case ALLOYB_KV_F16:
            launch_pdl(kv_write_range_kernel<ALLOYB_KV_F16>, dim3(blocks), dim3(256), 0, st, nk, nv, sb, sh, stok, kv,
                       start, start_count, B, KV_H, D, n_tokens, status);
            break;
        case ALLOYB_KV_Q8_SPLIT:
            launch_pdl(kv_write_range_kernel<ALLOYB_KV_Q8_SPLIT>, dim3(blocks), dim3(256), 0, st, nk, nv, sb, sh, stok,
                       kv, start, start_count, B, KV_H, D, n_tokens, status);
            break;
        case ALLOYB_KV_Q8_PAGED:
            launch_pdl(kv_write_range_kernel<ALLOYB_KV_Q8_PAGED>, dim3(blocks), dim3(256), 0, st, nk, nv, sb, sh, stok,
                       kv, start, start_count, B, KV_H, D, n_tokens, status);
            break;
        default:
            return ALLOYB_E_SHAPE;
    }
    return check_launch();
}

int launch_kv_append(int layout, const void* new_k, const void* new_v, int64_t sb, int64_t sh,
                     const KVPtrs& kv, const int32_t* pos, int pos_count, int B, int KV_H, int D,
                     int* status, cudaStream_t st) {
    const __half* nk = static_cast<const __half*>(new_k);
    const __half* nv = static_cast<const __half*>(new_v);
    const int64_t warps = static_cast<int64_t>(B) * KV_H * (D / 32) * 2;
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    switch (layout) {
        case ALLOYB_KV_F16:
            launch_pdl(kv_append_kernel<ALLOYB_KV_F16>, dim3(blocks), dim3(256), 0, st, nk, nv, sb, sh, kv, pos, pos_count,
                                                                    B, KV_H, D, status);
            break;
        case ALLOYB_KV_Q8_SPLIT:
            launch_pdl(kv_append_kernel<ALLOYB_KV_Q8_SPLIT>, dim3(blocks), dim3(256), 0, st, nk, nv, sb, sh, kv, pos,
                                                                         pos_count, B, KV_H, D, status);
            break;
        case ALLOYB_KV_Q8_PAGED:
            launch_pdl(kv_append_kernel<ALLOYB_KV_Q8_PAGED>, dim3(blocks), dim3(256), 0, st, nk, nv, sb, sh, kv, pos,
                                                                         pos_count, B, KV_H, D, status);
            break;
        default:
            return ALLOYB_E_SHAPE;
    }
    return check_launch();
}

}  // namespace alloyb

using namespace alloyb;

extern "C" int alloyb_kv_quantize_q8(const void* src, int64_t src_batch_stride,
                                     int64_t src_head_stride, int64_t src_tok_stride, void* codes,
                                     void* scales, int B, int KV_H, int S_max, int D, int start,
                                     int n_tokens, void* stream) {
    if (!src || !codes || !scales) return ALLOYB_E_NULL;
    if (B <= 0 || KV_H <= 0 || S_max <= 0 || D <= 0 || D % 32) return ALLOYB_E_SHAPE;
    if (n_tokens < 0 || start < 0 || start + n_tokens > S_max) return ALLOYB_E_SHAPE;
    if (n_tokens == 0) return ALLOYB_OK;
    const int64_t warps = static_cast<int64_t>(B) * KV_H * n_tokens * (D / 32);
    const int64_t blocks = (warps * 32 + 255) / 256;
    if (blocks > 0x7fffffff) return ALLOYB_E_SHAPE;
    launch_pdl(kv_quantize_range_kernel, dim3(static_cast<int>(blocks)), dim3(256), 0, as_stream(stream), 
        static_cast<const __half*>(src), src_batch_stride, src_head_stride, src_tok_stride,
        static_cast<int8_t*>(codes), static_cast<__half*>(scales), B, KV_H, S_max, D, start, n_tokens);
    return check_launch();
}

extern "C" int alloyb_kv_dequant_q8(const void* codes, const void* scales, void* out, int B, int KV_H,
                                    int S_max, int D, int end, void* stream) {
    if (!codes || !scales || !out) return ALLOYB_E_NULL;
    if (B <= 0 || KV_H <= 0 || S_max <= 0 || D <= 0 || D % 32 || end < 0 || end > S_max)
        return ALLOYB_E_SHAPE;
    if (end == 0) return ALLOYB_OK;
    const int64_t rows = static_cast<int64_t>(B) * KV_H * S_max;
    const int64_t want = (rows * D + 255) / 256;
    const int blocks = static_cast<int>(want < 148 * 32 ? want : 148 * 32);
    launch_pdl(kv_dequant_kernel, dim3(blocks), dim3(256), 0, as_stream(stream), 
        static_cast<const int8_t*>(codes), static_cast<const __half*>(scales),
        static_cast<__half*>(out), rows, S_max, D, end);
    return check_launch();
}

extern "C" int alloyb_kv_append_q8_paged(const void* new_k, const void* new_v, int64_t batch_stride,
                                         int64_t head_stride, void* pool, const int32_t* page_table,
                                         int max_pages, int64_t num_pages, const int32_t* seq_pos,
                                         int B, int KV_H, int D, int32_t* status, void* stream) {
    if (!new_k || !new_v || !pool || !page_table || !seq_pos) return ALLOYB_E_NULL;
    if (B <= 0 || KV_H <= 0 || D <= 0 || D % 32 || max_pages <= 0 || num_pages <= 0)
        return ALLOYB_E_SHAPE;
    KVPtrs kv;
    kv.k0 = pool;
    kv.k1 = const_cast<int32_t*>(page_table);
    kv.v0 = kv.v1 = nullptr;
    kv.S_max = max_pages * PAGE_TOKENS;
    kv.max_pages = max_pages;
    kv.num_pages = num_pages;
    return launch_kv_append(ALLOYB_KV_Q8_PAGED, new_k, new_v, batch_stride, head_stride, kv, seq_pos,
                            B, B, KV_H, D, status, as_stream(stream));
}

extern "C" int alloyb_rope_kv_append(int layout, void* q, const void* new_k, const void* new_v,
                                     int64_t new_batch_stride, int64_t new_head_stride, void* k0, void* k1,
                                     void* v0, void* v1, const int32_t* pos, int pos_count, const float* inv_freq,
                                     int B, int H, int KV_H, int D, int S_max, int64_t num_pages, int32_t* status,
                                     void* stream) {
    if (!q || !new_k || !new_v || !k0 || !pos || !inv_freq) return ALLOYB_E_NULL;
    if (B <= 0 || H <= 0 || KV_H <= 0 || D <= 0 || D % 64 || S_max <= 0) return ALLOYB_E_SHAPE;
    if (pos_count != 1 && pos_count != B) return ALLOYB_E_SHAPE;
    KVPtrs kv;
    kv.k0 = k0; kv.k1 = k1; kv.v0 = v0; kv.v1 = v1;
    kv.S_max = S_max;
    kv.max_pages = S_max / PAGE_TOKENS;
    kv.num_pages = num_pages;
    if (layout == ALLOYB_KV_F16) { if (!v0) return ALLOYB_E_NULL; }
    else if (layout == ALLOYB_KV_Q8_SPLIT) { if (!k1 || !v0 || !v1) return ALLOYB_E_NULL; }
    else if (layout == ALLOYB_KV_Q8_PAGED) {
        if (!k1) return ALLOYB_E_NULL;
        if (S_max % PAGE_TOKENS || num_pages <= 0) return ALLOYB_E_SHAPE;
    } else return ALLOYB_E_SHAPE;
    const int64_t warps = static_cast<int64_t>(B) * (H + KV_H) * (D / 64) + static_cast<int64_t>(B) * KV_H * (D / 32);
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    cudaStream_t st = as_stream(stream);
    __half* qh = static_cast<__half*>(q);
    const __half* nk = static_cast<const __half*>(new_k);
    const __half* nv = static_cast<const __half*>(new_v);
    int* stw = reinterpret_cast<int*>(status);
    switch (layout) {
        case ALLOYB_KV_F16:
            launch_pdl(rope_kv_append_kernel<ALLOYB_KV_F16>, dim3(blocks), dim3(256), 0, st, qh, nk, nv, new_batch_stride,
                       new_head_stride, kv, pos, pos_count, inv_freq, B, H, KV_H, D, stw);
            break;
        case ALLOYB_KV_Q8_SPLIT:
            launch_pdl(rope_kv_append_kernel<ALLOYB_KV_Q8_SPLIT>, dim3(blocks), dim3(256), 0, st, qh, nk, nv,
                       new_batch_stride, new_head_stride, kv, pos, pos_count, inv_freq, B, H, KV_H, D, stw);
            break;
        default:
            launch_pdl(rope_kv_append_kernel<ALLOYB_KV_Q8_PAGED>, dim3(blocks), dim3(256), 0, st, qh, nk, nv,
                       new_batch_stride, new_head_stride, kv, pos, pos_count, inv_freq, B, H, KV_H, D, stw);
            break;
    }
    return check_launch();
}

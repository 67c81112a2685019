// Causal attention of a CHUNK of query tokens (prefill, or the 2..16 tokens of a speculative
// verify step) over a KV cache that already holds the chunk's own rows: fp16, split q8_0 or the
// paged q8_0 pool.  Query token i of the chunk sits at position start + i and attends to cache
// positions [0, start + i].
//
// The reference runs this case as "dequantise history + chunk to an fp16 scratch in cache layout,
// then fp16 prefill attention" (torch/ops/kv_quant.py:121-162 with metal/std/kv_quant.py:73-108);
// here the q8_0 codes are read directly: a CTA dequantises each 64-token K/V tile ONCE into shared
// memory as fp16(code * scale) -- the same values the reference's scratch would hold -- and no
// global scratch exists.
//
// Work split.  A CTA owns one KV head, up to eight of its query heads and 64 / Gp query tokens
// (Gp = heads per CTA rounded up to a power of two), i.e. 64 (token, head) rows, 16 per warp; the
// K/V tile in shared memory is shared by every row.  S = Q K^T and O += P V run on
// mma.sync.m16n8k16 (fp16 operands, fp32 accumulation) with ldmatrix fragment loads; the softmax
// is the usual online one in the exp2 frame; P enters the second product as fp16 hi + lo halves.
#include "kv.cuh"

namespace alloyb {
namespace ac {

constexpr int ROWS = 64;          // (token, head) rows per CTA
constexpr int KT = 64;            // KV tokens per tile
constexpr int WARPS = 4;
constexpr float NEG_BIG = -1.0e30f;
constexpr float P_BIAS = 64.0f;   // keeps small probabilities out of fp16's subnormal range in the P * V product

struct Params {
    const void* q;
    int64_t q_bs, q_hs, q_ts;     // strides in elements: batch, head, token
    int q_dtype;
    KVPtrs kv;
    const int32_t* start;
    int start_count;
    void* out;                    // (B, S, H, D) dense, q's dtype
    int B, H, KV_H, S;
    int G, Gp, HG;                // query heads per KV head; heads per CTA padded; CTAs per KV head
    float scale_log2;
    int* status;
};

__device__ __forceinline__ uint32_t s32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float q_as_f16(const void* q, int dtype, int64_t i) {
    // the attention runs on fp16 queries, like the reference (torch/ops/kv_quant.py:175-180)
    if (dtype == ALLOYB_F16) return __half2float(static_cast<const __half*>(q)[i]);
    if (dtype == ALLOYB_BF16)
        return __half2float(__float2half_rn(__bfloat162float(static_cast<const __nv_bfloat16*>(q)[i])));
    return __half2float(__float2half_rn(static_cast<const float*>(q)[i]));
}
__device__ __forceinline__ void store_out(void* out, int dtype, int64_t i, float a, float b) {
    if (dtype == ALLOYB_F16) *reinterpret_cast<__half2*>(static_cast<__half*>(out) + i) = __floats2half2_rn(a, b);
    else if (dtype == ALLOYB_BF16)
        *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(out) + i) = __floats2bfloat162_rn(a, b);
    else *reinterpret_cast<float2*>(static_cast<float*>(out) + i) = make_float2(a, b);
}

// fp16(code * scale) of eight codes held in two 32-bit words -> four packed half2
__device__ __forceinline__ uint4 dequant8(uint32_t w0, uint32_t w1, float scale) {
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w = i < 2 ? w0 : w1;
        const int c0 = static_cast<int8_t>((w >> (16 * (i & 1))) & 0xffu);
        const int c1 = static_cast<int8_t>((w >> (16 * (i & 1) + 8)) & 0xffu);
        o[i] = pack_h2(__fmul_rn(static_cast<float>(c0), scale), __fmul_rn(static_cast<float>(c1), scale));
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// Fill one 64-token tile of K (which = 0) or V (1) of (b, kvh) starting at token j0 into
// dst[64][D + 8] as fp16; tokens >= n_kv become zero rows.
template <int LAYOUT, int D>
__device__ __forceinline__ void fill_tile(__half* dst, const Params& P, int which, int b, int kvh, int j0, int n_kv) {
    constexpr int PITCH = D + 8;
    constexpr int NB = D / 32;
    const int tid = threadIdx.x;
    if (LAYOUT == ALLOYB_KV_F16) {
        const __half* base = static_cast<const __half*>(which ? P.kv.v0 : P.kv.k0) +
                             (static_cast<int64_t>(b) * P.KV_H + kvh) * P.kv.S_max * D;
        for (int i = tid; i < KT * (D / 8); i += WARPS * 32) {
            const int tok = i / (D / 8), c = i - tok * (D / 8);
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (j0 + tok < n_kv) v = __ldg(reinterpret_cast<const uint4*>(base + static_cast<int64_t>(j0 + tok) * D) + c);
            *reinterpret_cast<uint4*>(dst + tok * PITCH + c * 8) = v;
        }
    } else if (LAYOUT == ALLOYB_KV_Q8_SPLIT) {
        const int64_t row0 = (static_cast<int64_t>(b) * P.KV_H + kvh) * P.kv.S_max;
        const int8_t* codes = static_cast<const int8_t*>(which ? P.kv.v0 : P.kv.k0);
        const __half* scales = static_cast<const __half*>(which ? P.kv.v1 : P.kv.k1);
        // one thread per (token, 16 codes)
        for (int i = tid; i < KT * (D / 16); i += WARPS * 32) {
            const int tok = i / (D / 16), c = i - tok * (D / 16);
            uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
            if (j0 + tok < n_kv) {
                const int64_t row = row0 + j0 + tok;
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(codes + row * D) + c);
                const float s = __half2float(__ldg(scales + row * NB + c / 2));
                lo = dequant8(w.x, w.y, s);
                hi = dequant8(w.z, w.w, s);
            }
            *reinterpret_cast<uint4*>(dst + tok * PITCH + c * 16) = lo;
            *reinterpret_cast<uint4*>(dst + tok * PITCH + c * 16 + 8) = hi;
        }
    } else {
        const int32_t* table = static_cast<const int32_t*>(P.kv.k1) + static_cast<int64_t>(b) * P.kv.max_pages;
        const uint8_t* pool = static_cast<const uint8_t*>(P.kv.k0);
        // one thread per (token, 32-code block); blocks are 2-byte aligned: 16-bit loads
        for (int i = tid; i < KT * NB; i += WARPS * 32) {
            const int tok = i / NB, blk = i - tok * NB;
            uint4 o[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) o[u] = make_uint4(0u, 0u, 0u, 0u);
            const int j = j0 + tok;
            if (j < n_kv) {
                const int64_t page = table[j / PAGE_TOKENS];
                if (page < 0 || page >= P.kv.num_pages) {
                    if (P.status) atomicOr(P.status, KV_STATUS_PAGE_RANGE);
                } else {
                    const uint16_t* bp = reinterpret_cast<const uint16_t*>(
                        pool + paged_row_offset(page, which, kvh, j % PAGE_TOKENS, P.KV_H, D) + blk * KV_BLOCK_BYTES);
                    const float s = half_bits_to_f32(__ldg(bp));
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t a0 = __ldg(bp + 1 + 4 * u), a1 = __ldg(bp + 2 + 4 * u);
                        const uint32_t a2 = __ldg(bp + 3 + 4 * u), a3 = __ldg(bp + 4 + 4 * u);
                        o[u] = dequant8(a0 | (a1 << 16), a2 | (a3 << 16), s);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(dst + tok * PITCH + blk * 32 + u * 8) = o[u];
        }
    }
}

template <int LAYOUT, int D>
__global__ void __launch_bounds__(WARPS * 32) attn_chunk_kernel(const Params P) {
    pdl_launch_dependents();
    constexpr int PITCH = D + 8;
    extern __shared__ __align__(16) uint8_t smem[];
    __half* Qs = reinterpret_cast<__half*>(smem);
    __half* Ks = Qs + ROWS * PITCH;
    __half* Vs = Ks + KT * PITCH;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.y / P.HG, hgrp = blockIdx.y - kvh * P.HG, b = blockIdx.z;
    const int TQ = ROWS / P.Gp;                         // query tokens per CTA
    const int tok0 = blockIdx.x * TQ;
    const int gp_shift = P.Gp == 1 ? 0 : (P.Gp == 2 ? 1 : (P.Gp == 4 ? 2 : 3));
    const int heads_here = min(8, P.G - hgrp * 8);      // live heads of this CTA
    pdl_wait();
    int start = P.start[P.start_count == 1 ? 0 : b];
    if (start < 0 || start + P.S > P.kv.S_max) {
        if (threadIdx.x == 0 && P.status) atomicOr(P.status, KV_STATUS_POS_RANGE);
        start = max(0, min(start, P.kv.S_max - P.S));
    }
    const int tok_last = min(P.S, tok0 + TQ) - 1;
    const int n_kv = start + tok_last + 1;              // positions this CTA may read

    // ---- Q rows -> shared memory (fp16); dead rows are zero
    for (int i = threadIdx.x; i < ROWS * (D / 2); i += WARPS * 32) {
        const int r = i / (D / 2), d = (i - r * (D / 2)) * 2;
        const int tl = r >> gp_shift, hg = r & (P.Gp - 1);
        float a = 0.f, c = 0.f;
        if (tok0 + tl < P.S && hg < heads_here) {
            const int64_t base = b * P.q_bs + static_cast<int64_t>(kvh * P.G + hgrp * 8 + hg) * P.q_hs +
                                 static_cast<int64_t>(tok0 + tl) * P.q_ts + d;
            a = q_as_f16(P.q, P.q_dtype, base);
            c = q_as_f16(P.q, P.q_dtype, base + 1);
        }
        *reinterpret_cast<uint32_t*>(Qs + r * PITCH + d) = pack_h2(a, c);
    }

    // this thread's two rows: warp*16 + g and + 8
    int row_pos[2];                                     // last position each row may see
    bool row_live[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r = warp * 16 + g + 8 * rr;
        const int tl = r >> gp_shift, hg = r & (P.Gp - 1);
        row_live[rr] = tok0 + tl < P.S && hg < heads_here;
        row_pos[rr] = start + tok0 + tl;
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {NEG_BIG, NEG_BIG}, l_run[2] = {0.f, 0.f};

    const uint32_t q_addr = s32(Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + ((lane >> 4) & 1) * 8);
    const uint32_t k_addr = s32(Ks + ((lane & 7) + ((lane >> 4) & 1) * 8) * PITCH + ((lane >> 3) & 1) * 8);
    const uint32_t v_addr = s32(Vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + ((lane >> 4) & 1) * 8);

    for (int j0 = 0; j0 < n_kv; j0 += KT) {
        __syncthreads();                                // previous tile fully consumed (and Q stored)
        fill_tile<LAYOUT, D>(Ks, P, 0, b, kvh, j0, n_kv);
        fill_tile<LAYOUT, D>(Vs, P, 1, b, kvh, j0, n_kv);
        __syncthreads();

        // ---- S = Q K^T : 16 rows x 64 tokens per warp
        float s[KT / 8][4];
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t a[4];
            ldsm_x4(q_addr + kk * 32, a);
#pragma unroll
            for (int n2 = 0; n2 < KT / 16; ++n2) {
                uint32_t bq[4];
                ldsm_x4(k_addr + (n2 * 16 * PITCH) * 2 + kk * 32, bq);
                mma16816(s[2 * n2], a, bq[0], bq[1]);
                mma16816(s[2 * n2 + 1], a, bq[2], bq[3]);
            }
        }
        // ---- mask + online softmax (rows g and g + 8; columns 8n + 2t, + 1)
        float mx[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
        for (int n = 0; n < KT / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int rr = e >> 1;
                const int j = j0 + 8 * n + 2 * t + (e & 1);
                const float v = (j <= row_pos[rr]) ? s[n][e] * P.scale_log2 : NEG_BIG;
                s[n][e] = v;
                mx[rr] = fmaxf(mx[rr], v);
            }
        float alpha[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            const float m_new = fmaxf(m_run[rr], mx[rr]);
            alpha[rr] = exp2f(m_run[rr] - m_new);
            m_run[rr] = m_new;
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= alpha[0];
            o[i][1] *= alpha[0];
            o[i][2] *= alpha[1];
            o[i][3] *= alpha[1];
        }
        // ---- O += P V, sixteen tokens at a time.  P enters the tensor core as fp16 hi + lo halves (two
        // products), which keeps ~22 bits of it: a single fp16 rounding of P alone would cost ~1e-3 of
        // the output's rms, more than the parity tolerance allows on outputs that cancel to near zero.
        float ls[2] = {0.f, 0.f};
#pragma unroll
        for (int k2 = 0; k2 < KT / 16; ++k2) {
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int nn = 0; nn < 2; ++nn) {
                const int n = 2 * k2 + nn;
                float pv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int rr = e >> 1;
                    pv[e] = s[n][e] > 0.5f * NEG_BIG ? exp2f(s[n][e] - m_run[rr]) : 0.f;
                }
                ls[0] += pv[0] + pv[1];
                ls[1] += pv[2] + pv[3];
#pragma unroll
                for (int e = 0; e < 4; ++e) pv[e] *= P_BIAS;
                const uint32_t h01 = pack_h2(pv[0], pv[1]), h23 = pack_h2(pv[2], pv[3]);
                const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
                const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
                ph[nn * 2] = h01;
                ph[nn * 2 + 1] = h23;
                pl[nn * 2] = pack_h2(pv[0] - f01.x, pv[1] - f01.y);
                pl[nn * 2 + 1] = pack_h2(pv[2] - f23.x, pv[3] - f23.y);
            }
#pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                uint32_t bv[4];
                ldsm_x4_t(v_addr + (k2 * 16 * PITCH) * 2 + n2 * 32, bv);
                mma16816(o[2 * n2], ph, bv[0], bv[1]);
                mma16816(o[2 * n2], pl, bv[0], bv[1]);
                mma16816(o[2 * n2 + 1], ph, bv[2], bv[3]);
                mma16816(o[2 * n2 + 1], pl, bv[2], bv[3]);
            }
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            ls[rr] += __shfl_xor_sync(0xffffffffu, ls[rr], 1);
            ls[rr] += __shfl_xor_sync(0xffffffffu, ls[rr], 2);
            l_run[rr] = l_run[rr] * alpha[rr] + ls[rr];
        }
    }

    // ---- normalise and store: out (B, S, H, D)
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        if (!row_live[rr]) continue;
        const int r = warp * 16 + g + 8 * rr;
        const int tl = r >> gp_shift, hg = r & (P.Gp - 1);
        const float inv = l_run[rr] > 0.f ? 1.0f / (P_BIAS * l_run[rr]) : 0.f;
        const int64_t base = ((static_cast<int64_t>(b) * P.S + tok0 + tl) * P.H + kvh * P.G + hgrp * 8 + hg) * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
            store_out(P.out, P.q_dtype, base + 8 * i + 2 * t, o[i][2 * rr] * inv, o[i][2 * rr + 1] * inv);
    }
}

template <int LAYOUT, int D>
static int launch_one(const Params& P, cudaStream_t st) {
    static bool configured[64] = {};
    auto kern = attn_chunk_kernel<LAYOUT, D>;
    constexpr int SMEM = 3 * ROWS * (D + 8) * 2;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
        configured[dev] = true;
    }
    const int TQ = ROWS / P.Gp;
    const dim3 grid((P.S + TQ - 1) / TQ, P.KV_H * P.HG, P.B);
    const cudaError_t e = launch_pdl(kern, grid, dim3(WARPS * 32), SMEM, st, P);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return check_launch();
}

template <int LAYOUT>
static int launch_d(const Params& P, int D, cudaStream_t st) {
    switch (D) {
        case 64: return launch_one<LAYOUT, 64>(P, st);
        case 128: return launch_one<LAYOUT, 128>(P, st);
        case 256: return launch_one<LAYOUT, 256>(P, st);
        default: return ALLOYB_E_SHAPE;
    }
}

}  // namespace ac

// defined in kv.cu (shares the block quantiser with the one-token append)
int launch_kv_write_range(int layout, const void* new_k, const void* new_v, int64_t sb, int64_t sh, int64_t stok,
                          const KVPtrs& kv, const int32_t* start, int start_count, int B, int KV_H, int D,
                          int n_tokens, int* status, cudaStream_t st);

}  // namespace alloyb

using namespace alloyb;

static int fill_kv(int layout, void* k0, void* k1, void* v0, void* v1, int S_max, int64_t num_pages, KVPtrs& kv) {
    kv.k0 = k0; kv.k1 = k1; kv.v0 = v0; kv.v1 = v1;
    kv.S_max = S_max;
    kv.max_pages = S_max / PAGE_TOKENS;
    kv.num_pages = num_pages;
    if (!k0) return ALLOYB_E_NULL;
    if (layout == ALLOYB_KV_F16) { if (!v0) return ALLOYB_E_NULL; }
    else if (layout == ALLOYB_KV_Q8_SPLIT) { if (!k1 || !v0 || !v1) return ALLOYB_E_NULL; }
    else if (layout == ALLOYB_KV_Q8_PAGED) {
        if (!k1) return ALLOYB_E_NULL;
        if (S_max % PAGE_TOKENS || num_pages <= 0) return ALLOYB_E_SHAPE;
    } else return ALLOYB_E_SHAPE;
    return ALLOYB_OK;
}

extern "C" int alloyb_kv_write(int layout, const void* new_k, const void* new_v, int64_t batch_stride,
                               int64_t head_stride, int64_t tok_stride, void* k0, void* k1, void* v0, void* v1,
                               const int32_t* start, int start_count, int B, int KV_H, int D, int S_max,
                               int64_t num_pages, int n_tokens, int32_t* status, void* stream) {
    if (!new_k || !new_v || !start) return ALLOYB_E_NULL;
    if (B <= 0 || KV_H <= 0 || D <= 0 || D % 32 || S_max <= 0 || n_tokens < 0 || n_tokens > S_max)
        return ALLOYB_E_SHAPE;
    if (start_count != 1 && start_count != B) return ALLOYB_E_SHAPE;
    KVPtrs kv;
    const int rc = fill_kv(layout, k0, k1, v0, v1, S_max, num_pages, kv);
    if (rc != ALLOYB_OK) return rc;
    if (n_tokens == 0) return ALLOYB_OK;
    return launch_kv_write_range(layout, new_k, new_v, batch_stride, head_stride, tok_stride, kv, start, start_count,
                                 B, KV_H, D, n_tokens, reinterpret_cast<int*>(status), as_stream(stream));
}

extern "C" int alloyb_attn_chunk(int layout, const void* q, int64_t q_batch_stride, int64_t q_head_stride,
                                 int64_t q_tok_stride, int q_dtype, void* k0, void* k1, void* v0, void* v1,
                                 const int32_t* start, int start_count, void* out, int B, int H, int KV_H, int D,
                                 int n_tokens, int S_max, int64_t num_pages, float scale, int32_t* status,
                                 void* stream) {
    if (!q || !start || !out) return ALLOYB_E_NULL;
    if (B <= 0 || H <= 0 || KV_H <= 0 || H % KV_H || D <= 0 || S_max <= 0 || n_tokens < 0 || n_tokens > S_max)
        return ALLOYB_E_SHAPE;
    if (D != 64 && D != 128 && D != 256) return ALLOYB_E_SHAPE;
    if (start_count != 1 && start_count != B) return ALLOYB_E_SHAPE;
    if (q_dtype != ALLOYB_F16 && q_dtype != ALLOYB_BF16 && q_dtype != ALLOYB_F32) return ALLOYB_E_DTYPE;
    ac::Params P;
    const int rc = fill_kv(layout, k0, k1, v0, v1, S_max, num_pages, P.kv);
    if (rc != ALLOYB_OK) return rc;
    if (layout != ALLOYB_KV_Q8_PAGED &&
        (reinterpret_cast<uintptr_t>(k0) % 16 || reinterpret_cast<uintptr_t>(v0) % 16))
        return ALLOYB_E_ALIGN;
    if (n_tokens == 0) return ALLOYB_OK;
    P.q = q; P.q_bs = q_batch_stride; P.q_hs = q_head_stride; P.q_ts = q_tok_stride; P.q_dtype = q_dtype;
    P.start = start; P.start_count = start_count; P.out = out;
    P.B = B; P.H = H; P.KV_H = KV_H; P.S = n_tokens;
    P.G = H / KV_H;
    P.HG = (P.G + 7) / 8;
    const int per = P.G < 8 ? P.G : 8;
    P.Gp = per <= 1 ? 1 : (per <= 2 ? 2 : (per <= 4 ? 4 : 8));
    const float sc = scale > 0.f ? scale : 1.0f / sqrtf(static_cast<float>(D));
    P.scale_log2 = sc * 1.4426950408889634f;
    P.status = reinterpret_cast<int*>(status);
    cudaStream_t st = as_stream(stream);
    switch (layout) {
        case ALLOYB_KV_F16: return ac::launch_d<ALLOYB_KV_F16>(P, D, st);
        case ALLOYB_KV_Q8_SPLIT: return ac::launch_d<ALLOYB_KV_Q8_SPLIT>(P, D, st);
        default: return ac::launch_d<ALLOYB_KV_Q8_PAGED>(P, D, st);
    }
}

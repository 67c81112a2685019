// Single-query (decode) GQA attention over fp16, split-q8 and paged-q8 KV caches.
//
// Grid (SPLITS, KV_H, B); each CTA (4 warps) streams one token range of one KV head
// ONCE and scores all G = H/KV_H query heads of the group against it.  Softmax runs
// in the exp2 frame (scale*log2e folded into q).  Each CTA writes a normalised
// partial output and its log-sum-exp; the last CTA of a (sequence, kv head) to
// finish merges the partials, so no second launch is needed.
#include "kv.cuh"

namespace alloyb {

constexpr int ATTN_MAX_SPLITS = 64;
constexpr float NEG_BIG = -1.0e30f;

struct AttnParams {
    const void* q;
    int64_t q_bs, q_hs;
    int q_dtype;
    KVPtrs kv;
    const int32_t* pos;
    int pos_count;
    void* out;
    int B, H, KV_H;
    float scale_log2;    // softmax scale * log2(e)
    int splits;
    float* part_o;       // (B, H, splits, D)
    float* part_lse;     // (B, H, splits), log2 frame
    unsigned int* counters;  // (B, KV_H)
    int* status;
};

__device__ __forceinline__ float load_q(const void* q, int dtype, int64_t i) {
    if (dtype == ALLOYB_F16) return __half2float(static_cast<const __half*>(q)[i]);
    if (dtype == ALLOYB_BF16) {
        // the reference computes decode attention with q in fp16 (torch/ops/kv_quant.py:175-180)
        return __half2float(__float2half_rn(__bfloat162float(static_cast<const __nv_bfloat16*>(q)[i])));
    }
    return __half2float(__float2half_rn(static_cast<const float*>(q)[i]));
}

__device__ __forceinline__ void store_out(void* out, int dtype, int64_t i, float v) {
    if (dtype == ALLOYB_F16) static_cast<__half*>(out)[i] = __float2half_rn(v);
    else if (dtype == ALLOYB_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else static_cast<float*>(out)[i] = v;
}

// Row base of token j for (b, h) in each layout.  Paged: returns nullptr for a bad page.
template <int LAYOUT, int D>
struct RowRef {
    const uint8_t* codes;    // f16: the fp16 row; split: int8 codes; paged: 34-byte blocks
    const __half* scales;    // split only
};

template <int LAYOUT, int D>
__device__ __forceinline__ RowRef<LAYOUT, D> row_ref(const KVPtrs& kv, int which, int b, int h,
                                                     int KV_H, int j, int* status) {
    RowRef<LAYOUT, D> r;
    r.scales = nullptr;
    if (LAYOUT == ALLOYB_KV_F16) {
        const __half* base = static_cast<const __half*>(which ? kv.v0 : kv.k0);
        r.codes = reinterpret_cast<const uint8_t*>(
            base + ((static_cast<int64_t>(b) * KV_H + h) * kv.S_max + j) * D);
    } else if (LAYOUT == ALLOYB_KV_Q8_SPLIT) {
        const int64_t row = (static_cast<int64_t>(b) * KV_H + h) * kv.S_max + j;
        r.codes = static_cast<const uint8_t*>(which ? kv.v0 : kv.k0) + row * D;
        r.scales = static_cast<const __half*>(which ? kv.v1 : kv.k1) + row * (D / 32);
    } else {
        const int32_t* table = static_cast<const int32_t*>(kv.k1);
        const int64_t page = table[static_cast<int64_t>(b) * kv.max_pages + j / PAGE_TOKENS];
        if (page < 0 || page >= kv.num_pages) {
            if (status) atomicOr(status, KV_STATUS_PAGE_RANGE);
            r.codes = nullptr;
        } else {
            r.codes = static_cast<const uint8_t*>(kv.k0) +
                      paged_row_offset(page, which, h, j % PAGE_TOKENS, KV_H, D);
        }
    }
    return r;
}

// s[g] = sum_d q[g][d] * K[j][d] for the lane's token (q pre-scaled, in shared memory).
template <int LAYOUT, int D, int G>
__device__ __forceinline__ void score_row(const RowRef<LAYOUT, D>& r, const float* __restrict__ qs,
                                          float (&s)[G]) {
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    if (r.codes == nullptr) return;
    if (LAYOUT == ALLOYB_KV_F16) {
        const uint4* p = reinterpret_cast<const uint4*>(r.codes);
#pragma unroll 4
        for (int i = 0; i < D / 8; ++i) {
            const uint4 v = __ldg(p + i);
            const __half2* h2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h2[e]);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    s[g] = fmaf(qs[g * D + i * 8 + 2 * e], f.x, s[g]);
                    s[g] = fmaf(qs[g * D + i * 8 + 2 * e + 1], f.y, s[g]);
                }
            }
        }
    } else {
#pragma unroll
        for (int blk = 0; blk < D / 32; ++blk) {
            float ks;
            float part[G];
#pragma unroll
            for (int g = 0; g < G; ++g) part[g] = 0.f;
            if (LAYOUT == ALLOYB_KV_Q8_SPLIT) {
                ks = __half2float(__ldg(r.scales + blk));
                const uint32_t* cw = reinterpret_cast<const uint32_t*>(r.codes + blk * 32);
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    const uint32_t cv = __ldg(cw + w);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float c = static_cast<float>(static_cast<int8_t>((cv >> (8 * e)) & 0xffu));
#pragma unroll
                        for (int g = 0; g < G; ++g)
                            part[g] = fmaf(qs[g * D + blk * 32 + w * 4 + e], c, part[g]);
                    }
                }
            } else {
                const uint16_t* bw = reinterpret_cast<const uint16_t*>(r.codes + blk * KV_BLOCK_BYTES);
                ks = half_bits_to_f32(__ldg(bw));
#pragma unroll
                for (int w = 0; w < 16; ++w) {
                    const uint32_t cv = __ldg(bw + 1 + w);
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float c = static_cast<float>(static_cast<int8_t>((cv >> (8 * e)) & 0xffu));
#pragma unroll
                        for (int g = 0; g < G; ++g)
                            part[g] = fmaf(qs[g * D + blk * 32 + w * 2 + e], c, part[g]);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = fmaf(ks, part[g], s[g]);
        }
    }
}

// Dequantised V values of token row r for this lane's DPL = D/32 consecutive dims.
template <int LAYOUT, int D>
__device__ __forceinline__ void load_v(const RowRef<LAYOUT, D>& r, int lane, float (&v)[D / 32]) {
    constexpr int DPL = D / 32;
    const int d0 = lane * DPL;
#pragma unroll
    for (int e = 0; e < DPL; ++e) v[e] = 0.f;
    if (r.codes == nullptr) return;
    if (LAYOUT == ALLOYB_KV_F16) {
        const __half* p = reinterpret_cast<const __half*>(r.codes) + d0;
        if (DPL == 4) {
            const uint2 w = __ldg(reinterpret_cast<const uint2*>(p));
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
            v[0] = a.x; v[1] = a.y; v[2 % DPL] = c.x; v[3 % DPL] = c.y;
        } else {
#pragma unroll
            for (int e = 0; e < DPL; ++e) v[e] = __half2float(__ldg(p + e));
        }
    } else if (LAYOUT == ALLOYB_KV_Q8_SPLIT) {
        const float s = __half2float(__ldg(r.scales + d0 / 32));
        const int8_t* p = reinterpret_cast<const int8_t*>(r.codes) + d0;
        if (DPL == 4) {
            const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(p));
#pragma unroll
            for (int e = 0; e < DPL; ++e)
                v[e] = s * static_cast<float>(static_cast<int8_t>((w >> (8 * (e & 3))) & 0xffu));
        } else {
#pragma unroll
            for (int e = 0; e < DPL; ++e) v[e] = s * static_cast<float>(__ldg(p + e));
        }
    } else {
        const uint8_t* blk = r.codes + (d0 / 32) * KV_BLOCK_BYTES;
        const float s = half_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(blk)));
        const int8_t* p = reinterpret_cast<const int8_t*>(blk + 2) + (d0 % 32);
#pragma unroll
        for (int e = 0; e < DPL; ++e) v[e] = s * static_cast<float>(__ldg(p + e));
    }
}

constexpr int ATTN_WARPS = 4;

// CTA = 4 warps.  The CTA's token range is cut into 32-token chunks dealt round-robin to the
// warps; each warp keeps its own online-softmax state, the four states are merged through
// shared memory, and the CTA writes ONE partial per query head.
template <int LAYOUT, int D, int G>
__global__ void __launch_bounds__(ATTN_WARPS * 32) attn_decode_kernel(AttnParams P) {
    pdl_launch_dependents();
    constexpr int DPL = D / 32;
    __shared__ float qs[G * D];
    __shared__ float sm_m[ATTN_WARPS][G], sm_l[ATTN_WARPS][G];
    __shared__ float sm_o[ATTN_WARPS][G][D];
    __shared__ int s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    pdl_wait();
    int pos = P.pos[P.pos_count == 1 ? 0 : b];
    if (pos >= P.kv.S_max) {
        if (threadIdx.x == 0 && P.status) atomicOr(P.status, KV_STATUS_POS_RANGE);
        pos = P.kv.S_max - 1;
    }
    const int len = pos + 1;                  // positions [0, pos]; pos < 0 -> empty
    for (int i = threadIdx.x; i < G * D; i += ATTN_WARPS * 32) {
        const int g = i / D, d = i - g * D;
        qs[i] = load_q(P.q, P.q_dtype, b * P.q_bs + (kvh * G + g) * P.q_hs + d) * P.scale_log2;
    }
    __syncthreads();

    int chunk = (len + P.splits - 1) / P.splits;
    chunk = (chunk + 31) & ~31;
    const int t0 = split * chunk;
    const int t1 = min(len, t0 + chunk);

    float m[G], l[G], o[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = NEG_BIG;
        l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < DPL; ++e) o[g][e] = 0.f;
    }

    for (int c0 = t0 + warp * 32; c0 < t1; c0 += ATTN_WARPS * 32) {
        const int j = c0 + lane;
        const bool valid = j < t1;
        float s[G];
        if (valid) {
            const RowRef<LAYOUT, D> kr = row_ref<LAYOUT, D>(P.kv, 0, b, kvh, P.KV_H, j, P.status);
            score_row<LAYOUT, D, G>(kr, qs, s);
        }
        float p[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float sv = valid ? s[g] : NEG_BIG;
            const float mn = fmaxf(m[g], warp_max(sv));
            const float alpha = exp2f(m[g] - mn);
            p[g] = valid ? exp2f(sv - mn) : 0.f;
            l[g] = l[g] * alpha + warp_sum(p[g]);
            m[g] = mn;
#pragma unroll
            for (int e = 0; e < DPL; ++e) o[g][e] *= alpha;
        }
        // P*V: the lanes own DPL dims each; token rows are fetched eight at a time so that eight
        // independent loads are in flight before the first multiply-add needs its data
        const int cnt = min(32, t1 - c0);
        for (int tb = 0; tb < cnt; tb += 8) {
            float v[8][DPL];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (tb + u < cnt) {
                    const RowRef<LAYOUT, D> vr =
                        row_ref<LAYOUT, D>(P.kv, 1, b, kvh, P.KV_H, c0 + tb + u, nullptr);
                    load_v<LAYOUT, D>(vr, lane, v[u]);
                } else {
#pragma unroll
                    for (int e = 0; e < DPL; ++e) v[u][e] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pt = __shfl_sync(0xffffffffu, p[g], (tb + u) & 31);
#pragma unroll
                    for (int e = 0; e < DPL; ++e) o[g][e] = fmaf(pt, v[u][e], o[g][e]);
                }
            }
        }
    }

    // merge the four warps
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
        for (int e = 0; e < DPL; ++e) sm_o[warp][g][lane * DPL + e] = o[g][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * D; i += ATTN_WARPS * 32) {
        const int g = i / D, d = i - g * D;
        float mx = NEG_BIG;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) mx = fmaxf(mx, sm_m[w][g]);
        float lt = 0.f, ot = 0.f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) {
            const float sc = exp2f(sm_m[w][g] - mx);
            lt = fmaf(sm_l[w][g], sc, lt);
            ot = fmaf(sm_o[w][g][d], sc, ot);
        }
        const int h = kvh * G + g;
        const int64_t pi = (static_cast<int64_t>(b) * P.H + h) * P.splits + split;
        P.part_o[pi * D + d] = lt > 0.f ? ot / lt : 0.f;
        if (d == 0) P.part_lse[pi] = lt > 0.f ? mx + log2f(lt) : NEG_BIG;
    }

    // last CTA of this (b, kv head) merges the splits
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(P.counters + b * P.KV_H + kvh, 1u);
        s_last = (prev == static_cast<unsigned int>(P.splits) - 1u);
        if (s_last) P.counters[b * P.KV_H + kvh] = 0u;   // ready for the next call
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < G * D; i += ATTN_WARPS * 32) {
        const int g = i / D, d = i - g * D;
        const int h = kvh * G + g;
        const int64_t base = (static_cast<int64_t>(b) * P.H + h) * P.splits;
        float mx = NEG_BIG;
        for (int s2 = 0; s2 < P.splits; ++s2) mx = fmaxf(mx, __ldcg(P.part_lse + base + s2));
        float acc = 0.f, wsum = 0.f;
        for (int s2 = 0; s2 < P.splits; ++s2) {
            const float lse = __ldcg(P.part_lse + base + s2);
            if (lse <= 0.5f * NEG_BIG) continue;
            const float w = exp2f(lse - mx);
            wsum += w;
            acc = fmaf(w, __ldcg(P.part_o + (base + s2) * D + d), acc);
        }
        store_out(P.out, P.q_dtype, (static_cast<int64_t>(b) * P.H + h) * D + d,
                  wsum > 0.f ? acc / wsum : 0.f);
    }
}

template <int LAYOUT, int D>
static int launch_attn_g(const AttnParams& P, int G, cudaStream_t st) {
    dim3 grid(P.splits, P.KV_H, P.B);
    switch (G) {
        case 1: launch_pdl(attn_decode_kernel<LAYOUT, D, 1>, dim3(grid), dim3(ATTN_WARPS * 32), 0, st, P); break;
        case 2: launch_pdl(attn_decode_kernel<LAYOUT, D, 2>, dim3(grid), dim3(ATTN_WARPS * 32), 0, st, P); break;
        case 4: launch_pdl(attn_decode_kernel<LAYOUT, D, 4>, dim3(grid), dim3(ATTN_WARPS * 32), 0, st, P); break;
        case 8: launch_pdl(attn_decode_kernel<LAYOUT, D, 8>, dim3(grid), dim3(ATTN_WARPS * 32), 0, st, P); break;
        default: return ALLOYB_E_SHAPE;
    }
    return check_launch();
}

template <int LAYOUT>
static int launch_attn_d(const AttnParams& P, int D, int G, cudaStream_t st) {
    switch (D) {
        case 64: return launch_attn_g<LAYOUT, 64>(P, G, st);
        case 128: return launch_attn_g<LAYOUT, 128>(P, G, st);
        case 256: return launch_attn_g<LAYOUT, 256>(P, G, st);
        default: return ALLOYB_E_SHAPE;
    }
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace alloyb

using namespace alloyb;

// workspace: [status word + counters | part_lse | part_o]
extern "C" size_t alloyb_attn_workspace_bytes(int B, int H, int D) {
    if (B <= 0 || H <= 0 || D <= 0) return 0;
    const size_t bh = static_cast<size_t>(B) * H;
    return align_up(256 + bh * sizeof(unsigned int), 256) +
           align_up(bh * ATTN_MAX_SPLITS * sizeof(float), 256) +
           align_up(bh * ATTN_MAX_SPLITS * D * sizeof(float), 256);
}

// Argument checks shared by the two decode entries (nothing is launched or written before they pass).
static int attn_decode_validate(int layout, const void* q, int q_dtype, const void* k0, const void* k1,
                                const void* v0, const void* v1, const void* new_k, const void* new_v,
                                const int32_t* pos, int pos_count, const void* out, int B, int H, int KV_H,
                                int D, int S_max, int64_t num_pages, int write_kv, const void* workspace,
                                size_t workspace_bytes) {
    if (!q || !k0 || !pos || !out || !workspace) return ALLOYB_E_NULL;
    if (B <= 0 || H <= 0 || KV_H <= 0 || H % KV_H || D <= 0 || D % 32 || S_max <= 0)
        return ALLOYB_E_SHAPE;
    if (pos_count != 1 && pos_count != B) return ALLOYB_E_SHAPE;
    if (q_dtype != ALLOYB_F16 && q_dtype != ALLOYB_BF16 && q_dtype != ALLOYB_F32) return ALLOYB_E_DTYPE;
    if (layout == ALLOYB_KV_F16) { if (!v0) return ALLOYB_E_NULL; }
    else if (layout == ALLOYB_KV_Q8_SPLIT) { if (!k1 || !v0 || !v1) return ALLOYB_E_NULL; }
    else if (layout == ALLOYB_KV_Q8_PAGED) {
        if (!k1) return ALLOYB_E_NULL;
        if (S_max % PAGE_TOKENS || num_pages <= 0) return ALLOYB_E_SHAPE;
    } else return ALLOYB_E_SHAPE;
    if (write_kv && (!new_k || !new_v)) return ALLOYB_E_NULL;
    if (reinterpret_cast<uintptr_t>(workspace) % 256) return ALLOYB_E_ALIGN;
    if (workspace_bytes < alloyb_attn_workspace_bytes(B, H, D)) return ALLOYB_E_WORKSPACE;
    return ALLOYB_OK;
}

// Shared by the decode entries: workspace carve-up, split count, optional append, launch.
static int attn_decode_run(int layout, const void* q, int64_t q_batch_stride, int64_t q_head_stride, int q_dtype,
                           void* k0, void* k1, void* v0, void* v1, const void* new_k, const void* new_v,
                           int64_t new_batch_stride, int64_t new_head_stride, const int32_t* pos, int pos_count,
                           void* out, int B, int H, int KV_H, int D, int S_max, int64_t num_pages, float scale,
                           int write_kv, void* workspace, void* stream, const AttnFuse* fuse) {
    cudaStream_t st = as_stream(stream);

    AttnParams P;
    P.q = q; P.q_bs = q_batch_stride; P.q_hs = q_head_stride; P.q_dtype = q_dtype;
    P.kv.k0 = k0; P.kv.k1 = k1; P.kv.v0 = v0; P.kv.v1 = v1;
    P.kv.S_max = S_max;
    P.kv.max_pages = S_max / PAGE_TOKENS;
    P.kv.num_pages = num_pages;
    P.pos = pos; P.pos_count = pos_count; P.out = out;
    P.B = B; P.H = H; P.KV_H = KV_H;
    const float sc = scale > 0.f ? scale : 1.0f / sqrtf(static_cast<float>(D));
    P.scale_log2 = sc * 1.4426950408889634f;
    const size_t bh = static_cast<size_t>(B) * H;
    char* ws = static_cast<char*>(workspace);
    P.status = reinterpret_cast<int*>(ws);
    P.counters = reinterpret_cast<unsigned int*>(ws + 256);
    ws += align_up(256 + bh * sizeof(unsigned int), 256);
    P.part_lse = reinterpret_cast<float*>(ws);
    ws += align_up(bh * ATTN_MAX_SPLITS * sizeof(float), 256);
    P.part_o = reinterpret_cast<float*>(ws);

    // Split count: the (b, kv head) pairs times the splits run in waves of as many CTAs per SM as the
    // layout's kernel keeps resident (registers: 2 for the fp16 cache, whose tiles are staged in registers,
    // 3 for the split q8_0 cache, 4 for the paged pool); a split costs its tokens (whole 64-token passes of
    // the four warps) plus a fixed start-up and merge share, and every extra split lengthens the final
    // merge.  Take the cheapest.
    const int ctas = B * KV_H;
    const int by_len = (S_max + 63) / 64;
    int max_s = by_len < ATTN_MAX_SPLITS ? by_len : ATTN_MAX_SPLITS;
    if (max_s < 1) max_s = 1;
    int splits = 1;
    int64_t best = INT64_MAX;
    const int merge_w = layout == ALLOYB_KV_F16 ? 3 : 4;       // tokens' worth of merge time per split (measured)
    const int resident = 148 * (layout == ALLOYB_KV_F16 ? 2 : (layout == ALLOYB_KV_Q8_SPLIT ? 3 : 4));
    for (int s = 1; s <= max_s; ++s) {
        const int64_t waves = (static_cast<int64_t>(ctas) * s + resident - 1) / resident;
        const int64_t per = ((S_max + s - 1) / s + 63) / 64 * 64 + 256;
        const int64_t cost = waves * per + merge_w * s;
        if (cost < best) { best = cost; splits = s; }
    }
    P.splits = splits;

    if (write_kv) {
        int rc = launch_kv_append(layout, new_k, new_v, new_batch_stride, new_head_stride, P.kv, pos,
                                  pos_count, B, KV_H, D, P.status, st);
        if (rc != ALLOYB_OK) return rc;
    }
    const int G = H / KV_H;
    if (D == 128 && G <= 8)
        return launch_attn_mma(layout, q, q_batch_stride, q_head_stride, q_dtype, P.kv, pos, pos_count, out, B, H,
                               KV_H, P.scale_log2, P.splits, P.part_o, P.part_lse, P.counters, P.status, st, fuse);
    if (fuse) return ALLOYB_NOT_TAKEN;
    switch (layout) {
        case ALLOYB_KV_F16: return launch_attn_d<ALLOYB_KV_F16>(P, D, G, st);
        case ALLOYB_KV_Q8_SPLIT: return launch_attn_d<ALLOYB_KV_Q8_SPLIT>(P, D, G, st);
        default: return launch_attn_d<ALLOYB_KV_Q8_PAGED>(P, D, G, st);
    }
}


extern "C" int alloyb_attn_decode(int layout, const void* q, int64_t q_batch_stride,
                                  int64_t q_head_stride, int q_dtype, void* k0, void* k1, void* v0,
                                  void* v1, const void* new_k, const void* new_v,
                                  int64_t new_batch_stride, int64_t new_head_stride,
                                  const int32_t* pos, int pos_count, void* out, int B, int H, int KV_H,
                                  int D, int S_max, int64_t num_pages, float scale, int write_kv,
                                  void* workspace, size_t workspace_bytes, void* stream) {
    const int vrc = attn_decode_validate(layout, q, q_dtype, k0, k1, v0, v1, new_k, new_v, pos, pos_count, out, B, H,
                                         KV_H, D, S_max, num_pages, write_kv, workspace, workspace_bytes);
    if (vrc != ALLOYB_OK) return vrc;
    return attn_decode_run(layout, q, q_batch_stride, q_head_stride, q_dtype, k0, k1, v0, v1, new_k, new_v,
                           new_batch_stride, new_head_stride, pos, pos_count, out, B, H, KV_H, D, S_max, num_pages,
                           scale, write_kv, workspace, stream, nullptr);
}

// The decode token's whole attention step in one launch: RoPE (rotate-half) of q and of the new K row, the
// append of the new K / V rows to the cache (any layout; the q8 layouts quantise them) and the attention
// itself.  Same results, bit for bit, as alloyb_rope_kv_append followed by alloyb_attn_decode with
// write_kv = 0, except that q is left unrotated in memory.  Covers fp16 q, head_dim 128, up to eight
// query heads per KV head, 16-byte-aligned q rows; anything else returns ALLOYB_NOT_TAKEN (1) and the
// caller makes the two calls.  No counterpart in the reference, which rotates in the model code and
// fuses only the cache write (metal/std/kv_quant.py:212-246).
extern "C" int alloyb_attn_decode_rope(int layout, const void* q, int64_t q_batch_stride, int64_t q_head_stride,
                                       void* k0, void* k1, void* v0, void* v1, const void* new_k, const void* new_v,
                                       int64_t new_batch_stride, int64_t new_head_stride, const int32_t* pos,
                                       int pos_count, const float* inv_freq, void* out, int B, int H, int KV_H,
                                       int D, int S_max, int64_t num_pages, float scale, void* workspace,
                                       size_t workspace_bytes, void* stream) {
    const int vrc = attn_decode_validate(layout, q, ALLOYB_F16, k0, k1, v0, v1, new_k, new_v, pos, pos_count, out, B,
                                         H, KV_H, D, S_max, num_pages, 1, workspace, workspace_bytes);
    if (vrc != ALLOYB_OK) return vrc;
    if (!inv_freq) return ALLOYB_E_NULL;
    if (D != 128 || H / KV_H > 8) return ALLOYB_NOT_TAKEN;
    if ((reinterpret_cast<uintptr_t>(q) | static_cast<uintptr_t>(q_batch_stride * 2) |
         static_cast<uintptr_t>(q_head_stride * 2)) & 15)
        return ALLOYB_NOT_TAKEN;
    AttnFuse fuse;
    fuse.inv_freq = inv_freq;
    fuse.new_k = static_cast<const __half*>(new_k);
    fuse.new_v = static_cast<const __half*>(new_v);
    fuse.new_bs = new_batch_stride;
    fuse.new_hs = new_head_stride;
    return attn_decode_run(layout, q, q_batch_stride, q_head_stride, ALLOYB_F16, k0, k1, v0, v1, new_k, new_v,
                           new_batch_stride, new_head_stride, pos, pos_count, out, B, H, KV_H, D, S_max, num_pages,
                           scale, 0, workspace, stream, &fuse);
}

// Zero the status word and completion counters of a fresh workspace (once after allocation).
extern "C" int alloyb_attn_workspace_init(void* workspace, size_t workspace_bytes, int B, int H,
                                          void* stream) {
    if (!workspace) return ALLOYB_E_NULL;
    const size_t head = 256 + static_cast<size_t>(B) * H * sizeof(unsigned int);
    if (workspace_bytes < head) return ALLOYB_E_WORKSPACE;
    const cudaError_t e = cudaMemsetAsync(workspace, 0, head, as_stream(stream));
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

// Device status word of the workspace (bit 0: position out of range, bit 1: page id out of
// range; offending accesses were skipped).  Synchronises the stream.
extern "C" int alloyb_attn_workspace_status(const void* workspace, int32_t* status_out, void* stream) {
    if (!workspace || !status_out) return ALLOYB_E_NULL;
    cudaError_t e = cudaMemcpyAsync(status_out, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                    as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

// ------------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc on the path that runs a decode step: code
// that runs inside a region where the CUDA allocator must stay quiet (a latency-critical serving
// loop with a frozen memory plan, a plugin whose host forbids allocations after start-up, a
// sandbox that only hands out the input and output buffers).  alloyb_attn_decode needs a caller-
// provided workspace for its split-K partials; this variant brings its own: a fixed array in
// device memory that is part of the library image, so every GPU that loads the library holds
// ALLOYB_ATTN_STATIC_BYTES of it until the process exits.
//
// The array is shared by every call on that device and keeps the previous call's contents.  The
// words that must start at zero (status word and completion counters) are cleared on the stream
// at the start of every call; the partials need no clearing.  Two calls that may overlap on the
// GPU (different streams, or one stream in two threads) race on the array: serialise them.
namespace alloyb {

static __device__ __align__(256) unsigned char g_attn_static_scratch[ALLOYB_ATTN_STATIC_BYTES];

constexpr int MAX_DEVICES = 64;
static void* g_attn_static_ptr[MAX_DEVICES] = {};   // device address per device ordinal

}  // namespace alloyb

extern "C" int alloyb_attn_decode_static(int layout, const void* q, int64_t q_batch_stride,
                                         int64_t q_head_stride, int q_dtype, void* k0, void* k1,
                                         void* v0, void* v1, const void* new_k, const void* new_v,
                                         int64_t new_batch_stride, int64_t new_head_stride,
                                         const int32_t* pos, int pos_count, void* out, int B, int H,
                                         int KV_H, int D, int S_max, int64_t num_pages, float scale,
                                         int write_kv, void* stream) {
    if (B <= 0 || H <= 0 || KV_H <= 0 || D <= 0) return ALLOYB_E_SHAPE;
    const size_t need = alloyb_attn_workspace_bytes(B, H, D);
    if (need == 0) return ALLOYB_E_SHAPE;
    if (need > static_cast<size_t>(ALLOYB_ATTN_STATIC_BYTES)) return ALLOYB_E_LIMIT;

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    if (dev < 0 || dev >= MAX_DEVICES) return ALLOYB_E_LIMIT;
    if (g_attn_static_ptr[dev] == nullptr) {
        // One-time set-up for this device (it is the current one).  In host code the array's name
        // is only a stand-in for the symbol; the address a kernel can use comes from the runtime.
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_cuda_error(e);
            return ALLOYB_E_CUDA;
        }
        g_attn_static_ptr[dev] = p;
    }
    void* ws = g_attn_static_ptr[dev];
    // every argument is checked before the shared array is touched
    const int vrc = attn_decode_validate(layout, q, q_dtype, k0, k1, v0, v1, new_k, new_v, pos, pos_count, out, B, H,
                                         KV_H, D, S_max, num_pages, write_kv, ws, ALLOYB_ATTN_STATIC_BYTES);
    if (vrc != ALLOYB_OK) return vrc;
    // status word + completion counters start every call at zero
    const size_t head = 256 + static_cast<size_t>(B) * H * sizeof(unsigned int);
    e = cudaMemsetAsync(ws, 0, head, as_stream(stream));
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return alloyb_attn_decode(layout, q, q_batch_stride, q_head_stride, q_dtype, k0, k1, v0, v1, new_k,
                              new_v, new_batch_stride, new_head_stride, pos, pos_count, out, B, H, KV_H,
                              D, S_max, num_pages, scale, write_kv, ws, ALLOYB_ATTN_STATIC_BYTES, stream);
}

// Status word of the most recent alloyb_attn_decode_static call on the current device (the same
// bits alloyb_attn_workspace_status reports; every static call starts it at zero).  Synchronises
// the stream.  ALLOYB_E_SHAPE before the first static call on this device.
extern "C" int alloyb_attn_static_status(int32_t* status_out, void* stream) {
    if (!status_out) return ALLOYB_E_NULL;
    int dev = -1;
    const cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    if (dev < 0 || dev >= MAX_DEVICES || g_attn_static_ptr[dev] == nullptr) return ALLOYB_E_SHAPE;
    return alloyb_attn_workspace_status(g_attn_static_ptr[dev], status_out, stream);
}

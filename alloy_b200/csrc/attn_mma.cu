// Tensor-core decode attention (head_dim 128, up to 8 query heads per KV head).
//
// A warp takes 16-token tiles.  Scores: S[head, token] = Q[head, d] * K[token, d]^T as
// mma.sync.m16n8k16 with the group's query heads as the (padded) M rows, eight tokens as N and the
// head dimension as K; the C fragment of two such products is exactly the A fragment of the
// P * V product (M = heads, K = 16 tokens, N = 8 output dims), so probabilities never leave
// registers.  The contraction index of either product may be permuted freely as long as both
// operands agree, which is used to make every thread's loads contiguous:
//   * K operand: thread (g, t) reads 8 consecutive dims of token g -> two k-steps of the S product;
//   * V operand: thread (g, t) reads 4 consecutive dims (4g..4g+3 of a 32-dim block) of its four
//     tokens and transposes them in registers; output column g of the e-th product of the block
//     is dim 32*kp + 4g + e.
// q8_0 caches: codes enter the MMA as unsigned bytes u = code + 128 in fp16 SUBNORMAL form
// (u * 2^-24, no int->float conversion); the block scale multiplies the block's partial sum
// afterwards and the +128 is taken out with sum(q) resp. sum(P') -- all in fp32.
// The paged layout (34-byte blocks, 2-byte aligned) is staged per 16-token page through shared
// memory with two bulk copies per tile; the other layouts are read straight from global memory.
// Fused form: q is rotated (RoPE, rotate-half) in registers as it is loaded, and the CTA whose token range
// holds the decode position rotates the new K row, appends it and the new V row to the cache (quantising
// for the q8 layouts) before it starts on its tiles -- the arithmetic and rounding points of the separate
// RoPE + append kernel, so results are bit-identical to the two-launch sequence.
#include <type_traits>

#include "kv.cuh"

namespace alloyb {

namespace am {

constexpr int D = 128;
constexpr int NKP = D / 32;
constexpr int WARPS = 4;
constexpr float NEG_BIG = -1.0e30f;
// Probabilities enter the P * V product as fp16 (hi + lo halves).  At long contexts a typical
// p * (block scale) is ~1e-5, inside fp16's subnormal range, where the two halves together keep
// only ~10 bits.  The A operand is therefore biased by 2^6 (taken out again in the epilogue):
// the largest possible value, 64 * 1 * 516 (the q8_0 scale of a block holding 65504), still fits.
constexpr float P_BIAS = 64.0f;
constexpr int SLAB = PAGE_TOKENS * NKP * KV_BLOCK_BYTES;     // 2176 bytes: one page of K (or V) of one head
constexpr uint32_t SPIN = 1u << 22;

__device__ int g_attn_error = 0;

struct Params {
    const void* q;
    int64_t q_bs, q_hs;
    int q_dtype;
    KVPtrs kv;
    const int32_t* pos;
    int pos_count;
    void* out;
    int B, H, KV_H, G;
    float scale_log2;
    int splits;
    float* part_o;
    float* part_lse;
    unsigned int* counters;
    int* status;
    AttnFuse fuse;           // valid when fused != 0: RoPE of q / new K and the K / V append happen in here
    int fused;
};

__device__ __forceinline__ uint32_t s32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    // rows 8..15 of A are zero (at most 8 query heads): a1 = a3 = 0
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}
// The same product onto a zero accumulator (the zeros are the instruction's own operand: no register is set up).
__device__ __forceinline__ void mma_z(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm("{\n\t.reg .f32 z;\n\tmov.f32 z, 0f00000000;\n\t"
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {z,z,z,z};\n\t}"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}
// Cache loads: through the read-only path, or (fused form, where this kernel itself wrote the newest row)
// from L2.
template <typename T>
__device__ __forceinline__ T ldkv(const T* p, bool from_l2) {
    return from_l2 ? __ldcg(p) : __ldg(p);
}
// Shared loads by 32-bit shared-window address (a tile's base is converted once; the rest is 32-bit arithmetic
// with constant offsets).
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
// n (1 or 2) 32-bit words starting at a 2-byte-aligned shared address.  Whether the address is 4-byte
// aligned is known at compile time from the block index (a row of 34-byte blocks starts 4-byte aligned, the
// codes of block kp at 34 * kp + 2): HALF = true reads across the word boundary with funnel shifts.
template <bool HALF>
__device__ __forceinline__ void lds_words_align2(uint32_t p, uint32_t& w0, uint32_t& w1, bool two) {
    if (HALF) {
        const uint32_t base = p - 2;
        const uint32_t x0 = lds32(base), x1 = lds32(base + 4);
        w0 = __funnelshift_r(x0, x1, 16);
        if (two) w1 = __funnelshift_r(x1, lds32(base + 8), 16);
    } else {
        w0 = lds32(p);
        if (two) w1 = lds32(p + 4);
    }
}
__device__ __forceinline__ void bar_init(uint64_t* b, uint32_t n) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n));
}
__device__ __forceinline__ void bar_expect(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* b, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(s32(b)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (i > 32) __nanosleep(64);
    }
    atomicExch(&g_attn_error, 4);
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     s32(dst)),
                 "l"(src), "r"(bytes), "r"(s32(bar))
                 : "memory");
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
__device__ __forceinline__ float q_elem(const void* q, int dtype, int64_t i) {
    if (dtype == ALLOYB_F16) return __half2float(static_cast<const __half*>(q)[i]);
    if (dtype == ALLOYB_BF16)
        return __half2float(__float2half_rn(__bfloat162float(static_cast<const __nv_bfloat16*>(q)[i])));
    return __half2float(__float2half_rn(static_cast<const float*>(q)[i]));
}
__device__ __forceinline__ void out_elem(void* out, int dtype, int64_t i, float v) {
    if (dtype == ALLOYB_F16) static_cast<__half*>(out)[i] = __float2half_rn(v);
    else if (dtype == ALLOYB_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else static_cast<float*>(out)[i] = v;
}

struct WarpStage {                       // paged layout only
    uint8_t k[2][SLAB];
    uint8_t v[2][SLAB];
};

template <int LAYOUT>
__global__ void __launch_bounds__(WARPS * 32) attn_mma_kernel(const Params P) {
    pdl_launch_dependents();
    constexpr bool Q8 = LAYOUT != ALLOYB_KV_F16;
    constexpr bool PAGED = LAYOUT == ALLOYB_KV_Q8_PAGED;
    __shared__ float sm_m[WARPS][8], sm_l[WARPS][8];
    __shared__ int s_last;
    // the page stages (paged layout) and, after the tile loop, the per-warp output rows share one buffer
    constexpr int O_BYTES = WARPS * 8 * D * 4;
    constexpr int STAGE_BYTES = PAGED ? WARPS * static_cast<int>(sizeof(WarpStage)) : 0;
    __shared__ __align__(16) uint8_t sm_buf[O_BYTES > STAGE_BYTES ? O_BYTES : STAGE_BYTES];
    __shared__ __align__(8) uint64_t sm_bar[WARPS][2];
    uint8_t* sm_stage = sm_buf;
    float (*sm_o)[8][D] = reinterpret_cast<float (*)[8][D]>(sm_buf);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int G = P.G;
    if (PAGED && lane == 0) {
        bar_init(&sm_bar[warp][0], 1);
        bar_init(&sm_bar[warp][1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    pdl_wait();
    int pos = P.pos[P.pos_count == 1 ? 0 : b];
    const int pos_in = pos;                           // as given: the rotation angle and the append use it
    if (pos >= P.kv.S_max) {
        if (threadIdx.x == 0 && P.status) atomicOr(P.status, KV_STATUS_POS_RANGE);
        pos = P.kv.S_max - 1;
    }
    const int len = pos + 1;
    // this CTA's token range (whole 64-token passes of the four warps per split)
    int chunk = (len + P.splits - 1) / P.splits;
    chunk = (chunk + 63) & ~63;
    const int t0 = split * chunk;
    const int t1 = min(len, t0 + chunk);
    const int n_tiles = t1 > t0 ? (t1 - t0 + 15) / 16 : 0;

    // q (and the angles' frequencies) are requested first: nothing below has to wait for them in turn
    const bool q_vec = P.q_dtype == ALLOYB_F16 && ((reinterpret_cast<uintptr_t>(P.q) | (P.q_bs * 2) | (P.q_hs * 2)) & 15) == 0;
    uint4 qraw[NKP];
    float freq_own[2] = {0.f, 0.f};
    if (q_vec) {
        // eight consecutive fp16 of head g per 32-dim block: one 16-byte load each
#pragma unroll
        for (int kp = 0; kp < NKP; ++kp) {
            const int64_t base = b * P.q_bs + static_cast<int64_t>(kvh * G + g) * P.q_hs + 32 * kp + 8 * t;
            qraw[kp] = make_uint4(0u, 0u, 0u, 0u);
            if (g < G) qraw[kp] = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(P.q) + base));
        }
        if (P.fused) {
#pragma unroll
            for (int kp = 0; kp < 2; ++kp) freq_own[kp] = __ldg(P.fuse.inv_freq + 32 * kp + 8 * t + g);
        }
    }

    if (P.fused && pos_in >= t0 && pos_in < t0 + chunk && pos_in >= 0 && pos_in < P.kv.S_max) {
        // ---- the decode token's K / V rows: rotate K, append both (this CTA reads them back below)
        if (warp < 2) {
            // pair-warp `warp`: rotation pairs (j, j + 64), j = 32 * warp + lane = blocks warp and warp + 2
            const int j = 32 * warp + lane;
            float sn, cs;
            sincosf(static_cast<float>(pos_in) * P.fuse.inv_freq[j], &sn, &cs);
            const __half* base = P.fuse.new_k + b * P.fuse.new_bs + kvh * P.fuse.new_hs;
            const float x1 = __half2float(base[j]), x2 = __half2float(base[j + D / 2]);
            store_kv_block<LAYOUT>(P.kv, 0, b, kvh, pos_in, warp, lane,
                                   __float2half_rn(__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn))), P.KV_H, D, P.status);
            store_kv_block<LAYOUT>(P.kv, 0, b, kvh, pos_in, warp + 2, lane,
                                   __float2half_rn(__fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn))), P.KV_H, D, P.status);
        }
        store_kv_block<LAYOUT>(P.kv, 1, b, kvh, pos_in, warp, lane,
                               P.fuse.new_v[b * P.fuse.new_bs + kvh * P.fuse.new_hs + 32 * warp + lane], P.KV_H, D, P.status);
        // this CTA reads the rows back: the barrier orders its own loads behind its stores; the paged tiles come
        // in by bulk copies, which sit behind a device-wide fence and one between the two memory proxies
        if (PAGED) {
            __threadfence();
            asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        __syncthreads();
    }

    // fp16 cache: a tile's K and V words are requested a phase ahead of their use -- the first tile's before the
    // q fragments are built, the next tile's K after this tile's scores, its V after this tile's products
    const bool fresh = P.fused != 0;
    const int64_t head_row = (static_cast<int64_t>(b) * P.KV_H + kvh) * P.kv.S_max;
    uint4 kreg[2][NKP];
    uint2 vreg[NKP][4];
    auto load_k = [&](int tok0) {
#pragma unroll
        for (int tb = 0; tb < 2; ++tb) {
            const int tok = min(tok0 + 8 * tb + g, t1 - 1);
            const uint4* kr = reinterpret_cast<const uint4*>(static_cast<const __half*>(P.kv.k0) + (head_row + tok) * D) + t;
#pragma unroll
            for (int kp = 0; kp < NKP; ++kp) kreg[tb][kp] = ldkv(kr + kp * 4, fresh);
        }
    };
    auto load_v = [&](int tok0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int vt = min(tok0 + (i >> 1) * 8 + 2 * t + (i & 1), t1 - 1);
            const uint2* vr = reinterpret_cast<const uint2*>(static_cast<const __half*>(P.kv.v0) + (head_row + vt) * D + 4 * g);
#pragma unroll
            for (int kp = 0; kp < NKP; ++kp) vreg[kp][i] = ldkv(vr + kp * 8, fresh);
        }
    };
    if (!Q8 && warp < n_tiles) {
        load_k(t0 + warp * 16);
        load_v(t0 + warp * 16);
    }

    // ---- Q fragments (rows = heads of this group; rows >= G are zero) and per-block sums of q
    uint32_t qa[NKP][2][2];
    float qsum[NKP];
    if (q_vec) {
        if (P.fused) {
            // rotate-half RoPE in registers: dims d = 32 kp + 8 t + e (kp = 0, 1) pair with d + 64 (kp + 2).
            // The eight lanes of a column t need the same eight angles: lane (g, t) evaluates e = g and
            // the values go round by shuffles.
#pragma unroll
            for (int kp = 0; kp < 2; ++kp) {
                __half* lo = reinterpret_cast<__half*>(&qraw[kp]);
                __half* hi = reinterpret_cast<__half*>(&qraw[kp + 2]);
                float sn_own, cs_own;
                sincosf(static_cast<float>(pos_in) * freq_own[kp], &sn_own, &cs_own);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float sn = __shfl_sync(0xffffffffu, sn_own, e * 4 + t);
                    const float cs = __shfl_sync(0xffffffffu, cs_own, e * 4 + t);
                    const float x1 = __half2float(lo[e]), x2 = __half2float(hi[e]);
                    lo[e] = __float2half_rn(__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn)));
                    hi[e] = __float2half_rn(__fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn)));
                }
            }
        }
    }
#pragma unroll
    for (int kp = 0; kp < NKP; ++kp) {
        float s = 0.f;
        const int64_t base = b * P.q_bs + static_cast<int64_t>(kvh * G + g) * P.q_hs + 32 * kp + 8 * t;
        if (q_vec) {
            const uint4 v = qraw[kp];
            qa[kp][0][0] = v.x;
            qa[kp][0][1] = v.y;
            qa[kp][1][0] = v.z;
            qa[kp][1][1] = v.w;
            const float2 a = unpack_h2(v.x), b2 = unpack_h2(v.y), c = unpack_h2(v.z), d2 = unpack_h2(v.w);
            s = ((a.x + a.y) + (b2.x + b2.y)) + ((c.x + c.y) + (d2.x + d2.y));
        } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (g < G) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] = q_elem(P.q, P.q_dtype, base + 4 * j + e);
                }
                qa[kp][j][0] = pack_h2(v[0], v[1]);
                qa[kp][j][1] = pack_h2(v[2], v[3]);
                s += (v[0] + v[1]) + (v[2] + v[3]);
            }
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        qsum[kp] = s;
    }

    float m_run = NEG_BIG, l_run = 0.f;               // for head g (replicated over t)
    float o[NKP * 4][2];                              // [(kp, e)][column 2t / 2t+1]
    float ocorr[NKP];
    float zz2 = 0.f, zz3 = 0.f;                       // rows 8..15 of every C fragment (always 0)
#pragma unroll
    for (int i = 0; i < NKP * 4; ++i) o[i][0] = o[i][1] = 0.f;
#pragma unroll
    for (int kp = 0; kp < NKP; ++kp) ocorr[kp] = 0.f;

    WarpStage* st = reinterpret_cast<WarpStage*>(sm_stage) + (PAGED ? warp : 0);
    const int32_t* table = static_cast<const int32_t*>(P.kv.k1) + static_cast<int64_t>(b) * P.kv.max_pages;

    auto issue_page = [&](int tile_idx, int slot) {
        // lane 0: both slabs of the page that holds tokens [tile*16, tile*16+16)
        const int tok0 = t0 + tile_idx * 16;
        int64_t page = table[tok0 / PAGE_TOKENS];
        if (page < 0 || page >= P.kv.num_pages) {
            if (P.status) atomicOr(P.status, KV_STATUS_PAGE_RANGE);
            page = 0;                                  // stay in bounds; the tile's tokens are masked below
        }
        const uint8_t* pool = static_cast<const uint8_t*>(P.kv.k0);
        bar_expect(&sm_bar[warp][slot], 2 * SLAB);
        bulk_g2s(st->k[slot], pool + paged_row_offset(page, 0, kvh, 0, P.KV_H, D), SLAB, &sm_bar[warp][slot]);
        bulk_g2s(st->v[slot], pool + paged_row_offset(page, 1, kvh, 0, P.KV_H, D), SLAB, &sm_bar[warp][slot]);
    };

    bool ok = true;
    int n_mine = 0;
    if (PAGED && warp < n_tiles && lane == 0) issue_page(warp, 0);
    for (int tile = warp; tile < n_tiles; tile += WARPS, ++n_mine) {
        const int tok0 = t0 + tile * 16;
        const int slot = n_mine & 1;
        if (PAGED) {
            if (tile + WARPS < n_tiles && lane == 0) issue_page(tile + WARPS, slot ^ 1);
            if (ok) ok = bar_wait(&sm_bar[warp][slot], (n_mine >> 1) & 1);
            if (!ok) continue;
        }
        // A tile whose sixteen tokens all lie below t1 (every tile but the last one of the sequence) takes the
        // FULL form of the body, without the per-token range tests and address clamps.
        // paged tiles: the lane's base addresses inside this slot's two slabs
        const uint32_t k_slab = PAGED ? s32(st->k[slot]) : 0u, v_slab = PAGED ? s32(st->v[slot]) : 0u;
        const uint32_t k_code0 = k_slab + g * (NKP * KV_BLOCK_BYTES) + 2 + 8 * t;         // codes of token g, bytes 8t..
        const uint32_t k_scale0 = k_slab + 2 * t * (NKP * KV_BLOCK_BYTES);               // scales of tokens 2t, 2t + 1
        const uint32_t v_row0 = v_slab + 2 * t * (NKP * KV_BLOCK_BYTES);                 // rows of tokens 2t, 2t + 1
        auto tile_body = [&](auto full_c) {
        constexpr bool FULL = decltype(full_c)::value;
        // ---------------- S = Q K^T
        float s[2][2];
#pragma unroll
        for (int tb = 0; tb < 2; ++tb) {
            const int tok = FULL ? tok0 + 8 * tb + g : min(tok0 + 8 * tb + g, t1 - 1);   // B column of this thread
            float sc[2] = {0.f, 0.f};
            if (!Q8) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int kp = 0; kp < NKP; ++kp) {
                    const uint4 kv = kreg[tb][kp];
                    mma(c, qa[kp][0][0], qa[kp][0][1], kv.x, kv.y);
                    mma(c, qa[kp][1][0], qa[kp][1][1], kv.z, kv.w);
                }
                sc[0] = c[0];
                sc[1] = c[1];
                zz2 = c[2];
                zz3 = c[3];
            } else {
#pragma unroll
                for (int kp = 0; kp < NKP; ++kp) {
                    uint32_t w0, w1;
                    float ks[2];
                    if (PAGED) {
                        const uint32_t kc = k_code0 + (8 * tb) * (NKP * KV_BLOCK_BYTES) + kp * KV_BLOCK_BYTES;
                        if (kp & 1) lds_words_align2<false>(kc, w0, w1, true);      // 34 * kp + 2 is a multiple of 4
                        else lds_words_align2<true>(kc, w0, w1, true);
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            ks[e] = (FULL || tok0 + 8 * tb + 2 * t + e < t1)
                                        ? half_bits_to_f32(lds16(k_scale0 + (8 * tb + e) * (NKP * KV_BLOCK_BYTES) + kp * KV_BLOCK_BYTES))
                                        : 0.f;
                    } else {
                        const uint2 cw = ldkv(reinterpret_cast<const uint2*>(static_cast<const int8_t*>(P.kv.k0) + (head_row + tok) * D + 32 * kp + 8 * t), fresh);
                        w0 = cw.x;
                        w1 = cw.y;
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int tk = FULL ? tok0 + 8 * tb + 2 * t + e : min(tok0 + 8 * tb + 2 * t + e, t1 - 1);
                            ks[e] = __half2float(ldkv(static_cast<const __half*>(P.kv.k1) + (head_row + tk) * NKP + kp, fresh));
                        }
                    }
                    const uint32_t u0 = w0 ^ 0x80808080u, u1 = w1 ^ 0x80808080u;
                    float c[4];
                    mma_z(c, qa[kp][0][0], qa[kp][0][1], prmt(u0, 0u, 0x4140u), prmt(u0, 0u, 0x4342u));
                    mma(c, qa[kp][1][0], qa[kp][1][1], prmt(u1, 0u, 0x4140u), prmt(u1, 0u, 0x4342u));
                    sc[0] = fmaf(ks[0], fmaf(c[0], 16777216.0f, -128.0f * qsum[kp]), sc[0]);
                    sc[1] = fmaf(ks[1], fmaf(c[1], 16777216.0f, -128.0f * qsum[kp]), sc[1]);
                }
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool valid = FULL || tok0 + 8 * tb + 2 * t + e < t1;
                s[tb][e] = valid ? sc[e] * P.scale_log2 : NEG_BIG;
            }
        }
        if (!Q8 && tile + WARPS < n_tiles) load_k(tok0 + WARPS * 16);
        // ---------------- online softmax for head g (the four lanes of a group hold the 16 tokens)
        float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float alpha = exp2f(m_run - m_new);
        float p[2][2];
        float ls = 0.f;
#pragma unroll
        for (int tb = 0; tb < 2; ++tb)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                p[tb][e] = (FULL || s[tb][e] > 0.5f * NEG_BIG) ? exp2f(s[tb][e] - m_new) : 0.f;
                ls += p[tb][e];
            }
        ls += __shfl_xor_sync(0xffffffffu, ls, 1);
        ls += __shfl_xor_sync(0xffffffffu, ls, 2);
        l_run = l_run * alpha + ls;
        m_run = m_new;
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
            for (int i = 0; i < NKP * 4; ++i) {
                o[i][0] *= alpha;
                o[i][1] *= alpha;
            }
#pragma unroll
            for (int kp = 0; kp < NKP; ++kp) ocorr[kp] *= alpha;
        }
        // ---------------- O += P V
        int vtok[4];                                   // this thread's four contraction tokens
#pragma unroll
        for (int i = 0; i < 4; ++i)
            vtok[i] = FULL ? tok0 + (i >> 1) * 8 + 2 * t + (i & 1) : min(tok0 + (i >> 1) * 8 + 2 * t + (i & 1), t1 - 1);
        // P enters the tensor core as fp16 hi + lo halves (two products), which keeps ~22 bits of it
        const float pb[4] = {p[0][0] * P_BIAS, p[0][1] * P_BIAS, p[1][0] * P_BIAS, p[1][1] * P_BIAS};
        uint32_t pa0 = pack_h2(pb[0], pb[1]), pa2 = pack_h2(pb[2], pb[3]);
        uint32_t pl0, pl2;
        {
            const float2 r0 = unpack_h2(pa0), r2 = unpack_h2(pa2);
            pl0 = pack_h2(pb[0] - r0.x, pb[1] - r0.y);
            pl2 = pack_h2(pb[2] - r2.x, pb[3] - r2.y);
        }
#pragma unroll
        for (int kp = 0; kp < NKP; ++kp) {
            uint32_t b0[4], b1[4];                     // B fragments of the four products e = 0..3
            if (!Q8) {
                const uint2 (&w)[4] = vreg[kp];
                b0[0] = prmt(w[0].x, w[1].x, 0x5410u); b0[1] = prmt(w[0].x, w[1].x, 0x7632u);
                b0[2] = prmt(w[0].y, w[1].y, 0x5410u); b0[3] = prmt(w[0].y, w[1].y, 0x7632u);
                b1[0] = prmt(w[2].x, w[3].x, 0x5410u); b1[1] = prmt(w[2].x, w[3].x, 0x7632u);
                b1[2] = prmt(w[2].y, w[3].y, 0x5410u); b1[3] = prmt(w[2].y, w[3].y, 0x7632u);
            } else {
                uint32_t w[4];
                float vs[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (PAGED) {
                        const uint32_t row = v_row0 + ((i >> 1) * 8 + (i & 1)) * (NKP * KV_BLOCK_BYTES) + kp * KV_BLOCK_BYTES;
                        uint32_t dummy;
                        if (kp & 1) lds_words_align2<false>(row + 2 + 4 * g, w[i], dummy, false);
                        else lds_words_align2<true>(row + 2 + 4 * g, w[i], dummy, false);
                        vs[i] = (FULL || tok0 + (i >> 1) * 8 + 2 * t + (i & 1) < t1) ? half_bits_to_f32(lds16(row)) : 0.f;
                    } else {
                        w[i] = ldkv(reinterpret_cast<const uint32_t*>(static_cast<const int8_t*>(P.kv.v0) + (head_row + vtok[i]) * D + 32 * kp + 4 * g), fresh);
                        vs[i] = __half2float(ldkv(static_cast<const __half*>(P.kv.v1) + (head_row + vtok[i]) * NKP + kp, fresh));
                    }
                }
                // product e takes byte e of the four words: a byte permute puts the codes of two tokens into the
                // low bytes of the two halves, one logic op clears the high bytes and adds the 128
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint32_t sel = 0x4400u + 0x1111u * e;
                    b0[e] = (prmt(w[0], w[1], sel) & 0x00ff00ffu) ^ 0x00800080u;
                    b1[e] = (prmt(w[2], w[3], sel) & 0x00ff00ffu) ^ 0x00800080u;
                }
                // P' = p * (block scale of the token) as fp16 hi + lo; keep its sum for the +128
                const float f0 = pb[0] * vs[0], f1 = pb[1] * vs[1], f2 = pb[2] * vs[2], f3 = pb[3] * vs[3];
                pa0 = pack_h2(f0, f1);
                pa2 = pack_h2(f2, f3);
                const float2 r0 = unpack_h2(pa0), r2 = unpack_h2(pa2);
                pl0 = pack_h2(f0 - r0.x, f1 - r0.y);
                pl2 = pack_h2(f2 - r2.x, f3 - r2.y);
                // (hi + lo equals f to 2^-22: below what the offset's factor 128 could make visible)
                ocorr[kp] += (f0 + f1) + (f2 + f3);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (Q8) {
                    // Codes carry a +128 offset, so the accumulator would grow ~100x faster than the
                    // signal it holds; the tensor core's accumulate step truncates, and over thousands
                    // of tiles that bias reached 1e-3 of the output.  Each tile's product therefore
                    // starts from zero and is added to the running sum on the CUDA cores (round to
                    // nearest), where the offset is later taken out through ocorr.
                    float c[4];
                    mma_z(c, pa0, pa2, b0[e], b1[e]);
                    mma(c, pl0, pl2, b0[e], b1[e]);
                    o[kp * 4 + e][0] += c[0];
                    o[kp * 4 + e][1] += c[1];
                } else {
                    float c[4] = {o[kp * 4 + e][0], o[kp * 4 + e][1], zz2, zz3};
                    mma(c, pa0, pa2, b0[e], b1[e]);
                    mma(c, pl0, pl2, b0[e], b1[e]);
                    o[kp * 4 + e][0] = c[0];
                    o[kp * 4 + e][1] = c[1];
                    zz2 = c[2];
                    zz3 = c[3];
                }
            }
        }
        if (!Q8 && tile + WARPS < n_tiles) load_v(tok0 + WARPS * 16);
        };
        if (tok0 + 16 <= t1) tile_body(std::true_type{});
        else tile_body(std::false_type{});
        __syncwarp();
    }
    if (PAGED && !ok) {
        for (uint32_t i = 0; i < 1024; ++i) __nanosleep(512);        // let copies in flight land
    }

    // ---- this warp's state -> shared memory (head g; the thread's dims are 32kp + 4(2t+c) + e)
    if (Q8) {
#pragma unroll
        for (int kp = 0; kp < NKP; ++kp) {
            float cs = ocorr[kp];
            cs += __shfl_xor_sync(0xffffffffu, cs, 1);
            cs += __shfl_xor_sync(0xffffffffu, cs, 2);
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    o[kp * 4 + e][c] = fmaf(o[kp * 4 + e][c], 16777216.0f / P_BIAS, (-128.0f / P_BIAS) * cs);
        }
    } else {
#pragma unroll
        for (int i = 0; i < NKP * 4; ++i) {
            o[i][0] *= 1.0f / P_BIAS;
            o[i][1] *= 1.0f / P_BIAS;
        }
    }
    __syncthreads();                                   // every warp is done with the page stages
    if (t == 0) { sm_m[warp][g] = m_run; sm_l[warp][g] = l_run; }
#pragma unroll
    for (int kp = 0; kp < NKP; ++kp)
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int c = 0; c < 2; ++c) sm_o[warp][g][32 * kp + 4 * (2 * t + c) + e] = o[kp * 4 + e][c];
    __syncthreads();

    // ---- merge the four warps, write the split's partial, let the last CTA combine the splits
    // per (warp, head) rescale factor once: exp2(m_w - max) / sum_w l_w exp2(m_w - max)
    if (threadIdx.x < G) {
        const int hg = threadIdx.x;
        float mx = NEG_BIG;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, sm_m[w][hg]);
        float sc[WARPS], lt = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            sc[w] = exp2f(sm_m[w][hg] - mx);
            lt = fmaf(sm_l[w][hg], sc[w], lt);
        }
        const float inv = lt > 0.f ? 1.0f / lt : 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) sm_l[w][hg] = sc[w] * inv;       // sm_l now holds the factors
        const int64_t pi = (static_cast<int64_t>(b) * P.H + kvh * G + hg) * P.splits + split;
        P.part_lse[pi] = lt > 0.f ? mx + log2f(lt) : NEG_BIG;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * (D / 4); i += WARPS * 32) {
        const int hg = i / (D / 4), d = (i - hg * (D / 4)) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = sm_l[w][hg];
            const float4 v = *reinterpret_cast<const float4*>(&sm_o[w][hg][d]);
            acc.x = fmaf(v.x, f, acc.x);
            acc.y = fmaf(v.y, f, acc.y);
            acc.z = fmaf(v.z, f, acc.z);
            acc.w = fmaf(v.w, f, acc.w);
        }
        const int64_t pi = (static_cast<int64_t>(b) * P.H + kvh * G + hg) * P.splits + split;
        *reinterpret_cast<float4*>(P.part_o + pi * D + d) = acc;
    }
    // One release-acquire count per CTA instead of a fence by every thread: the barrier puts the CTA's stores
    // before thread 0's release, the last CTA's acquire (and its barrier) puts every split's stores before the
    // loads below.
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int prev;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(P.counters + b * P.KV_H + kvh) : "memory");
        s_last = (prev == static_cast<unsigned int>(P.splits) - 1u);
        if (s_last) P.counters[b * P.KV_H + kvh] = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    // split weights: one warp per head (lanes over the splits), then 16-byte loads of the partials
    float* wgt = reinterpret_cast<float*>(sm_buf);            // [G][splits], splits <= 64
    // the first eight partials of this thread's output are requested before the weights are worked out
    const bool mine = threadIdx.x < G * (D / 4);
    const int my_hg = threadIdx.x / (D / 4), my_d = (threadIdx.x - my_hg * (D / 4)) * 4;
    const float4* my_po =
        reinterpret_cast<const float4*>(P.part_o + (static_cast<int64_t>(b) * P.H + kvh * G + my_hg) * P.splits * D + my_d);
    float4 first[8];
    if (mine && P.splits >= 8) {
#pragma unroll
        for (int u = 0; u < 8; ++u) first[u] = __ldcg(my_po + static_cast<int64_t>(u) * (D / 4));
    }
    __syncthreads();
    for (int hg = warp; hg < G; hg += WARPS) {
        const float* lse = P.part_lse + (static_cast<int64_t>(b) * P.H + kvh * G + hg) * P.splits;
        const float l0 = lane < P.splits ? __ldcg(lse + lane) : NEG_BIG;
        const float l1 = lane + 32 < P.splits ? __ldcg(lse + lane + 32) : NEG_BIG;
        const float mx = warp_max(fmaxf(l0, l1));
        const float e0 = l0 > 0.5f * NEG_BIG ? exp2f(l0 - mx) : 0.f;
        const float e1 = l1 > 0.5f * NEG_BIG ? exp2f(l1 - mx) : 0.f;
        const float sum = warp_sum(e0 + e1);
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
        if (lane < P.splits) wgt[hg * P.splits + lane] = e0 * inv;
        if (lane + 32 < P.splits) wgt[hg * P.splits + lane + 32] = e1 * inv;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * (D / 4); i += WARPS * 32) {
        const int hg = i / (D / 4), d = (i - hg * (D / 4)) * 4;
        const int h = kvh * G + hg;
        const float4* po = reinterpret_cast<const float4*>(P.part_o + (static_cast<int64_t>(b) * P.H + h) * P.splits * D + d);
        const float* w = wgt + hg * P.splits;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int s2 = 0;
        for (; s2 + 8 <= P.splits; s2 += 8) {
            float4 v[8];
            if (s2 == 0 && i == threadIdx.x) {
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = first[u];
            } else {
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = __ldcg(po + static_cast<int64_t>(s2 + u) * (D / 4));
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                acc.x = fmaf(w[s2 + u], v[u].x, acc.x);
                acc.y = fmaf(w[s2 + u], v[u].y, acc.y);
                acc.z = fmaf(w[s2 + u], v[u].z, acc.z);
                acc.w = fmaf(w[s2 + u], v[u].w, acc.w);
            }
        }
        for (; s2 < P.splits; ++s2) {
            const float4 v = __ldcg(po + static_cast<int64_t>(s2) * (D / 4));
            acc.x = fmaf(w[s2], v.x, acc.x);
            acc.y = fmaf(w[s2], v.y, acc.y);
            acc.z = fmaf(w[s2], v.z, acc.z);
            acc.w = fmaf(w[s2], v.w, acc.w);
        }
        const int64_t o = (static_cast<int64_t>(b) * P.H + h) * D + d;
        out_elem(P.out, P.q_dtype, o, acc.x);
        out_elem(P.out, P.q_dtype, o + 1, acc.y);
        out_elem(P.out, P.q_dtype, o + 2, acc.z);
        out_elem(P.out, P.q_dtype, o + 3, acc.w);
    }
}

}  // namespace am

// Launch the tensor-core kernel; the caller has validated shapes and laid the workspace out.
int launch_attn_mma(int layout, const void* q, int64_t q_bs, int64_t q_hs, int q_dtype, const KVPtrs& kv,
                    const int32_t* pos, int pos_count, void* out, int B, int H, int KV_H, float scale_log2,
                    int splits, float* part_o, float* part_lse, unsigned int* counters, int* status,
                    cudaStream_t st, const AttnFuse* fuse) {
    am::Params P;
    P.fused = fuse ? 1 : 0;
    if (fuse) P.fuse = *fuse;
    else P.fuse = AttnFuse{nullptr, nullptr, nullptr, 0, 0};
    P.q = q; P.q_bs = q_bs; P.q_hs = q_hs; P.q_dtype = q_dtype;
    P.kv = kv; P.pos = pos; P.pos_count = pos_count; P.out = out;
    P.B = B; P.H = H; P.KV_H = KV_H; P.G = H / KV_H;
    P.scale_log2 = scale_log2; P.splits = splits;
    P.part_o = part_o; P.part_lse = part_lse; P.counters = counters; P.status = status;
    const dim3 grid(splits, KV_H, B);
    switch (layout) {
        case ALLOYB_KV_F16: launch_pdl(am::attn_mma_kernel<ALLOYB_KV_F16>, dim3(grid), dim3(am::WARPS * 32), 0, st, P); break;
        case ALLOYB_KV_Q8_SPLIT: launch_pdl(am::attn_mma_kernel<ALLOYB_KV_Q8_SPLIT>, dim3(grid), dim3(am::WARPS * 32), 0, st, P); break;
        default: launch_pdl(am::attn_mma_kernel<ALLOYB_KV_Q8_PAGED>, dim3(grid), dim3(am::WARPS * 32), 0, st, P); break;
    }
    return check_launch();
}

int attn_mma_device_error(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, am::g_attn_error, sizeof(int)) != cudaSuccess) return 0;
    if (clear && v) {
        const int z = 0;
        cudaMemcpyToSymbol(am::g_attn_error, &z, sizeof(int));
    }
    return v;
}

}  // namespace alloyb

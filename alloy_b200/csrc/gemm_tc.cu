// Prefill dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   C[M tokens, N] = X[M, K] (bf16 | fp16)  *  deq(W)[N, K]^T      fp32 accumulate, C in X's type
//
// One CTA computes a 256-token x 128-row output tile.  Per 64-wide K step:
//   * warp 0 (one lane) brings the 256 x 64 activation tile in with ONE TMA tensor copy
//     (128-byte swizzle) and, once per super-block, the 128 packed weight rows with bulk copies;
//   * warps 2-5 (128 threads, one weight row each) decode 64 weights of their row to fp32
//     exactly as the block format defines them (Q4_K: d*sc*nib - dmin*m with ONE rounding;
//     Q6_K: d*sc*(q-32), exact; Q8_0: scale*code, exact), round ONCE to the activation type and store them into the
//     K-major, 128-byte-swizzled layout the MMA reads;
//   * warp 1 (one lane) issues two tcgen05.mma (M = 128 tokens each, N = 128, K = 16 x 4) whose
//     accumulators live in tensor memory (256 columns), and releases the stage with
//     tcgen05.commit.
// Decoding a weight tile once per 256 tokens (not per 128) halves the CUDA-core work per flop;
// the decode of step k+1 overlaps the MMAs of step k through a 3-deep stage ring.
// After the last K step the four decode warps read the accumulators back with tcgen05.ld and
// store C.  Every wait is bounded: on a time-out the sticky device error word is set, the CTA
// still frees its tensor memory and returns.
#include <cuda.h>

#include "linear.cuh"

namespace alloyb {


namespace tc {

__device__ int g_tc_error = 0;          // sticky: a bounded wait of this file's kernel ran out

constexpr int BM = 256;                 // tokens per CTA (two UMMA M = 128 halves)
constexpr int BN = 128;                 // weight rows per CTA (UMMA N)
constexpr int BK = 64;                  // K step: 64 x 2 bytes = one 128-byte swizzle row
constexpr int STAGES = 3;
constexpr int A_STAGE = BM * BK * 2;    // 32 KB
constexpr int B_STAGE = BN * BK * 2;    // 16 KB
constexpr int PACK_ROW = 272;           // packed super-block per row: 144 (Q4_K) / <= 224-byte window (Q6_K) /
                                        // 256 codes + 8 fp16 scales (Q8_0); 17 x 16 bytes keeps 128-bit reads
                                        // of 8 rows conflict-free
constexpr int PACK_STAGE = BN * PACK_ROW;   // 28 KB
constexpr int PACK_STAGES = 2;
constexpr int DEC_THREADS = 256;        // two decode threads per weight row (half a k-step each)
constexpr int THREADS = 64 + DEC_THREADS;   // warp 0 copies, warp 1 MMA, warps 2-9 decode + epilogue
constexpr int TMEM_COLS = 256;
constexpr uint32_t SPIN = 1u << 22;

struct Bars {
    uint64_t a_full[STAGES];      // TMA -> MMA
    uint64_t b_full[STAGES];      // decode -> MMA (128 arrivals)
    uint64_t empty[STAGES];       // MMA -> TMA + decode (tcgen05.commit)
    uint64_t p_full[PACK_STAGES];     // bulk copies -> decode
    uint64_t p_empty[PACK_STAGES];    // decode -> copies (128 arrivals)
    uint64_t acc_full;            // MMA -> epilogue
    uint32_t tmem_base;
    uint32_t pad;
};

constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * (A_STAGE + B_STAGE) + PACK_STAGES * PACK_STAGE + 256;

struct Params {
    const uint8_t* w;         // packed rows (Q8_0: int8 codes, K per row)
    const __half* scales;     // Q8_0: fp16 (N, K/32)
    int64_t row_bytes;
    int format;               // ALLOYB_Q4_K / ALLOYB_Q6_K / ALLOYB_Q8_0
    void* y;
    int64_t ldy;
    int M, N, K;
    int is_bf16;
};

__device__ __forceinline__ uint32_t s32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void bar_init(uint64_t* b, uint32_t n) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n));
}
__device__ __forceinline__ void bar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(s32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_wait(uint64_t* b, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN; ++i) {
        if (bar_try(b, parity)) return true;
        if (i > 32) __nanosleep(64);
    }
    atomicExch(&g_tc_error, 2);
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     s32(dst)),
                 "l"(src), "r"(bytes), "r"(s32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            s32(dst)),
        "l"(map), "r"(s32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ uint32_t lds_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(s32(p)));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(s32(p)));
    return v;
}
__device__ __forceinline__ uint4 lds_u128(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(s32(p)));
    return v;
}
__device__ __forceinline__ void sts_u128(void* p, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(s32(p)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// K-major, 128-byte-swizzled operand: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);          // start address
    d |= static_cast<uint64_t>(1) << 16;                             // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                     // stride byte offset: 8 rows x 128 B
    d |= static_cast<uint64_t>(1) << 46;                             // descriptor version (Blackwell)
    d |= static_cast<uint64_t>(2) << 61;                             // SWIZZLE_128B
    return d;
}
// kind::f16: D fp32, A/B both bf16 (1) or fp16 (0), both K-major, M = 128, N = BN.
__device__ __forceinline__ uint32_t umma_idesc(int is_bf16) {
    uint32_t d = 0;
    d |= 1u << 4;                                   // D format F32
    d |= static_cast<uint32_t>(is_bf16 ? 1 : 0) << 7;    // A format
    d |= static_cast<uint32_t>(is_bf16 ? 1 : 0) << 10;   // B format
    d |= static_cast<uint32_t>(BN >> 3) << 17;      // N
    d |= static_cast<uint32_t>(128 >> 4) << 24;     // M
    return d;
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(addr));
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    uint32_t r;
    if (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
}

// Row `r` of a [rows x 64] 2-byte tile in the swizzled K-major layout: 8 chunks of 16 bytes.
__device__ __forceinline__ uint8_t* swz(uint8_t* tile, int r, int chunk) {
    return tile + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4);
}

// Decode k-step `ks` (0..3) of one Q4_K super-block of this thread's row: 64 weights.
template <bool BF16>
__device__ __forceinline__ void decode_q4k(const uint8_t* blk, int ks, uint8_t* tile, int r, int hsel) {
    const uint4 hdr = lds_u128(blk);
    const float d = half_bits_to_f32(hdr.x & 0xffffu), dmin = half_bits_to_f32(hdr.x >> 16);
    int sc0, m0, sc1, m1;
    q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * ks, sc0, m0);
    q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * ks + 1, sc1, m1);
    const float dl = d * static_cast<float>(sc0), ml = dmin * static_cast<float>(m0);
    const float dh = d * static_cast<float>(sc1), mh = dmin * static_cast<float>(m1);
    // this thread's half of the 32 quant bytes: bytes 16*hsel .. +15 -> chunks 2*hsel, 2*hsel+1
    const uint4 q0 = lds_u128(blk + 16 + ks * 32 + 16 * hsel);
    const uint32_t qw[4] = {q0.x, q0.y, q0.z, q0.w};
    // low nibbles -> k 0..31 (chunks 0-3), high nibbles -> k 32..63 (chunks 4-7)
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * hsel + cc;
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = qw[cc * 2 + h];
            float fl[4], fh[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t byte = (w >> (8 * e)) & 0xffu;
                // exact products, one rounding at the subtract (FMA), then one rounding to 16 bits
                fl[e] = fmaf(dl, static_cast<float>(byte & 15u), -ml);
                fh[e] = fmaf(dh, static_cast<float>(byte >> 4), -mh);
            }
            lo[h * 2] = pack2<BF16>(fl[0], fl[1]);
            lo[h * 2 + 1] = pack2<BF16>(fl[2], fl[3]);
            hi[h * 2] = pack2<BF16>(fh[0], fh[1]);
            hi[h * 2 + 1] = pack2<BF16>(fh[2], fh[3]);
        }
        sts_u128(swz(tile, r, c), make_uint4(lo[0], lo[1], lo[2], lo[3]));
        sts_u128(swz(tile, r, c + 4), make_uint4(hi[0], hi[1], hi[2], hi[3]));
    }
}

// Q6_K: the block sits at `blk` (2-byte aligned).  k-step ks: elements 64*ks .. +63.
template <bool BF16>
__device__ __forceinline__ void decode_q6k(const uint8_t* blk, int ks, uint8_t* tile, int r, int hsel) {
    const int h = ks >> 1, jb = (ks & 1) * 2;            // sub-blocks j = jb, jb+1 of half h
    const float d = half_bits_to_f32(lds_u16(blk + 208));
    {
        const int jj = hsel;                             // this thread's sub-block pair of the k-step
        const int j = jb + jj;
        const uint8_t* ql = blk + h * 64 + (j & 1) * 32;
        const uint8_t* qh = blk + 128 + h * 32;
        const uint32_t sc2 = lds_u16(blk + 192 + h * 8 + 2 * j);
        const float s0 = d * static_cast<float>(static_cast<int8_t>(sc2 & 0xffu));
        const float s1 = d * static_cast<float>(static_cast<int8_t>(sc2 >> 8));
#pragma unroll
        for (int c = 0; c < 4; ++c) {                    // 8 elements per 16-byte chunk
            uint32_t out[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {                // 2 elements per 16-bit load
                const int l = c * 8 + p * 2;
                const uint32_t a = lds_u16(ql + l), b = lds_u16(qh + l);
                float f[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t byte = (a >> (8 * e)) & 0xffu;
                    const uint32_t nib = (j >= 2) ? (byte >> 4) : (byte & 15u);
                    const uint32_t hi = (b >> (8 * e + 2 * j)) & 3u;
                    const float q = static_cast<float>(static_cast<int>(nib | (hi << 4)) - 32);
                    f[e] = (l + e < 16 ? s0 : s1) * q;   // exact in fp32
                }
                out[p] = pack2<BF16>(f[0], f[1]);
            }
            sts_u128(swz(tile, r, jj * 4 + c), make_uint4(out[0], out[1], out[2], out[3]));
        }
    }
}

// Q8_0: the stage row holds 256 codes then the super-block's eight fp16 scales.  k-step ks: elements
// 64*ks .. +63 = two 32-element blocks, one per thread of the pair; w = scale * code (exact in fp32).
template <bool BF16>
__device__ __forceinline__ void decode_q8_0(const uint8_t* blk, int ks, uint8_t* tile, int r, int hsel) {
    const float sc = half_bits_to_f32(lds_u16(blk + 256 + (2 * ks + hsel) * 2));
    const uint8_t* q = blk + ks * 64 + hsel * 32;
#pragma unroll
    for (int c = 0; c < 2; ++c) {                        // 16 codes -> two 16-byte chunks
        const uint4 v = lds_u128(q + 16 * c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float f0 = sc * static_cast<float>(static_cast<int8_t>(w[j] & 0xffu));
            const float f1 = sc * static_cast<float>(static_cast<int8_t>((w[j] >> 8) & 0xffu));
            const float f2 = sc * static_cast<float>(static_cast<int8_t>((w[j] >> 16) & 0xffu));
            const float f3 = sc * static_cast<float>(static_cast<int8_t>(w[j] >> 24));
            o[2 * j] = pack2<BF16>(f0, f1);
            o[2 * j + 1] = pack2<BF16>(f2, f3);
        }
        sts_u128(swz(tile, r, 4 * hsel + 2 * c), make_uint4(o[0], o[1], o[2], o[3]));
        sts_u128(swz(tile, r, 4 * hsel + 2 * c + 1), make_uint4(o[4], o[5], o[6], o[7]));
    }
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_st = smem;                                   // STAGES x 32 KB
    uint8_t* b_st = smem + STAGES * A_STAGE;                // STAGES x 16 KB
    uint8_t* p_st = b_st + STAGES * B_STAGE;                // 2 x 28 KB packed rows
    Bars* bars = reinterpret_cast<Bars*>(p_st + PACK_STAGES * PACK_STAGE);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int nsb = P.K / QK_K, ksteps = nsb * 4;
    const int blk_bytes = P.format == ALLOYB_Q4_K ? Q4K_BYTES : (P.format == ALLOYB_Q6_K ? Q6K_BYTES : 256);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            bar_init(&bars->a_full[s], 1);
            bar_init(&bars->b_full[s], DEC_THREADS);
            bar_init(&bars->empty[s], 1);
        }
        for (int s = 0; s < PACK_STAGES; ++s) {
            bar_init(&bars->p_full[s], 1);
            bar_init(&bars->p_empty[s], DEC_THREADS);
        }
        bar_init(&bars->acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {      // tensor memory: one warp allocates, the same warp frees
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&bars->tmem_base)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------ copies: packed rows (per super-block) + A tiles
        bool ok = true;
        for (int ks = 0; ks < ksteps && ok; ++ks) {
            if ((ks & 3) == 0) {
                const int sb = ks >> 2, ps = sb % PACK_STAGES;
                if (sb >= PACK_STAGES) ok = bar_wait(&bars->p_empty[ps], ((sb / PACK_STAGES) - 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                // Q4_K blocks are 16-byte aligned; a Q6_K block (210 bytes, 2-byte aligned) is copied
                // as the aligned 224-byte window around it
                const int start = sb * blk_bytes;
                const int ws = start & ~15;
                const uint32_t bytes = P.format == ALLOYB_Q6_K ? static_cast<uint32_t>(((start & 15) + Q6K_BYTES + 15) & ~15)
                                                               : static_cast<uint32_t>(blk_bytes);
                const bool q8 = P.format == ALLOYB_Q8_0;
                if (lane == 0) bar_expect(&bars->p_full[ps], (bytes + (q8 ? 16u : 0u)) * BN);
                __syncwarp();
                for (int r = lane; r < BN; r += 32) {
                    int row = n0 + r;
                    if (row >= P.N) row = P.N - 1;
                    bulk_g2s(p_st + ps * PACK_STAGE + r * PACK_ROW, P.w + static_cast<int64_t>(row) * P.row_bytes + ws,
                             bytes, &bars->p_full[ps]);
                    if (q8)      // the super-block's eight block scales behind its codes
                        bulk_g2s(p_st + ps * PACK_STAGE + r * PACK_ROW + 256,
                                 P.scales + static_cast<int64_t>(row) * (P.K / Q8_BLOCK) + sb * 8, 16, &bars->p_full[ps]);
                }
            }
            const int s = ks % STAGES;
            if (ks >= STAGES) ok = bar_wait(&bars->empty[s], ((ks / STAGES) - 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane == 0) {
                bar_expect(&bars->a_full[s], A_STAGE);
                tma_2d(a_st + s * A_STAGE, &xmap, ks * BK, m0, &bars->a_full[s]);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issue (one lane)
        const uint32_t idesc = umma_idesc(BF16 ? 1 : 0);
        bool ok = true;
        for (int ks = 0; ks < ksteps && ok; ++ks) {
            const int s = ks % STAGES;
            ok = bar_wait(&bars->a_full[s], (ks / STAGES) & 1) && bar_wait(&bars->b_full[s], (ks / STAGES) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t a0 = s32(a_st + s * A_STAGE), b0 = s32(b_st + s * B_STAGE);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) {
                    const uint64_t db = umma_desc(b0 + kk * 32);
                    const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
                    umma(tmem, umma_desc(a0 + kk * 32), db, idesc, acc);                    // tokens 0..127
                    umma(tmem + BN, umma_desc(a0 + 128 * 128 + kk * 32), db, idesc, acc);   // tokens 128..255
                }
                umma_commit(&bars->empty[s]);
                if (ks == ksteps - 1) umma_commit(&bars->acc_full);
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------ decode (two threads per weight row)
        const int r = (threadIdx.x - 64) & (BN - 1), hsel = (threadIdx.x - 64) >> 7;
        const bool live = n0 + r < P.N;
        bool ok = true;
        for (int ks = 0; ks < ksteps; ++ks) {
            const int sb = ks >> 2, ps = sb % PACK_STAGES, s = ks % STAGES;
            if (ok && (ks & 3) == 0) ok = bar_wait(&bars->p_full[ps], (sb / PACK_STAGES) & 1);
            if (ok && ks >= STAGES) ok = bar_wait(&bars->empty[s], ((ks / STAGES) - 1) & 1);
            if (ok) {
                uint8_t* tile = b_st + s * B_STAGE;
                const uint8_t* blk = p_st + ps * PACK_STAGE + r * PACK_ROW +
                                     (P.format == ALLOYB_Q6_K ? ((sb * Q6K_BYTES) & 15) : 0);
                if (!live) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) sts_u128(swz(tile, r, 4 * hsel + c), make_uint4(0u, 0u, 0u, 0u));
                } else if (P.format == ALLOYB_Q4_K) {
                    decode_q4k<BF16>(blk, ks & 3, tile, r, hsel);
                } else if (P.format == ALLOYB_Q6_K) {
                    decode_q6k<BF16>(blk, ks & 3, tile, r, hsel);
                } else {
                    decode_q8_0<BF16>(blk, ks & 3, tile, r, hsel);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic stores -> MMA reads
            }
            bar_arrive(&bars->b_full[s]);
            if ((ks & 3) == 3) bar_arrive(&bars->p_empty[ps]);
        }
        // ------------------------------------------------ epilogue: TMEM -> registers -> C
        if (ok) ok = bar_wait(&bars->acc_full, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int quarter = warp & 3;                   // TMEM lanes this warp may read
            const int half = (warp - 2) >> 2;               // warps 2-5: tokens 0..127, warps 6-9: 128..255
            {
                const int tok = m0 + half * 128 + quarter * 32 + lane;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + half * BN + c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (tok < P.M) {
                        uint32_t o[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            o[e] = pack2<BF16>(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
                        uint16_t* dst = static_cast<uint16_t*>(P.y) + static_cast<int64_t>(tok) * P.ldy + n0 + c0;
                        if (n0 + c0 + 16 <= P.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
                            reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
                            reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
                        } else {
                            for (int e = 0; e < 16; ++e)
                                if (n0 + c0 + e < P.N) dst[e] = static_cast<uint16_t>(o[e >> 1] >> (16 * (e & 1)));
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
}

}  // namespace tc

// Sticky error word of the GEMM kernel (merged into alloyb_device_error).
int gemm_tc_device_error(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_tc_error, sizeof(int)) != cudaSuccess) return 0;
    if (clear && v) {
        const int z = 0;
        cudaMemcpyToSymbol(tc::g_tc_error, &z, sizeof(int));
    }
    return v;
}

// C = X * deq(W)^T for one packed matrix.  NOT_TAKEN unless the shape is the prefill kind.
int try_gemm_tc(const void* x, int M, int K, int dtype, const WeightSeg& seg, cudaStream_t st) {
    using namespace tc;
    if (dtype != ALLOYB_F16 && dtype != ALLOYB_BF16) return ALLOYB_NOT_TAKEN;
    if (seg.format != ALLOYB_Q4_K && seg.format != ALLOYB_Q6_K && seg.format != ALLOYB_Q8_0) return ALLOYB_NOT_TAKEN;
    if (M < 64 || K % QK_K) return ALLOYB_NOT_TAKEN;
    if (seg.format == ALLOYB_Q8_0 && (!seg.scales || reinterpret_cast<uintptr_t>(seg.scales) % 16 || seg.row_bytes != K))
        return ALLOYB_NOT_TAKEN;
    if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(seg.data) % 16 || seg.row_bytes % 16)
        return ALLOYB_NOT_TAKEN;
    if (seg.format == ALLOYB_Q6_K) {
        // the aligned window of a row's last block must end inside the row pitch
        const int64_t last = static_cast<int64_t>(K / QK_K - 1) * Q6K_BYTES;
        if ((last & ~15LL) + (((last & 15) + Q6K_BYTES + 15) & ~15LL) > seg.row_bytes) return ALLOYB_NOT_TAKEN;
    }

    CUtensorMap map;
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
    const cuuint64_t gstr[1] = {static_cast<cuuint64_t>(K) * 2};
    const cuuint32_t box[2] = {BK, BM};
    const cuuint32_t estr[2] = {1, 1};
    // The driver's tensor-map encoder is looked up through the runtime, so the library carries no
    // link-time dependency on the driver and still loads (for symbol checks) on a machine without one.
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr);
        if (e != cudaSuccess || qr != cudaDriverEntryPointSuccess || !fn) {
            set_cuda_error(e != cudaSuccess ? e : cudaErrorNotSupported);
            return ALLOYB_E_CUDA;
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const CUresult cr = encode(
        &map, dtype == ALLOYB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
        const_cast<void*>(x), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        set_cuda_error(cudaErrorInvalidValue);
        return ALLOYB_E_CUDA;
    }
    Params P;
    P.w = static_cast<const uint8_t*>(seg.data);
    P.scales = static_cast<const __half*>(seg.scales);
    P.row_bytes = seg.row_bytes;
    P.format = seg.format;
    P.y = seg.y;
    P.ldy = seg.ldy;
    P.M = M;
    P.N = seg.N;
    P.K = K;
    P.is_bf16 = dtype == ALLOYB_BF16;

    static bool configured[64] = {};          // per device ordinal
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
        configured[dev] = true;
    }
    const dim3 grid((seg.N + BN - 1) / BN, (M + BM - 1) / BM);
    if (dtype == ALLOYB_BF16) gemm_tc_kernel<true><<<grid, THREADS, SMEM_BYTES, st>>>(map, P);
    else gemm_tc_kernel<false><<<grid, THREADS, SMEM_BYTES, st>>>(map, P);
    return check_launch();
}

}  // namespace alloyb

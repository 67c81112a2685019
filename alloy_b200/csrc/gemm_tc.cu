// Prefill dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   C[M tokens, N] = X[M, K] (bf16 | fp16)  *  deq(W)[N, K]^T      fp32 accumulate, C in X's type
//
// One CTA computes a 256-token x 128-row output tile.  Per 64-wide K step:
//   * warp 0 (one lane) brings the 256 x 64 activation tile in with ONE TMA tensor copy
//     (128-byte swizzle);
//   * warp 10 (one lane) brings the 128 packed weight rows of a super-block in with ONE tensor copy over
//     a byte view of the weight matrix (Q8_0: two swizzled copies of codes and one of scales), issued as
//     soon as the slot's previous super-block is decoded, i.e. a whole super-block ahead of its use;
//   * warps 2-9 (256 threads, two per weight row) decode 64 weights of their row to fp32
//     exactly as the block format defines them (Q4_K: d*sc*nib - dmin*m with ONE rounding;
//     Q6_K: d*sc*(q-32), exact; Q8_0: scale*code, exact), round ONCE to the activation type and store them into the
//     K-major, 128-byte-swizzled layout the MMA reads.  Codes become floats without a conversion
//     instruction (a byte permute drops the code into the mantissa of 2^23) and the arithmetic runs on
//     the two-wide fp32 instructions (add/mul/fma .f32x2);
//   * warp 1 (one lane) issues four tcgen05.mma per step with the WEIGHT rows as the M = 128 operand
//     and the 256 tokens as N (K = 16 each): one instruction reads each operand tile once, which
//     matters because shared-memory bandwidth, shared with the copies and the decode stores, is
//     what bounds the step.  The accumulator (128 lanes = weight rows, 256 columns = tokens) lives
//     in tensor memory; tcgen05.commit releases the stage.  The wait for the next stage is issued
//     while the last queued MMAs still run.
// Decoding a weight tile once per 256 tokens (not per 128) halves the CUDA-core work per flop;
// the decode of step k+1 overlaps the MMAs of step k through a 3-deep stage ring.
// After the last K step the eight decode warps read the accumulators back with tcgen05.ld and
// store C (each lane one weight row: a warp writes 64 contiguous bytes per token).  Every wait is bounded: on a time-out the sticky device error word is set, the CTA
// still frees its tensor memory and returns.
#include <cuda.h>

#include "linear.cuh"

namespace alloyb {


namespace tc {

__device__ int g_tc_error = 0;          // sticky: a bounded wait of this file's kernel ran out

constexpr int BM = 256;                 // tokens per CTA (UMMA N)
constexpr int BN = 128;                 // weight rows per CTA (UMMA M)
constexpr int BK = 64;                  // K step: 64 x 2 bytes = one 128-byte swizzle row
constexpr int STAGES = 3;
constexpr int A_STAGE = BM * BK * 2;    // 32 KB
constexpr int B_STAGE = BN * BK * 2;    // 16 KB
// One super-block of 128 packed rows in shared memory:
//   Q4_K  144-byte rows (9 x 16 bytes: 128-bit reads of 8 consecutive rows hit distinct banks);
//   Q6_K  240-byte rows: the 16-byte-aligned window around the 210-byte block (15 x 16 bytes);
//   Q8_0  two [128 rows x 128 codes] tiles in the 128-byte swizzle, then 16 bytes of scales per row.
constexpr int Q4_ROW = 144, Q6_ROW = 240;
constexpr int Q8_HALF = BN * 128;           // 16 KB
constexpr int PACK_STAGE = 2 * Q8_HALF + BN * 16;   // 34 KB, the largest of the three
constexpr int PACK_STAGES = 2;
constexpr int DEC_THREADS = 256;        // two decode threads per weight row (half a k-step each)
constexpr int THREADS = 64 + DEC_THREADS + 32;   // warp 0 A copies, warp 1 MMA, warps 2-9 decode + epilogue,
                                                 // warp 10 packed-row copies
constexpr int TMEM_COLS = 256;
constexpr uint32_t SPIN = 1u << 22;

struct Bars {
    uint64_t full[STAGES];        // token-tile copy (1 arrival + bytes) and decode (256 arrivals) -> MMA
    uint64_t empty[STAGES];       // MMA -> TMA + decode (tcgen05.commit)
    uint64_t p_full[PACK_STAGES];     // packed-row copies -> decode
    uint64_t p_empty[PACK_STAGES];    // decode -> copies (256 arrivals)
    uint64_t acc_full;            // MMA -> epilogue
    uint32_t tmem_base;
    uint32_t pad;
};

constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * (A_STAGE + B_STAGE) + PACK_STAGES * PACK_STAGE + 256;

struct Params {
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
// kind::f16: D fp32, A/B both bf16 (1) or fp16 (0), both K-major, M = BN weight rows, N = BM tokens.
__device__ __forceinline__ uint32_t umma_idesc(int is_bf16) {
    uint32_t d = 0;
    d |= 1u << 4;                                   // D format F32
    d |= static_cast<uint32_t>(is_bf16 ? 1 : 0) << 7;    // A format
    d |= static_cast<uint32_t>(is_bf16 ? 1 : 0) << 10;   // B format
    d |= static_cast<uint32_t>(BM >> 3) << 17;      // N
    d |= static_cast<uint32_t>(BN >> 4) << 24;      // M
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

// Two fp32 values in one 64-bit register and the two-wide fp32 instructions on them.
__device__ __forceinline__ uint64_t f2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(uint64_t v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return pack2<BF16>(lo, hi);
}
// Bytes e and e+1 of `codes` as the floats 2^23 + code: the byte lands in the low mantissa bits of
// 0x4B000000 (2^23), where one unit in the last place is exactly 1.
template <int E>
__device__ __forceinline__ uint64_t magic2(uint32_t codes) {
    return f2(__uint_as_float(__byte_perm(codes, 0x4B000000u, 0x7540 | E)),
              __uint_as_float(__byte_perm(codes, 0x4B000000u, 0x7540 | (E + 1))));
}

// Row `r` of a [rows x 64] 2-byte tile in the swizzled K-major layout: 8 chunks of 16 bytes.
__device__ __forceinline__ uint8_t* swz(uint8_t* tile, int r, int chunk) {
    return tile + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4);
}

// Decode k-step `ks` (0..3) of one Q4_K super-block of this thread's row: 64 weights, of which this
// thread (hsel) owns quant bytes 16*hsel .. +15: their low nibbles are k 16*hsel .. +15 (chunks
// 2*hsel, 2*hsel+1), their high nibbles k 32 + the same (chunks 4 + ...).
template <bool BF16>
__device__ __forceinline__ void decode_q4k(const uint8_t* blk, int ks, uint8_t* tile, int r, int hsel) {
    const uint4 hdr = lds_u128(blk);
    const float d = half_bits_to_f32(hdr.x & 0xffffu), dmin = half_bits_to_f32(hdr.x >> 16);
    int sc0, m0, sc1, m1;
    q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * ks, sc0, m0);
    q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * ks + 1, sc1, m1);
    const float dl = d * static_cast<float>(sc0), ml = dmin * static_cast<float>(m0);
    const float dh = d * static_cast<float>(sc1), mh = dmin * static_cast<float>(m1);
    const uint64_t dl2 = f2(dl, dl), ml2 = f2(-ml, -ml), dh2 = f2(dh, dh), mh2 = f2(-mh, -mh);
    const uint64_t unbias = f2(-8388608.0f, -8388608.0f);
    const uint4 q0 = lds_u128(blk + 16 + ks * 32 + 16 * hsel);
    const uint32_t qw[4] = {q0.x, q0.y, q0.z, q0.w};
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = qw[cc * 2 + h];
            const uint32_t l4 = w & 0x0f0f0f0fu, h4 = (w >> 4) & 0x0f0f0f0fu;
            // (2^23 + nib) - 2^23 is exact; then exact product and ONE rounding at the subtract (FMA)
            lo[h * 2] = pack2<BF16>(f2_fma(f2_add(magic2<0>(l4), unbias), dl2, ml2));
            lo[h * 2 + 1] = pack2<BF16>(f2_fma(f2_add(magic2<2>(l4), unbias), dl2, ml2));
            hi[h * 2] = pack2<BF16>(f2_fma(f2_add(magic2<0>(h4), unbias), dh2, mh2));
            hi[h * 2 + 1] = pack2<BF16>(f2_fma(f2_add(magic2<2>(h4), unbias), dh2, mh2));
        }
        const int c = 2 * hsel + cc;
        sts_u128(swz(tile, r, c), make_uint4(lo[0], lo[1], lo[2], lo[3]));
        sts_u128(swz(tile, r, c + 4), make_uint4(hi[0], hi[1], hi[2], hi[3]));
    }
}

// Q6_K: the block sits at `blk` (2-byte aligned inside its 16-byte-aligned window).  k-step ks covers
// elements 64*ks .. +63 = sub-rows j = jb, jb+1 of half h; this thread owns sub-row jb + hsel: 32
// elements whose low nibbles are 32 bytes of ql and whose top two bits are 32 bytes of qh.  Both runs
// are read as nine 4-byte-aligned words and shifted into place.
template <bool BF16>
__device__ __forceinline__ void decode_q6k(const uint8_t* blk, int ks, uint8_t* tile, int r, int hsel) {
    const int h = ks >> 1, j = (ks & 1) * 2 + hsel;
    const float d = half_bits_to_f32(lds_u16(blk + 208));
    const uint32_t sc2 = lds_u16(blk + 192 + h * 8 + 2 * j);
    const float s0 = d * static_cast<float>(static_cast<int8_t>(sc2 & 0xffu));
    const float s1 = d * static_cast<float>(static_cast<int8_t>(sc2 >> 8));
    const uint64_t s02 = f2(s0, s0), s12 = f2(s1, s1);
    const uint64_t unbias = f2(-8388640.0f, -8388640.0f);          // -(2^23 + 32)
    const uint32_t a_ql = s32(blk + h * 64 + (j & 1) * 32), a_qh = s32(blk + 128 + h * 32);
    const uint32_t sh = (a_ql & 3u) * 8u;                          // 0 or 16: same for both runs
    uint32_t wl[9], wh[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) {
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wl[i]) : "r"((a_ql & ~3u) + 4 * i));
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wh[i]) : "r"((a_qh & ~3u) + 4 * i));
    }
    const uint32_t shq = j >= 2 ? 4u : 0u, shh = 2u * j;
#pragma unroll
    for (int c = 0; c < 4; ++c) {                    // 8 elements per 16-byte chunk
        uint32_t out[4];
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const int i = 2 * c + p;
            const uint32_t ql = __funnelshift_r(wl[i], wl[i + 1], sh), qh = __funnelshift_r(wh[i], wh[i + 1], sh);
            // four 6-bit codes, one per byte: nibble | (two high bits << 4)
            const uint32_t q = ((ql >> shq) & 0x0f0f0f0fu) + ((qh >> shh) & 0x03030303u) * 16u;
            const uint64_t s = i < 4 ? s02 : s12;    // elements 0-15 / 16-31 of the sub-row
            out[p * 2] = pack2<BF16>(f2_mul(f2_add(magic2<0>(q), unbias), s));       // exact in fp32
            out[p * 2 + 1] = pack2<BF16>(f2_mul(f2_add(magic2<2>(q), unbias), s));
        }
        sts_u128(swz(tile, r, hsel * 4 + c), make_uint4(out[0], out[1], out[2], out[3]));
    }
}

// Q8_0: `st` is the stage: two [128 rows x 128 codes] tiles in the 128-byte swizzle, then eight fp16 scales
// per row.  k-step ks: elements 64*ks .. +63 = two 32-element blocks, one per thread of the pair;
// w = scale * code (exact in fp32).
template <bool BF16>
__device__ __forceinline__ void decode_q8_0(const uint8_t* st, int ks, uint8_t* tile, int r, int hsel) {
    const float sc = half_bits_to_f32(lds_u16(st + 2 * Q8_HALF + r * 16 + (2 * ks + hsel) * 2));
    const uint64_t sc2 = f2(sc, sc), unbias = f2(-8388736.0f, -8388736.0f);     // -(2^23 + 128)
    const uint8_t* row = st + (ks >> 1) * Q8_HALF + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
    for (int c = 0; c < 2; ++c) {                        // 16 codes -> two 16-byte chunks
        const int chunk = (ks & 1) * 4 + hsel * 2 + c;
        const uint4 v = lds_u128(row + ((chunk ^ (r & 7)) << 4));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const uint32_t u = w[jj] ^ 0x80808080u;      // code + 128 as an unsigned byte
            o[2 * jj] = pack2<BF16>(f2_mul(f2_add(magic2<0>(u), unbias), sc2));
            o[2 * jj + 1] = pack2<BF16>(f2_mul(f2_add(magic2<2>(u), unbias), sc2));
        }
        sts_u128(swz(tile, r, 4 * hsel + 2 * c), make_uint4(o[0], o[1], o[2], o[3]));
        sts_u128(swz(tile, r, 4 * hsel + 2 * c + 1), make_uint4(o[4], o[5], o[6], o[7]));
    }
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
               const __grid_constant__ CUtensorMap smap, const Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_st = smem;                                   // STAGES x 32 KB
    uint8_t* b_st = smem + STAGES * A_STAGE;                // STAGES x 16 KB
    uint8_t* p_st = b_st + STAGES * B_STAGE;                // 2 x 34 KB packed rows
    Bars* bars = reinterpret_cast<Bars*>(p_st + PACK_STAGES * PACK_STAGE);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int nsb = P.K / QK_K, ksteps = nsb * 4;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            bar_init(&bars->full[s], 1 + DEC_THREADS);
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
        // ------------------------------------------------ A tiles
        bool ok = true;
        for (int ks = 0; ks < ksteps && ok; ++ks) {
            const int s = ks % STAGES;
            if (ks >= STAGES) ok = bar_wait(&bars->empty[s], ((ks / STAGES) - 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane == 0) {
                bar_expect(&bars->full[s], A_STAGE);
                tma_2d(a_st + s * A_STAGE, &xmap, ks * BK, m0, &bars->full[s]);
            }
            __syncwarp();
        }
    } else if (warp == 10) {
        // ------------------------------------------------ packed rows: one tensor copy per super-block
        bool ok = true;
        for (int sb = 0; sb < nsb && ok; ++sb) {
            const int ps = sb % PACK_STAGES;
            if (sb >= PACK_STAGES) ok = bar_wait(&bars->p_empty[ps], ((sb / PACK_STAGES) - 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane == 0) {
                uint8_t* dst = p_st + ps * PACK_STAGE;
                if (P.format == ALLOYB_Q4_K) {
                    bar_expect(&bars->p_full[ps], BN * Q4_ROW);
                    tma_2d(dst, &wmap, sb * Q4K_BYTES, n0, &bars->p_full[ps]);
                } else if (P.format == ALLOYB_Q6_K) {
                    // a block is 2-byte aligned: copy the aligned window around it (reads past the row's
                    // end are filled with zeros)
                    bar_expect(&bars->p_full[ps], BN * Q6_ROW);
                    tma_2d(dst, &wmap, (sb * Q6K_BYTES) & ~15, n0, &bars->p_full[ps]);
                } else {
                    bar_expect(&bars->p_full[ps], 2 * Q8_HALF + BN * 16);
                    tma_2d(dst, &wmap, sb * 256, n0, &bars->p_full[ps]);
                    tma_2d(dst + Q8_HALF, &wmap, sb * 256 + 128, n0, &bars->p_full[ps]);
                    tma_2d(dst + 2 * Q8_HALF, &smap, sb * 16, n0, &bars->p_full[ps]);
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issue (one lane)
        const uint32_t idesc = umma_idesc(BF16 ? 1 : 0);
        bool ok = bar_wait(&bars->full[0], 0);
        ok = __all_sync(0xffffffffu, ok);
        for (int ks = 0; ks < ksteps && ok; ++ks) {
            const int s = ks % STAGES;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t x0 = s32(a_st + s * A_STAGE), w0 = s32(b_st + s * B_STAGE);
            if (lane == 0) {
#pragma unroll
                for (int kk = 0; kk < BK / 16 - 1; ++kk)
                    umma(tmem, umma_desc(w0 + kk * 32), umma_desc(x0 + kk * 32), idesc, (ks > 0 || kk > 0) ? 1u : 0u);
            }
            // the next stage's wait overlaps the MMAs queued above
            if (ks + 1 < ksteps) ok = bar_wait(&bars->full[(ks + 1) % STAGES], ((ks + 1) / STAGES) & 1);
            if (lane == 0) {
                umma(tmem, umma_desc(w0 + 96), umma_desc(x0 + 96), idesc, 1u);
                umma_commit(&bars->empty[s]);
                if (ks == ksteps - 1) umma_commit(&bars->acc_full);
            }
            ok = __all_sync(0xffffffffu, ok);
        }
    } else if (warp < 10) {
        // ------------------------------------------------ decode (two threads per weight row)
        const int r = (threadIdx.x - 64) & (BN - 1), hsel = (threadIdx.x - 64) >> 7;
        bool ok = true;
        for (int ks = 0; ks < ksteps; ++ks) {
            const int sb = ks >> 2, ps = sb % PACK_STAGES, s = ks % STAGES;
            if (ok && (ks & 3) == 0) ok = bar_wait(&bars->p_full[ps], (sb / PACK_STAGES) & 1);
            if (ok && ks >= STAGES) ok = bar_wait(&bars->empty[s], ((ks / STAGES) - 1) & 1);
            if (ok) {
                uint8_t* tile = b_st + s * B_STAGE;
                const uint8_t* stg = p_st + ps * PACK_STAGE;
                // rows past N arrive as zeros from the tensor copy and decode to zeros
                if (P.format == ALLOYB_Q4_K) {
                    decode_q4k<BF16>(stg + r * Q4_ROW, ks & 3, tile, r, hsel);
                } else if (P.format == ALLOYB_Q6_K) {
                    decode_q6k<BF16>(stg + r * Q6_ROW + ((sb * Q6K_BYTES) & 15), ks & 3, tile, r, hsel);
                } else {
                    decode_q8_0<BF16>(stg, ks & 3, tile, r, hsel);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic stores -> MMA reads
            }
            bar_arrive(&bars->full[s]);
            if ((ks & 3) == 3) bar_arrive(&bars->p_empty[ps]);
        }
        // ------------------------------------------------ epilogue: TMEM -> registers -> C
        if (ok) ok = bar_wait(&bars->acc_full, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int quarter = warp & 3;                   // TMEM lanes this warp may read
            const int half = (warp - 2) >> 2;               // warps 2-5: tokens 0..127, warps 6-9: 128..255
            const int n = n0 + quarter * 32 + lane;         // this lane's weight row = output column
            uint16_t* col = static_cast<uint16_t*>(P.y) + n;
#pragma unroll 1
            for (int c0 = 0; c0 < BM / 2; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + half * (BM / 2) + c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int tok = m0 + half * (BM / 2) + c0;
                if (n < P.N) {
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        if (tok + e < P.M)
                            col[static_cast<int64_t>(tok + e) * P.ldy] =
                                static_cast<uint16_t>(pack2<BF16>(__uint_as_float(v[e]), 0.0f) & 0xffffu);
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
    // 2-D map over a row-major matrix: `inner` elements per row, `rows` rows `pitch` bytes apart.
    auto map2d = [&](CUtensorMap* m, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t rows,
                     uint64_t pitch, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
        const cuuint64_t gdim[2] = {inner, rows};
        const cuuint64_t gstr[1] = {pitch};
        const cuuint32_t box[2] = {box_inner, box_rows};
        const cuuint32_t estr[2] = {1, 1};
        return encode(m, type, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    CUtensorMap map, wmap, smap;
    bool ok = map2d(&map, dtype == ALLOYB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x,
                    K, M, static_cast<uint64_t>(K) * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    // the packed rows as bytes: one box = one super-block of 128 rows
    if (seg.format == ALLOYB_Q8_0) {
        ok = ok && map2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, seg.data, K, seg.N, seg.row_bytes, 128, BN,
                         CU_TENSOR_MAP_SWIZZLE_128B);
        ok = ok && map2d(&smap, CU_TENSOR_MAP_DATA_TYPE_UINT8, seg.scales, static_cast<uint64_t>(K / Q8_BLOCK) * 2, seg.N,
                         static_cast<uint64_t>(K / Q8_BLOCK) * 2, 16, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else {
        ok = ok && map2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, seg.data, seg.row_bytes, seg.N, seg.row_bytes,
                         seg.format == ALLOYB_Q4_K ? Q4_ROW : Q6_ROW, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
        smap = wmap;
    }
    if (!ok) {
        set_cuda_error(cudaErrorInvalidValue);
        return ALLOYB_E_CUDA;
    }
    Params P;
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
    if (dtype == ALLOYB_BF16) gemm_tc_kernel<true><<<grid, THREADS, SMEM_BYTES, st>>>(map, wmap, smap, P);
    else gemm_tc_kernel<false><<<grid, THREADS, SMEM_BYTES, st>>>(map, wmap, smap, P);
    return check_launch();
}

}  // namespace alloyb

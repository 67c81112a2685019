// Prefill dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   C[M tokens, N] = X[M, K] (bf16 | fp16)  *  deq(W)[N, K]^T      fp32 accumulate, C in X's type
//
// A persistent kernel: one CTA per SM walks output tiles of 128 weight rows x 256 tokens.  In the MMA
// the WEIGHT rows are the M = 128 operand and the 256 tokens are N, and the decoded weights never touch
// shared memory: the decode warps write them straight into TENSOR MEMORY (tcgen05.st), from where
// tcgen05.mma reads its A operand, so the only shared-memory traffic of the tensor pipe is the token
// tile -- shared-memory bandwidth is what bounds this kernel otherwise.  Per 64-wide K step:
//   * warp 0 (one lane) brings the 256 x 64 token tile in with ONE TMA tensor copy (128-byte swizzle);
//   * warp 10 (one lane) brings the 128 packed weight rows of a super-block (four K steps) in with ONE
//     tensor copy over a byte view of the weight matrix (Q8_0: two swizzled copies of codes and one of
//     scales), issued as soon as the slot's previous super-block is decoded;
//   * warps 2-9 decode: two groups of four warps take alternate K steps, so each has two step times for
//     its chain of waits, loads and stores; a thread sits on the tensor-memory lane of its weight row and
//     decodes the row's 64 weights of the step to fp32 exactly as the block format defines them (Q4_K:
//     d*sc*nib - dmin*m with ONE rounding; Q6_K: d*sc*(q-32), exact; Q8_0: scale*code, exact), round
//     ONCE to the activation type and store 32 packed columns.  Codes become floats without a
//     conversion instruction (a byte permute drops the code into the mantissa of 2^23) and the
//     arithmetic runs on the two-wide fp32 instructions (add/mul/fma .f32x2);
//   * warp 1 (one lane) issues four tcgen05.mma (M = 128, N = 256, K = 16) per step into a 256-column
//     fp32 accumulator and releases the stage with tcgen05.commit; the wait for the next stage overlaps
//     the MMAs just queued.
// Four stages of tokens (shared memory) and decoded weights (tensor memory) and two or three of packed
// rows run ahead across tile boundaries.  Warps 11-18 drain the finished accumulator with tcgen05.ld into
// REGISTERS (64 packed pairs per thread), hand tensor memory back to the MMA warp at once, and only then
// store C (each lane one weight row: a warp writes 64 contiguous bytes per token) while the next tile's
// MMAs already run.
// Every wait is bounded: on a time-out the sticky device error word is set, the CTA still frees its
// tensor memory and returns.
#include <cuda.h>

#include "linear.cuh"

namespace alloyb {


namespace tc {

__device__ int g_tc_error = 0;          // sticky: a bounded wait of this file's kernel ran out

constexpr int BM = 256;                 // tokens per tile (UMMA N)
constexpr int BN = 128;                 // weight rows per tile (UMMA M = tensor-memory lanes)
constexpr int BK = 64;                  // K step: 64 x 2 bytes = one 128-byte swizzle row
constexpr int STAGES = 4;
constexpr int X_STAGE = BM * BK * 2;    // 32 KB of tokens
constexpr int W_COLS = BK / 2;          // tensor-memory columns of one decoded weight stage (two per column)
constexpr int ACC_COLS = BM;            // fp32 accumulator: one column per token
constexpr int TMEM_COLS = 512;          // 256 accumulator + 4 x 32 weights, rounded up to a power of two
// One super-block of 128 packed rows in shared memory:
//   Q4_K  144-byte rows (9 x 16 bytes: 128-bit reads of 8 consecutive rows hit distinct banks);
//   Q6_K  240-byte rows: the 16-byte-aligned window around the 210-byte block (15 x 16 bytes);
//   Q8_0  two [128 rows x 128 codes] tiles in the 128-byte swizzle, then 16 bytes of scales per row.
constexpr int Q4_ROW = 144, Q6_ROW = 240;
constexpr int Q8_HALF = BN * 128;           // 16 KB
constexpr int Q4_STAGE = BN * Q4_ROW, Q6_STAGE = BN * Q6_ROW, Q8_STAGE = 2 * Q8_HALF + BN * 16;
constexpr int PACK_MAX_STAGES = 3;          // Q4_K and Q6_K run three deep, Q8_0 two
constexpr int PACK_BYTES = 3 * Q6_STAGE;    // 90 KB: 3 x Q4_K, 3 x Q6_K or 2 x Q8_0 stages
static_assert(2 * Q8_STAGE <= PACK_BYTES && 3 * Q4_STAGE <= PACK_BYTES, "packed-row region");
constexpr int DEC_THREADS = 256;        // two groups of 128 (one thread per weight row) on alternate k-steps
constexpr int DEC_GROUP = 128;
constexpr int EPI_THREADS = 256;        // two per accumulator lane (128 token columns each)
// warp 0 token copies, warp 1 MMA, warps 2-9 decode, warp 10 packed-row copies, warps 11-18 epilogue
constexpr int THREADS = 64 + DEC_THREADS + 32 + EPI_THREADS;
constexpr uint32_t SPIN = 1u << 22;

struct Bars {
    uint64_t full[STAGES];        // token-tile copy (1 arrival + bytes) and decode (128 arrivals) -> MMA
    uint64_t empty[STAGES];       // MMA -> token copies + decode (tcgen05.commit)
    uint64_t p_full[PACK_MAX_STAGES];     // packed-row copies -> decode
    uint64_t p_empty[PACK_MAX_STAGES];    // decode -> copies (256 arrivals)
    uint64_t acc_full;            // MMA -> epilogue (tcgen05.commit)
    uint64_t acc_empty;           // epilogue -> MMA (256 arrivals)
    uint32_t tmem_base;
    uint32_t pad;
};

constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * X_STAGE + PACK_BYTES + 256;
static_assert(sizeof(Bars) <= 256, "barrier block");

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
__device__ __forceinline__ bool bar_test(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(s32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_wait(uint64_t* b, uint32_t parity) {
    if (bar_test(b, parity)) return true;       // the usual case: the phase completed long ago
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
// D[tmem_d] (+)= A[tmem_a] * B[shared, db]^T: the A operand (128 lanes x 8 columns of 16-bit pairs per
// K = 16) is read from tensor memory.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with the shared-memory descriptor given as its two halves (the low one carries the address)
// and accumulation always on.
__device__ __forceinline__ void umma_ts_acc(uint32_t tmem_d, uint32_t tmem_a, uint32_t db_lo, uint32_t db_hi,
                                            uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 d;\n\tsetp.eq.u32 p, 0, 0;\n\tmov.b64 d, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(db_lo), "r"(db_hi), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void umma_ts_first(uint32_t tmem_d, uint32_t tmem_a, uint32_t db_lo, uint32_t db_hi,
                                              uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 d;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 d, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(db_lo), "r"(db_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_a(uint32_t bar_addr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
// Shared-address forms of the barrier test and the bounded wait behind it.
__device__ __forceinline__ bool bar_test_a(uint32_t bar_addr, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar_addr), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __noinline__ bool bar_wait_slow(uint32_t bar_addr, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar_addr), "r"(parity)
            : "memory");
        if (ok) return true;
        if (i > 32) __nanosleep(64);
    }
    atomicExch(&g_tc_error, 2);
    return false;
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
__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(addr));
}
// Eight 32-bit columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_st8(uint32_t addr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(addr), "r"(v[0]),
                 "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
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

// The same with the code in mantissa bits 16-22 (code < 128): the floats 2^16 * (128 + code).
template <int E>
__device__ __forceinline__ uint64_t magic2_hi(uint32_t codes) {
    return f2(__uint_as_float(__byte_perm(codes, 0x4B000000u, 0x7044 | (E << 8))),
              __uint_as_float(__byte_perm(codes, 0x4B000000u, 0x7044 | ((E + 1) << 8))));
}

// Gate in front of a thread's first tensor-memory store of a k-step: the stage must have been released by
// the MMAs that read it last.  `free_now` is the result of a test issued before the decode arithmetic.
struct StageGate {
    uint32_t bar, parity;
    bool free_now, ok;
    __device__ __forceinline__ void pass() {
        if (!free_now) {
            ok = bar_wait_slow(bar, parity);
            free_now = true;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
};

// Decode k-step `ks` (0..3) of one Q4_K super-block of this thread's row: 64 weights = the low
// nibbles (sub-block 2*ks, k 0..31 -> columns 0..15) and the high nibbles (sub-block 2*ks + 1,
// k 32..63 -> columns 16..31) of 32 quant bytes.
template <bool BF16>
__device__ __forceinline__ void decode_q4k(const uint8_t* blk, int ks, uint32_t dst, StageGate& gate) {
    const uint4 hdr = lds_u128(blk);
    const uint4 q0 = lds_u128(blk + 16 + ks * 32), q1 = lds_u128(blk + 32 + ks * 32);
    const float d = half_bits_to_f32(hdr.x & 0xffffu), dmin = half_bits_to_f32(hdr.x >> 16);
    const uint64_t unbias = f2(-8388608.0f, -8388608.0f);
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int pl = 0; pl < 2; ++pl) {                     // nibble plane = sub-block 2*ks + pl
        int sc, mn;
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * ks + pl, sc, mn);
        const float dl = d * static_cast<float>(sc), ml = dmin * static_cast<float>(mn);
        const uint64_t dl2 = f2(dl, dl), ml2 = f2(-ml, -ml);
        uint32_t out[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t n4 = (qw[i] >> (4 * pl)) & 0x0f0f0f0fu;
            // (2^23 + nib) - 2^23 is exact; then exact product and ONE rounding at the subtract (FMA)
            out[2 * i] = pack2<BF16>(f2_fma(f2_add(magic2<0>(n4), unbias), dl2, ml2));
            out[2 * i + 1] = pack2<BF16>(f2_fma(f2_add(magic2<2>(n4), unbias), dl2, ml2));
        }
        if (pl == 0) gate.pass();
        tmem_st8(dst + 16 * pl, out);
        tmem_st8(dst + 16 * pl + 8, out + 8);
    }
}

// Q6_K: the block sits at `blk` (2-byte aligned inside its 16-byte-aligned window).  k-step ks covers
// elements 64*ks .. +63 = sub-rows j = jb, jb+1 of half h (32 elements = 16 columns each).  Sub-row j
// takes the low (j < 2) or high nibbles of ql bytes 32*(j&1) .. +31 and bit pair j of qh bytes 0..31.
// Each run is read as nine 4-byte-aligned words and shifted into place; the 16 columns of a sub-row
// go to tensor memory at `dst` + 16*jj as soon as they are ready.
template <bool BF16>
__device__ __forceinline__ void decode_q6k(const uint8_t* blk, int ks, uint32_t dst, StageGate& gate) {
    const int h = ks >> 1, jb = (ks & 1) * 2;
    const float d = half_bits_to_f32(lds_u16(blk + 208));
    const uint32_t sc4 = lds_u16(blk + 192 + h * 8 + 2 * jb) | (lds_u16(blk + 194 + h * 8 + 2 * jb) << 16);
    const uint32_t a_ql = s32(blk + h * 64), a_qh = s32(blk + 128 + h * 32);
    const uint32_t sh = (a_ql & 3u) * 8u;                          // 0 or 16: same for all runs
    uint32_t wh[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wh[i]) : "r"((a_qh & ~3u) + 4 * i));
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
        uint32_t wl[9];
#pragma unroll
        for (int i = 0; i < 9; ++i)
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wl[i]) : "r"((a_ql & ~3u) + 32 * jj + 4 * i));
        const float s0 = d * static_cast<float>(static_cast<int8_t>((sc4 >> (16 * jj)) & 0xffu));
        const float s1 = d * static_cast<float>(static_cast<int8_t>((sc4 >> (16 * jj + 8)) & 0xffu));
        // The code byte sits in mantissa bits 16-22 of 2^23: f = 2^16 * (128 + q).  With t = s * 2^-16,
        // fma(t, f, -160 * s) = s * (q - 32): both constants and the result are exact in fp32.
        const uint64_t t02 = f2(s0 * 0x1p-16f, s0 * 0x1p-16f), t12 = f2(s1 * 0x1p-16f, s1 * 0x1p-16f);
        const uint64_t c02 = f2(-160.0f * s0, -160.0f * s0), c12 = f2(-160.0f * s1, -160.0f * s1);
        // one funnel shift realigns the run AND brings the wanted nibble / bit pair down; what it drags
        // in from the next word lands in masked bits
        const uint32_t shq = sh + (jb >= 2 ? 4u : 0u), shh = sh + 2u * (jb + jj);
        uint32_t out[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t ql = __funnelshift_r(wl[i], wl[i + 1], shq), qh = __funnelshift_r(wh[i], wh[i + 1], shh);
            // four 6-bit codes, one per byte: nibble | (two high bits << 4)
            const uint32_t q = (ql & 0x0f0f0f0fu) + (qh & 0x03030303u) * 16u;
            const bool first = i < 4;                    // elements 0-15 / 16-31 of the sub-row
            out[2 * i] = pack2<BF16>(f2_fma(magic2_hi<0>(q), first ? t02 : t12, first ? c02 : c12));
            out[2 * i + 1] = pack2<BF16>(f2_fma(magic2_hi<2>(q), first ? t02 : t12, first ? c02 : c12));
        }
        if (jj == 0) gate.pass();
        tmem_st8(dst + 16 * jj, out);
        tmem_st8(dst + 16 * jj + 8, out + 8);
    }
}

// Q8_0: `st` is the stage: two [128 rows x 128 codes] tiles in the 128-byte swizzle, then eight fp16 scales
// per row.  k-step ks: elements 64*ks .. +63 = two 32-element blocks; w = scale * code (exact in fp32).
template <bool BF16>
__device__ __forceinline__ void decode_q8_0(const uint8_t* st, int ks, int r, uint32_t dst, StageGate& gate) {
    const uint32_t scw = lds_u32(st + 2 * Q8_HALF + r * 16 + ks * 4);
    const uint8_t* row = st + (ks >> 1) * Q8_HALF + (r >> 3) * 1024 + (r & 7) * 128;
    const uint64_t unbias = f2(-8388736.0f, -8388736.0f);     // -(2^23 + 128)
#pragma unroll
    for (int c = 0; c < 4; ++c) {                        // 16 codes per 16-byte chunk, two chunks per block
        const float sc = half_bits_to_f32((scw >> (16 * (c >> 1))) & 0xffffu);
        const uint64_t sc2 = f2(sc, sc);
        const int chunk = (ks & 1) * 4 + c;
        const uint4 v = lds_u128(row + ((chunk ^ (r & 7)) << 4));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t out[8];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const uint32_t u = w[jj] ^ 0x80808080u;      // code + 128 as an unsigned byte
            out[2 * jj] = pack2<BF16>(f2_mul(f2_add(magic2<0>(u), unbias), sc2));
            out[2 * jj + 1] = pack2<BF16>(f2_mul(f2_add(magic2<2>(u), unbias), sc2));
        }
        if (c == 0) gate.pass();
        tmem_st8(dst + 8 * c, out);
    }
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
               const __grid_constant__ CUtensorMap smap, const Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* x_st = smem;                                   // STAGES x 32 KB token tiles
    uint8_t* p_st = smem + STAGES * X_STAGE;                // packed rows
    Bars* bars = reinterpret_cast<Bars*>(p_st + PACK_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = P.K / QK_K, ksteps = nsb * 4;
    const int tiles_n = (P.N + BN - 1) / BN, tiles_m = (P.M + BM - 1) / BM, n_tiles = tiles_n * tiles_m;
    const int pstages = P.format == ALLOYB_Q8_0 ? 2 : 3;
    const int pstage_bytes = P.format == ALLOYB_Q4_K ? Q4_STAGE : (P.format == ALLOYB_Q6_K ? Q6_STAGE : Q8_STAGE);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            bar_init(&bars->full[s], 1 + DEC_GROUP);
            bar_init(&bars->empty[s], 1);
        }
        for (int s = 0; s < PACK_MAX_STAGES; ++s) {
            bar_init(&bars->p_full[s], 1);
            bar_init(&bars->p_empty[s], DEC_THREADS);
        }
        bar_init(&bars->acc_full, 1);
        bar_init(&bars->acc_empty, EPI_THREADS);
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
    const uint32_t tmem = bars->tmem_base;          // accumulator: columns 0..255; weight stages behind it
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------ token tiles
        bool ok = true;
        uint32_t it = 0;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            const int m0 = (t / tiles_n) * BM;
            for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
                const uint32_t s = it % STAGES;
                if (it >= STAGES) ok = bar_wait(&bars->empty[s], ((it / STAGES) - 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    bar_expect(&bars->full[s], X_STAGE);
                    tma_2d(x_st + s * X_STAGE, &xmap, ks * BK, m0, &bars->full[s]);
                }
                __syncwarp();
            }
        }
    } else if (warp == 10) {
        // ------------------------------------------------ packed rows: one tensor copy per super-block
        bool ok = true;
        uint32_t sbi = 0;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            const int n0 = (t % tiles_n) * BN;
            for (int sb = 0; sb < nsb && ok; ++sb, ++sbi) {
                const uint32_t ps = sbi % pstages;
                if (sbi >= static_cast<uint32_t>(pstages)) ok = bar_wait(&bars->p_empty[ps], ((sbi / pstages) - 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    uint8_t* dst = p_st + ps * pstage_bytes;
                    if (P.format == ALLOYB_Q4_K) {
                        bar_expect(&bars->p_full[ps], Q4_STAGE);
                        tma_2d(dst, &wmap, sb * Q4K_BYTES, n0, &bars->p_full[ps]);
                    } else if (P.format == ALLOYB_Q6_K) {
                        // a block is 2-byte aligned: copy the aligned window around it (reads past the
                        // row's end are filled with zeros)
                        bar_expect(&bars->p_full[ps], Q6_STAGE);
                        tma_2d(dst, &wmap, (sb * Q6K_BYTES) & ~15, n0, &bars->p_full[ps]);
                    } else {
                        bar_expect(&bars->p_full[ps], Q8_STAGE);
                        tma_2d(dst, &wmap, sb * 256, n0, &bars->p_full[ps]);
                        tma_2d(dst + Q8_HALF, &wmap, sb * 256 + 128, n0, &bars->p_full[ps]);
                        tma_2d(dst + 2 * Q8_HALF, &smap, sb * 16, n0, &bars->p_full[ps]);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issue (one lane)
        // The tensor pipe queues about one instruction behind the running one, so nothing slow may sit
        // between two issues: the wait for the NEXT stage is placed before the last MMA of this one
        // (two MMAs are still in the pipe then) and the rest of the loop is a few instructions.
        // This ONE thread's instruction stream paces the tensor pipe, so the loop is kept to a few dozen
        // instructions per step: descriptors advance by adding to their low word, barriers are addressed
        // by shared address, and the common already-complete wait is a single test.
        const uint32_t idesc = umma_idesc(BF16 ? 1 : 0);
        if (lane == 0) {
            const uint64_t d0 = umma_desc(s32(x_st));
            const uint32_t d_lo = static_cast<uint32_t>(d0), d_hi = static_cast<uint32_t>(d0 >> 32);
            const uint32_t full0 = s32(&bars->full[0]), empty0 = s32(&bars->empty[0]), w_base = tmem + ACC_COLS;
            bool ok = true;
            uint32_t it = 0, tl = 0;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tl) {
                // the epilogue must have read the previous tile's accumulator before it is overwritten
                if (tl > 0) ok = bar_wait(&bars->acc_empty, (tl - 1) & 1);
                if (ok) ok = bar_wait(&bars->full[it % STAGES], (it / STAGES) & 1);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
                    const uint32_t s = it % STAGES;
                    const uint32_t lo = d_lo + s * (X_STAGE >> 4), w0 = w_base + s * W_COLS;
                    umma_ts_first(tmem, w0, lo, d_hi, idesc, ks > 0 ? 1u : 0u);
                    umma_ts_acc(tmem, w0 + 8, lo + 2, d_hi, idesc);
                    umma_ts_acc(tmem, w0 + 16, lo + 4, d_hi, idesc);
                    if (ks + 1 < ksteps) {
                        const uint32_t nb = full0 + 8 * ((it + 1) % STAGES), np = ((it + 1) / STAGES) & 1;
                        if (!bar_test_a(nb, np)) ok = bar_wait_slow(nb, np);
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    }
                    umma_ts_acc(tmem, w0 + 24, lo + 6, d_hi, idesc);
                    umma_commit_a(empty0 + 8 * s);
                }
                if (ok) umma_commit(&bars->acc_full);
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ------------------------------------------------ decode: thread = weight row = the tensor-memory
        // lane this warp may access (its index modulo 4 picks the quarter); group g takes k-steps it = g mod 2
        const int r = (warp & 3) * 32 + lane, g = (warp - 2) >> 2;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + ACC_COLS;
        bool ok = true;
        uint32_t it = 0, sbi = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
                const uint32_t ps = sbi % pstages, s = it % STAGES;
                if ((ks & 1) == g) {
                    // first step of this group in the super-block: its packed rows must have landed
                    if (ok && (ks & 3) == g) ok = bar_wait(&bars->p_full[ps], (sbi / pstages) & 1);
                    // the stage's previous use must be over before the first store to it, not before the
                    // loads and the arithmetic: test now, and only wait (inside the decode, right before
                    // its first tensor-memory store) if the test failed
                    const uint32_t e_bar = s32(&bars->empty[s]), e_par = ((it / STAGES) - 1) & 1;
                    const bool free_now = it < STAGES || bar_test_a(e_bar, e_par);
                    if (ok) {
                        const uint8_t* stg = p_st + ps * pstage_bytes;
                        const uint32_t dst = lane_base + s * W_COLS;
                        StageGate gate{e_bar, e_par, free_now, true};
                        // rows past N arrive as zeros from the tensor copy and decode to zeros
                        if (P.format == ALLOYB_Q4_K)
                            decode_q4k<BF16>(stg + r * Q4_ROW, ks & 3, dst, gate);
                        else if (P.format == ALLOYB_Q6_K)
                            decode_q6k<BF16>(stg + r * Q6_ROW + ((static_cast<int>(sbi % nsb) * Q6K_BYTES) & 15), ks & 3, dst, gate);
                        else
                            decode_q8_0<BF16>(stg, ks & 3, r, dst, gate);
                        ok = gate.ok;
                        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    }
                    bar_arrive(&bars->full[s]);
                    if ((ks & 3) == 2 + g) bar_arrive(&bars->p_empty[ps]);      // this group's last step of the super-block
                }
                if ((ks & 3) == 3) ++sbi;
            }
        }
    } else {
        // ------------------------------------------------ epilogue: TMEM -> registers, release, -> C
        const int quarter = warp & 3;                       // TMEM lanes this warp may read
        const int half = (warp - 11) >> 2;                  // token columns half*128 .. +127
        bool ok = true;
        uint32_t tl = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++tl) {
            const int n0 = (t % tiles_n) * BN, m0 = (t / tiles_n) * BM;
            if (ok) ok = bar_wait(&bars->acc_full, tl & 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t acc[BM / 4];                           // 128 tokens of this lane's row, two per register
            if (ok) {
                const uint32_t src = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + half * (BM / 2);
#pragma unroll
                for (int c = 0; c < BM / 16; ++c) {
                    uint32_t v[8];
                    tmem_ld8(src + c * 8, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        acc[c * 4 + e] = pack2<BF16>(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            bar_arrive(&bars->acc_empty);                   // the accumulator is free: the next tile may start
            if (ok) {
                const int n = n0 + quarter * 32 + lane;     // this lane's weight row = output column
                const int tok0 = m0 + half * (BM / 2);
                if (n < P.N) {
                    uint16_t* col = static_cast<uint16_t*>(P.y) + static_cast<int64_t>(tok0) * P.ldy + n;
#pragma unroll
                    for (int e = 0; e < BM / 4; ++e) {
                        if (tok0 + 2 * e < P.M) col[static_cast<int64_t>(2 * e) * P.ldy] = static_cast<uint16_t>(acc[e] & 0xffffu);
                        if (tok0 + 2 * e + 1 < P.M) col[static_cast<int64_t>(2 * e + 1) * P.ldy] = static_cast<uint16_t>(acc[e] >> 16);
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

    static int sm_count[64] = {};             // per device ordinal; 0 = kernel not configured yet
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!sm_count[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        int sms = 0;
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms <= 0) { set_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidValue); return ALLOYB_E_CUDA; }
        sm_count[dev] = sms;
    }
    // persistent: one CTA per SM walks the tiles (weight-row tile fastest, so neighbours share a token tile)
    const int n_tiles = ((seg.N + BN - 1) / BN) * ((M + BM - 1) / BM);
    const dim3 grid(n_tiles < sm_count[dev] ? n_tiles : sm_count[dev]);
    if (dtype == ALLOYB_BF16) gemm_tc_kernel<true><<<grid, THREADS, SMEM_BYTES, st>>>(map, wmap, smap, P);
    else gemm_tc_kernel<false><<<grid, THREADS, SMEM_BYTES, st>>>(map, wmap, smap, P);
    return check_launch();
}

}  // namespace alloyb

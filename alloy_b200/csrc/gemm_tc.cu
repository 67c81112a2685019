// Dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a: every linear of the path
// with more than a handful of tokens (prefill, verification chunks, batched decode).
//
//   C[M tokens, N] = X[M, K] (bf16 | fp16)  *  deq(W)[N, K]^T  (+ residual)     fp32 accumulate, C in X's type
//   C = act(X G^T) * (X U^T)  for a gate/up pair (up to 128 tokens)
//
// A persistent kernel: one CTA per SM walks work items = (tile of 128 weight rows x BM tokens, K range),
// BM in {32, 64, 128, 256} chosen from M.  In the MMA the WEIGHT rows are the M = 128 operand and the
// tokens are N, and the decoded weights never touch shared memory: the decode warps write them straight
// into TENSOR MEMORY (tcgen05.st), from where tcgen05.mma reads its A operand, so the only shared-memory
// traffic of the tensor pipe is the token tile -- shared-memory bandwidth is what bounds this kernel
// otherwise.  Per 64-wide K step:
//   * warp 0 (one lane) brings the BM x 64 token tile in with ONE TMA tensor copy (128-byte swizzle);
//   * the packed-row warp (one lane) brings the 128 packed weight rows of a super-block (four K steps) in
//     with ONE tensor copy over a byte view of the weight matrix (Q8_0: two swizzled copies of codes and
//     one of scales), issued as soon as the slot's previous super-block is decoded;
//   * the decode warps work in DG groups of four warps that take K steps round robin, so each group has
//     DG step times for its chain of waits, loads and stores (DG = 2 under the 256-token tile, whose
//     epilogue needs the registers; 4 otherwise, where decode alone bounds the kernel); a thread sits on the
//     tensor-memory lane of its weight row and decodes the row's 64 weights of the step to fp32 exactly
//     as the block format defines them (Q4_K: d*sc*nib - dmin*m with ONE rounding; Q6_K: d*sc*(q-32),
//     exact; Q8_0: scale*code, exact), rounds ONCE to the activation type and stores 32 packed columns.
//     Codes become floats without a conversion instruction (a byte permute drops the code into the
//     mantissa of 2^23) and the arithmetic runs on the two-wide fp32 instructions (add/mul/fma .f32x2);
//   * warp 1 (one lane) issues four tcgen05.mma (M = 128, N = BM, K = 16) per step into a BM-column fp32
//     accumulator and releases the stage with tcgen05.commit; the wait for the next stage sits before the
//     last MMA of the step.
// Four stages of tokens (shared memory) and decoded weights (tensor memory) and two or three of packed
// rows run ahead across item boundaries.  Eight epilogue warps drain the finished accumulator with
// tcgen05.ld into REGISTERS, hand tensor memory back to the MMA warp at once, and only then store C (each
// lane one weight row: a warp writes 64 contiguous bytes per token) while the next item's MMAs run.
// When a matrix has fewer row tiles than the GPU has SMs and all tokens fit one tile, K is split: every
// item adds its partial tile to a zeroed fp32 buffer (red.global) and the LAST item of a tile to finish
// (a per-tile counter) reads the sums back, applies residual / activation, stores C and re-zeroes both.
// A gate/up pair runs as two K loops into two accumulators; the epilogue combines them.
// Every wait is bounded: on a time-out the sticky device error word is set, the CTA still frees its
// tensor memory and returns.
#include <cuda.h>

#include <climits>

#include "linear.cuh"

namespace alloyb {


namespace tc {

__device__ int g_tc_error = 0;          // sticky: a bounded wait of this file's kernel ran out

constexpr int BN = 128;                 // weight rows per tile (UMMA M = tensor-memory lanes)
constexpr int BK = 64;                  // K step: 64 x 2 bytes = one 128-byte swizzle row
constexpr int MAX_STAGES = 8;
constexpr int W_COLS = BK / 2;          // tensor-memory columns of one decoded weight stage (two per column)
// One super-block of 128 packed rows in shared memory:
//   Q4_K  144-byte rows (9 x 16 bytes: 128-bit reads of 8 consecutive rows hit distinct banks);
//   Q6_K  240-byte rows: the 16-byte-aligned window around the 210-byte block (15 x 16 bytes);
//   Q8_0  two [128 rows x 128 codes] tiles in the 128-byte swizzle, then 16 bytes of scales per row.
constexpr int Q4_ROW = 144, Q6_ROW = 240;
constexpr int Q8_HALF = BN * 128;           // 16 KB
constexpr int Q4_STAGE = BN * Q4_ROW, Q6_STAGE = BN * Q6_ROW, Q8_STAGE = 2 * Q8_HALF + BN * 16;
constexpr int PACK_MAX_STAGES = 5;          // Q4_K runs five deep, Q6_K three, Q8_0 two
constexpr int PACK_BYTES = 3 * Q6_STAGE;    // 90 KB: 5 x Q4_K, 3 x Q6_K or 2 x Q8_0 stages
static_assert(2 * Q8_STAGE <= PACK_BYTES && 5 * Q4_STAGE <= PACK_BYTES, "packed-row region");
// A super-block of rows comes in as PACK_BOXES tensor copies of PACK_BOX_ROWS rows each: the copy unit
// walks a box row by row, and several short boxes in flight finish sooner than one tall one.
constexpr int PACK_BOXES = 4, PACK_BOX_ROWS = BN / PACK_BOXES;
constexpr int DEC_GROUP = 128;          // one decode group: a thread per weight row
constexpr int EPI_THREADS = 256;        // two per accumulator lane (half of the token columns each)
constexpr uint32_t SPIN = 1u << 22;
// Split-K scratch: fp32 sums [token][row] for up to SPLIT_MAX_ROWS rows (x 2 planes for a gate/up pair)
// and SPLIT_MAX_BM tokens, and one counter per row tile.  Zero at load, re-zeroed by whoever finishes a
// tile, so two GEMMs that split K must not overlap in time on one device.
constexpr int SPLIT_MAX_TILES = 147, SPLIT_MAX_ROWS = SPLIT_MAX_TILES * BN, SPLIT_MAX_BM = 128;
__device__ float g_split_sum[2 * SPLIT_MAX_BM * SPLIT_MAX_ROWS];
__device__ unsigned int g_split_count[SPLIT_MAX_TILES];

template <int BM, int DG>
struct Cfg {
    static constexpr int X_STAGE = BM * BK * 2;                 // one token tile
    // Stages of tokens (shared memory) and decoded weights (tensor memory).  With DG decode groups on
    // DG stages every group would wait for the MMAs of its own previous step before it may store the
    // next one; twice as many stages let it run a step ahead.
    static constexpr int STAGES = BM <= 128 ? 8 : 4;
    static constexpr int DEC_WARPS = 4 * DG;
    static constexpr int PACK_WARP = 2 + DEC_WARPS;             // warp 0 token copies, warp 1 MMA, then decode
    static constexpr int EPI_WARP0 = PACK_WARP + 1;
    // Under a narrow token tile an MMA is short and the issuing thread's own instruction stream (about a
    // hundred cycles per tcgen05.mma) would pace the steps: NI threads (warp 1 and NI - 1 warps behind the
    // epilogue's) then issue a quarter or a half of every step's MMAs each, into an accumulator of their
    // own, and the epilogue adds the accumulators up.  (Worth 7 %: the decode warps bound these shapes.)
    static constexpr int NI = BM <= 32 ? 4 : (BM <= 64 ? 2 : 1);
    static constexpr int MMA_WARP1 = EPI_WARP0 + EPI_THREADS / 32;      // issuers 1 .. NI-1
    static constexpr int THREADS = (MMA_WARP1 + NI - 1) * 32;
    // accumulators [gate/up][issuer] of BM columns each from column 0, decoded weights behind them
    static constexpr int W_COL0 = 2 * NI * BM <= 256 ? 2 * NI * BM : BM;
    static constexpr int TMEM_COLS = W_COL0 + STAGES * W_COLS <= 256 ? 256 : 512;
    static constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * X_STAGE + PACK_BYTES + 256;
    static_assert(W_COL0 + STAGES * W_COLS <= 512 && STAGES <= MAX_STAGES, "tensor memory");
};

struct Bars {
    uint64_t full[MAX_STAGES];    // token-tile copy (1 arrival + bytes) and decode (128 arrivals) -> MMA
    uint64_t empty[MAX_STAGES];   // MMA -> token copies + decode (tcgen05.commit)
    uint64_t p_full[PACK_MAX_STAGES];     // packed-row copies -> decode
    uint64_t p_empty[PACK_MAX_STAGES];    // decode -> copies (one arrival per decode thread)
    uint64_t acc_full;            // MMA -> epilogue (tcgen05.commit)
    uint64_t acc_empty;           // epilogue -> MMA (256 arrivals)
    uint32_t tmem_base;
    uint32_t last;                // split-K: this CTA finished a tile last
};
static_assert(sizeof(Bars) <= 256, "barrier block");

struct Maps {
    CUtensorMap x;                // tokens
    CUtensorMap w[2];             // packed rows as bytes (gate/up: both matrices)
    CUtensorMap s[2];             // Q8_0 scales
};

struct Params {
    int format;               // ALLOYB_Q4_K / ALLOYB_Q6_K / ALLOYB_Q8_0
    void* y;
    const void* residual;     // same shape and pitch as y, or null
    int64_t ldy;
    int M, N, K;
    int splits;               // K ranges per row tile (1: the item owns its output tile)
    int gated, act;           // gate/up pair: y = act(gate) * up
    // Two matrices that lie back to back in memory run as one: rows from n_split on belong to the second
    // one and go to its own output (INT_MAX: a single matrix).
    int n_split;
    void* y2;
    int64_t ldy2;
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
// kind::f16: D fp32, A/B both bf16 (1) or fp16 (0), both K-major, M = BN weight rows, N = `tokens`.
__device__ __forceinline__ uint32_t umma_idesc(int is_bf16, int tokens) {
    uint32_t d = 0;
    d |= 1u << 4;                                   // D format F32
    d |= static_cast<uint32_t>(is_bf16 ? 1 : 0) << 7;    // A format
    d |= static_cast<uint32_t>(is_bf16 ? 1 : 0) << 10;   // B format
    d |= static_cast<uint32_t>(tokens >> 3) << 17;  // N
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

// One work item: a tile of 128 weight rows x BM tokens over super-blocks [sb0, sb1).
struct Item {
    int n0, tile_n, tile_m, sb0, sb1;
};
__device__ __forceinline__ Item item_of(int w, int tiles_n, int tiles_m, int nsb, int splits) {
    Item it;
    it.tile_n = w % tiles_n;
    const int r = w / tiles_n, split = r / tiles_m;
    it.n0 = it.tile_n * BN;
    it.tile_m = r % tiles_m;
    it.sb0 = static_cast<int>(static_cast<int64_t>(split) * nsb / splits);
    it.sb1 = static_cast<int>(static_cast<int64_t>(split + 1) * nsb / splits);
    return it;
}

__device__ __forceinline__ float apply_act(float g, int act) {
    if (act == ALLOYB_ACT_SILU) return g / (1.0f + __expf(-g));
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(u));
}

template <bool BF16>
__device__ __forceinline__ float to_f32(uint16_t v) {
    return BF16 ? __uint_as_float(static_cast<uint32_t>(v) << 16) : half_bits_to_f32(v);
}
template <bool BF16>
__device__ __forceinline__ uint16_t to_16(float v) {
    return static_cast<uint16_t>(pack2<BF16>(v, 0.0f) & 0xffffu);
}

// Eight columns of this thread's lane, summed over the NI issuers' accumulators (BM columns apart).
template <int NI, int BM>
__device__ __forceinline__ void load_sum(uint32_t addr, uint32_t (&v)[8]) {
    tmem_ld8(addr, v);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int a = 1; a < NI; ++a) {
        uint32_t t[8];
        tmem_ld8(addr + a * BM, t);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(t[e]));
    }
}

template <bool BF16, int BM, int DG>
__global__ void __launch_bounds__(Cfg<BM, DG>::THREADS, 1)
gemm_tc_kernel(const __grid_constant__ Maps maps, const Params P) {
    using C = Cfg<BM, DG>;
    constexpr int X_STAGE = C::X_STAGE, STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* x_st = smem;                                   // STAGES token tiles
    uint8_t* p_st = smem + STAGES * X_STAGE;                // packed rows
    Bars* bars = reinterpret_cast<Bars*>(p_st + PACK_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = P.K / QK_K;
    const int tiles_n = (P.N + BN - 1) / BN, tiles_m = (P.M + BM - 1) / BM, n_items = tiles_n * tiles_m * P.splits;
    const int n_sub = P.gated ? 2 : 1;                      // K loops (accumulators) per item
    const int pstages = P.format == ALLOYB_Q4_K ? 5 : (P.format == ALLOYB_Q6_K ? 3 : 2);
    const int pstage_bytes = P.format == ALLOYB_Q4_K ? Q4_STAGE : (P.format == ALLOYB_Q6_K ? Q6_STAGE : Q8_STAGE);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            bar_init(&bars->full[s], 1 + DEC_GROUP);
            bar_init(&bars->empty[s], C::NI);
        }
        for (int s = 0; s < PACK_MAX_STAGES; ++s) {
            bar_init(&bars->p_full[s], 1);
            bar_init(&bars->p_empty[s], DG * DEC_GROUP);
        }
        bar_init(&bars->acc_full, C::NI);
        bar_init(&bars->acc_empty, EPI_THREADS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {      // tensor memory: one warp allocates, the same warp frees
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&bars->tmem_base)),
                     "r"(C::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;          // accumulator(s) from column 0; weight stages at W_COL0
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------ token tiles
        bool ok = true;
        uint32_t it = 0;
        for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
            const Item im = item_of(w, tiles_n, tiles_m, nsb, P.splits);
            for (int sub = 0; sub < n_sub && ok; ++sub) {
                for (int ks = im.sb0 * 4; ks < im.sb1 * 4 && ok; ++ks, ++it) {
                    const uint32_t s = it % STAGES;
                    if (it >= STAGES) ok = bar_wait(&bars->empty[s], ((it / STAGES) - 1) & 1);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    if (lane == 0) {
                        bar_expect(&bars->full[s], X_STAGE);
                        tma_2d(x_st + s * X_STAGE, &maps.x, ks * BK, im.tile_m * BM, &bars->full[s]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == C::PACK_WARP) {
        // ------------------------------------------------ packed rows: one tensor copy per super-block
        bool ok = true;
        uint32_t sbi = 0;
        for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
            const Item im = item_of(w, tiles_n, tiles_m, nsb, P.splits);
            for (int sub = 0; sub < n_sub && ok; ++sub) {
                for (int sb = im.sb0; sb < im.sb1 && ok; ++sb, ++sbi) {
                    const uint32_t ps = sbi % pstages;
                    if (sbi >= static_cast<uint32_t>(pstages)) ok = bar_wait(&bars->p_empty[ps], ((sbi / pstages) - 1) & 1);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    if (lane == 0) {
                        uint8_t* dst = p_st + ps * pstage_bytes;
                        if (P.format == ALLOYB_Q4_K) {
                            bar_expect(&bars->p_full[ps], Q4_STAGE);
#pragma unroll
                            for (int b = 0; b < PACK_BOXES; ++b)
                                tma_2d(dst + b * PACK_BOX_ROWS * Q4_ROW, &maps.w[sub], sb * Q4K_BYTES, im.n0 + b * PACK_BOX_ROWS,
                                       &bars->p_full[ps]);
                        } else if (P.format == ALLOYB_Q6_K) {
                            // a block is 2-byte aligned: copy the aligned window around it (reads past the
                            // row's end are filled with zeros)
                            bar_expect(&bars->p_full[ps], Q6_STAGE);
#pragma unroll
                            for (int b = 0; b < PACK_BOXES; ++b)
                                tma_2d(dst + b * PACK_BOX_ROWS * Q6_ROW, &maps.w[sub], (sb * Q6K_BYTES) & ~15,
                                       im.n0 + b * PACK_BOX_ROWS, &bars->p_full[ps]);
                        } else {
                            bar_expect(&bars->p_full[ps], Q8_STAGE);
#pragma unroll
                            for (int b = 0; b < PACK_BOXES; ++b) {
                                const int r0 = b * PACK_BOX_ROWS;
                                tma_2d(dst + r0 * 128, &maps.w[sub], sb * 256, im.n0 + r0, &bars->p_full[ps]);
                                tma_2d(dst + Q8_HALF + r0 * 128, &maps.w[sub], sb * 256 + 128, im.n0 + r0, &bars->p_full[ps]);
                                tma_2d(dst + 2 * Q8_HALF + r0 * 16, &maps.s[sub], sb * 16, im.n0 + r0, &bars->p_full[ps]);
                            }
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 1 || warp >= C::MMA_WARP1) {
        // ------------------------------------------------ MMA issue (one lane per issuer)
        // This ONE thread's instruction stream paces the tensor pipe (which queues about one instruction
        // behind the running one), so the loop is kept to a few dozen instructions per step: descriptors
        // advance by adding to their low word, barriers are addressed by shared address, the common
        // already-complete wait is a single test, and the wait for the NEXT stage sits before the last
        // MMA of this one, while two MMAs are still in the pipe.
        const uint32_t idesc = umma_idesc(BF16 ? 1 : 0, BM);
        if (lane == 0) {
            const uint64_t d0 = umma_desc(s32(x_st));
            const uint32_t d_lo = static_cast<uint32_t>(d0), d_hi = static_cast<uint32_t>(d0 >> 32);
            const uint32_t full0 = s32(&bars->full[0]), empty0 = s32(&bars->empty[0]), w_base = tmem + C::W_COL0;
            constexpr int NI = C::NI, KK = 4 / NI;              // this issuer's MMAs per step: kk0 .. kk0 + KK - 1
            const int issuer = warp == 1 ? 0 : warp - C::MMA_WARP1 + 1, kk0 = issuer * KK;
            bool ok = true;
            uint32_t it = 0, tl = 0;
            for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++tl) {
                const Item im = item_of(w, tiles_n, tiles_m, nsb, P.splits);
                const int ksteps = (im.sb1 - im.sb0) * 4;
                // the epilogue must have read the previous item's accumulators before they are overwritten
                if (tl > 0) ok = bar_wait(&bars->acc_empty, (tl - 1) & 1);
                for (int sub = 0; sub < n_sub && ok; ++sub) {
                    const uint32_t acc = tmem + (sub * NI + issuer) * BM;
                    ok = bar_wait(&bars->full[it % STAGES], (it / STAGES) & 1);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t lo = d_lo + s * (X_STAGE >> 4) + 2 * kk0, w0 = w_base + s * W_COLS + 8 * kk0;
                        umma_ts_first(acc, w0, lo, d_hi, idesc, ks > 0 ? 1u : 0u);
                        if (KK == 4) {
                            umma_ts_acc(acc, w0 + 8, lo + 2, d_hi, idesc);
                            umma_ts_acc(acc, w0 + 16, lo + 4, d_hi, idesc);
                        }
                        if (ks + 1 < ksteps) {
                            const uint32_t nb = full0 + 8 * ((it + 1) % STAGES), np = ((it + 1) / STAGES) & 1;
                            if (!bar_test_a(nb, np)) ok = bar_wait_slow(nb, np);
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        if (KK >= 2) umma_ts_acc(acc, w0 + 8 * (KK - 1), lo + 2 * (KK - 1), d_hi, idesc);
                        umma_commit_a(empty0 + 8 * s);
                    }
                }
                if (ok) umma_commit(&bars->acc_full);
            }
        }
        __syncwarp();
    } else if (warp < C::PACK_WARP) {
        // ------------------------------------------------ decode: thread = weight row = the tensor-memory
        // lane this warp may access (its index modulo 4 picks the quarter); group g takes the k-steps whose
        // running count is g modulo DG
        const int r = (warp & 3) * 32 + lane, g = (warp - 2) >> 2;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + C::W_COL0;
        bool ok = true;
        uint32_t it = 0, sbi = 0;
        for (int w = blockIdx.x; w < n_items; w += gridDim.x) {
            const Item im = item_of(w, tiles_n, tiles_m, nsb, P.splits);
            for (int sub = 0; sub < n_sub; ++sub) {
                for (int sb = im.sb0; sb < im.sb1; ++sb, ++sbi) {
                    const uint32_t ps = sbi % pstages;
                    bool have = false;                   // this thread waited for the super-block's rows
#pragma unroll 1
                    for (int k4 = 0; k4 < 4; ++k4, ++it) {
                        if (static_cast<int>(it % DG) != g) continue;
                        const uint32_t s = it % STAGES;
                        if (ok && !have) ok = bar_wait(&bars->p_full[ps], (sbi / pstages) & 1);
                        have = true;
                        // the stage's previous use must be over before the first store to it, not before
                        // the loads and the arithmetic: test now, and only wait (inside the decode, right
                        // before its first tensor-memory store) if the test failed
                        const uint32_t e_bar = s32(&bars->empty[s]), e_par = ((it / STAGES) - 1) & 1;
                        const bool free_now = it < STAGES || bar_test_a(e_bar, e_par);
                        if (ok) {
                            const uint8_t* stg = p_st + ps * pstage_bytes;
                            const uint32_t dst = lane_base + s * W_COLS;
                            StageGate gate{e_bar, e_par, free_now, true};
                            // rows past N arrive as zeros from the tensor copy and decode to zeros
                            if (P.format == ALLOYB_Q4_K)
                                decode_q4k<BF16>(stg + r * Q4_ROW, k4, dst, gate);
                            else if (P.format == ALLOYB_Q6_K)
                                decode_q6k<BF16>(stg + r * Q6_ROW + ((sb * Q6K_BYTES) & 15), k4, dst, gate);
                            else
                                decode_q8_0<BF16>(stg, k4, r, dst, gate);
                            ok = gate.ok;
                            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        }
                        bar_arrive(&bars->full[s]);
                    }
                    // every decode thread releases the super-block once, after its last step of it (a
                    // group with no step in it -- DG = 4 always has one -- releases it at once)
                    bar_arrive(&bars->p_empty[ps]);
                }
            }
        }
    } else {
        // ------------------------------------------------ epilogue: TMEM -> registers, release, -> C
        constexpr int HT = BM / 2;                          // tokens per thread
        const int ew = warp - C::EPI_WARP0;
        const int quarter = warp & 3;                       // TMEM lanes this warp may read
        const int half = ew >> 2;                           // token columns half*HT .. +HT-1
        const int et = threadIdx.x - C::EPI_WARP0 * 32;     // 0..255
        bool ok = true;
        uint32_t tl = 0;
        for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++tl) {
            const Item im = item_of(w, tiles_n, tiles_m, nsb, P.splits);
            const int n = im.n0 + quarter * 32 + lane;      // this lane's weight row = output column
            const int tok0 = im.tile_m * BM + half * HT;
            if (ok) ok = bar_wait(&bars->acc_full, tl & 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t src = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + half * HT;
            if (P.splits == 1) {
                uint32_t acc[HT / 2];                       // this lane's row, two tokens per register
                if (ok) {
#pragma unroll
                    for (int c = 0; c < HT / 8; ++c) {
                        uint32_t v[8];
                        load_sum<C::NI, BM>(src + c * 8, v);
                        if (P.gated) {
                            uint32_t u[8];
                            load_sum<C::NI, BM>(src + C::NI * BM + c * 8, u);
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                v[e] = __float_as_uint(apply_act(__uint_as_float(v[e]), P.act) * __uint_as_float(u[e]));
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            acc[c * 4 + e] = pack2<BF16>(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                }
                bar_arrive(&bars->acc_empty);               // the accumulators are free: the next item may start
                if (ok && n < P.N) {
                    const bool second = n >= P.n_split;                 // the second of two stacked matrices
                    const int64_t ld = second ? P.ldy2 : P.ldy;
                    uint16_t* col = static_cast<uint16_t*>(second ? P.y2 : P.y) + static_cast<int64_t>(tok0) * ld +
                                    (second ? n - P.n_split : n);
                    const uint16_t* res =
                        P.residual ? static_cast<const uint16_t*>(P.residual) + static_cast<int64_t>(tok0) * P.ldy + n : nullptr;
#pragma unroll
                    for (int e = 0; e < HT; ++e) {
                        if (tok0 + e < P.M) {
                            uint16_t o = static_cast<uint16_t>(e & 1 ? acc[e >> 1] >> 16 : acc[e >> 1] & 0xffffu);
                            // residual: dtype(residual + dtype(acc))
                            if (res) o = to_16<BF16>(to_f32<BF16>(res[static_cast<int64_t>(e) * P.ldy]) + to_f32<BF16>(o));
                            col[static_cast<int64_t>(e) * ld] = o;
                        }
                    }
                }
            } else {
                // split K: add this item's partial tile to the fp32 sums, [plane][token][row]
                const int pitch = tiles_n * BN;
                float* sum = g_split_sum + static_cast<int64_t>(tok0) * pitch + n;
                const int64_t plane = static_cast<int64_t>(SPLIT_MAX_BM) * pitch;
                if (ok) {
                    for (int sub = 0; sub < n_sub; ++sub) {
#pragma unroll
                        for (int c = 0; c < HT / 8; ++c) {
                            uint32_t v[8];
                            load_sum<C::NI, BM>(src + sub * C::NI * BM + c * 8, v);
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (tok0 + c * 8 + e < P.M)
                                    atomicAdd(sum + sub * plane + static_cast<int64_t>(c * 8 + e) * pitch, __uint_as_float(v[e]));
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                }
                bar_arrive(&bars->acc_empty);
                // The last item of the tile to get here finishes it.  One release-acquire count per CTA: the
                // barrier puts the epilogue threads' reductions before thread 0's release, the last CTA's acquire
                // and its barrier put every item's reductions before the loads below.
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
                if (et == 0) {
                    unsigned int old;
                    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(&g_split_count[im.tile_n]) : "memory");
                    bars->last = old == static_cast<unsigned int>(P.splits - 1) ? 1u : 0u;
                    if (bars->last) g_split_count[im.tile_n] = 0u;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
                if (bars->last && ok) {
                    if (n < P.N) {
                        const bool second = n >= P.n_split;
                        const int64_t ld = second ? P.ldy2 : P.ldy;
                        uint16_t* col = static_cast<uint16_t*>(second ? P.y2 : P.y) + static_cast<int64_t>(tok0) * ld +
                                        (second ? n - P.n_split : n);
                        const uint16_t* res = P.residual ? static_cast<const uint16_t*>(P.residual) +
                                                               static_cast<int64_t>(tok0) * P.ldy + n
                                                         : nullptr;
                        // eight tokens' sums (and residuals) are requested together, then finished: one round
                        // trip to L2 per eight tokens instead of one per token
                        constexpr int FB = HT < 8 ? HT : 8;
#pragma unroll 1
                        for (int e0 = 0; e0 < HT; e0 += FB) {
                            float v[FB], u[FB], r[FB];
#pragma unroll
                            for (int j = 0; j < FB; ++j) {
                                const int e = e0 + j;
                                const bool live = tok0 + e < P.M;
                                const float* a = sum + static_cast<int64_t>(e) * pitch;
                                v[j] = live ? __ldcg(a) : 0.f;
                                u[j] = (live && P.gated) ? __ldcg(a + plane) : 0.f;
                                r[j] = (live && res) ? to_f32<BF16>(res[static_cast<int64_t>(e) * P.ldy]) : 0.f;
                            }
#pragma unroll
                            for (int j = 0; j < FB; ++j) {
                                const int e = e0 + j;
                                if (tok0 + e < P.M) {
                                    float* a = sum + static_cast<int64_t>(e) * pitch;
                                    __stcg(a, 0.0f);
                                    float val = v[j];
                                    if (P.gated) {
                                        val = apply_act(val, P.act) * u[j];
                                        __stcg(a + plane, 0.0f);
                                    }
                                    uint16_t o = to_16<BF16>(val);
                                    if (res) o = to_16<BF16>(r[j] + to_f32<BF16>(o));
                                    col[static_cast<int64_t>(e) * ld] = o;
                                }
                            }
                        }
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");     // bars->last may be rewritten
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS));
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

namespace tc {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder is looked up through the runtime, so the library carries no link-time
// dependency on the driver and still loads (for symbol checks) on a machine without one.
static EncodeFn encoder() {
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr);
        if (e != cudaSuccess || qr != cudaDriverEntryPointSuccess || !fn) {
            set_cuda_error(e != cudaSuccess ? e : cudaErrorNotSupported);
            return nullptr;
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    return encode;
}

// 2-D map over a row-major matrix: `inner` elements per row, `rows` rows `pitch` bytes apart.
static bool map2d(EncodeFn encode, CUtensorMap* m, CUtensorMapDataType type, const void* base, uint64_t inner,
                  uint64_t rows, uint64_t pitch, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
    const cuuint64_t gdim[2] = {inner, rows};
    const cuuint64_t gstr[1] = {pitch};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return encode(m, type, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sm_count_of_device(int& dev) {
    static int sms[64] = {};
    dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 0;
        sms[dev] = n;
    }
    return sms[dev];
}

template <bool BF16, int BM, int DG>
static int launch(const Maps& maps, const Params& P, int grid, int dev, cudaStream_t st) {
    static bool configured[64] = {};
    using C = Cfg<BM, DG>;
    if (!configured[dev]) {
        const cudaError_t e =
            cudaFuncSetAttribute(gemm_tc_kernel<BF16, BM, DG>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
        configured[dev] = true;
    }
    gemm_tc_kernel<BF16, BM, DG><<<grid, C::THREADS, C::SMEM_BYTES, st>>>(maps, P);
    return check_launch();
}

template <bool BF16>
static int launch_bm(int BM, const Maps& maps, const Params& P, int grid, int dev, cudaStream_t st) {
    switch (BM) {
        case 32: return launch<BF16, 32, 4>(maps, P, grid, dev, st);
        case 64: return launch<BF16, 64, 4>(maps, P, grid, dev, st);
        case 128: return launch<BF16, 128, 4>(maps, P, grid, dev, st);
        default: return launch<BF16, 256, 2>(maps, P, grid, dev, st);
    }
}

}  // namespace tc

namespace tc {

// y = type(residual + y), rows of N elements `ld` apart, eight elements per thread where the row allows.
template <bool BF16>
__global__ void residual_add_kernel(uint16_t* __restrict__ y, const uint16_t* __restrict__ res, int M, int N, int64_t ld) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = (N + 7) / 8;
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<int64_t>(M) * per_row) return;
    const int m = static_cast<int>(i / per_row), c = static_cast<int>(i % per_row) * 8;
    uint16_t* yp = y + m * ld + c;
    const uint16_t* rp = res + m * ld + c;
    if (c + 8 <= N && ((reinterpret_cast<uintptr_t>(yp) | reinterpret_cast<uintptr_t>(rp)) & 15) == 0) {
        uint4 a = *reinterpret_cast<const uint4*>(yp);
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(rp));
        uint16_t* ah = reinterpret_cast<uint16_t*>(&a);
        const uint16_t* bh = reinterpret_cast<const uint16_t*>(&b);
#pragma unroll
        for (int e = 0; e < 8; ++e) ah[e] = to_16<BF16>(to_f32<BF16>(bh[e]) + to_f32<BF16>(ah[e]));
        *reinterpret_cast<uint4*>(yp) = a;
    } else {
        for (int e = 0; e < 8 && c + e < N; ++e) yp[e] = to_16<BF16>(to_f32<BF16>(rp[e]) + to_f32<BF16>(yp[e]));
    }
}

}  // namespace tc

// Beyond this many tokens the residual is added by a kernel of its own after the GEMM: the GEMM's epilogue
// holds one weight row per thread and fetches its residual values token by token (strided), which a single
// tile per CTA hides and a walk over many tiles does not.
constexpr int GEMM_FUSED_RESIDUAL_MAX_M = 128;

int gemm_tc_residual_add(void* y, const void* residual, int M, int N, int64_t ldy, int dtype, cudaStream_t st) {
    const int64_t threads = static_cast<int64_t>(M) * ((N + 7) / 8);
    const dim3 grid(static_cast<unsigned int>((threads + 255) / 256));
    if (dtype == ALLOYB_BF16)
        launch_pdl(tc::residual_add_kernel<true>, grid, dim3(256), 0, st, static_cast<uint16_t*>(y),
                   static_cast<const uint16_t*>(residual), M, N, ldy);
    else
        launch_pdl(tc::residual_add_kernel<false>, grid, dim3(256), 0, st, static_cast<uint16_t*>(y),
                   static_cast<const uint16_t*>(residual), M, N, ldy);
    return check_launch();
}

// C = X * deq(W)^T (+ residual) for one packed matrix, or act(X G^T) * (X U^T) for a gate/up pair
// (`up` non-null; both matrices in seg's format and shape, M <= 128).  NOT_TAKEN unless the shape and
// the alignment are the kind the kernel is built for.
int try_gemm_tc(const void* x, int M, int K, int dtype, const WeightSeg& seg, const void* residual, const void* up,
                const void* up_scales, int act, cudaStream_t st, const WeightSeg* tail) {
    using namespace tc;
    if (dtype != ALLOYB_F16 && dtype != ALLOYB_BF16) return ALLOYB_NOT_TAKEN;
    if (seg.format != ALLOYB_Q4_K && seg.format != ALLOYB_Q6_K && seg.format != ALLOYB_Q8_0) return ALLOYB_NOT_TAKEN;
    if (M < GEMM_TC_MIN_M || K % QK_K) return ALLOYB_NOT_TAKEN;
    if (up && M > SPLIT_MAX_BM) return ALLOYB_NOT_TAKEN;
    const bool q8 = seg.format == ALLOYB_Q8_0;
    if (q8 && (!seg.scales || reinterpret_cast<uintptr_t>(seg.scales) % 16 || seg.row_bytes != K)) return ALLOYB_NOT_TAKEN;
    if (q8 && up && (!up_scales || reinterpret_cast<uintptr_t>(up_scales) % 16)) return ALLOYB_NOT_TAKEN;
    if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(seg.data) % 16 || seg.row_bytes % 16 ||
        reinterpret_cast<uintptr_t>(up) % 16)
        return ALLOYB_NOT_TAKEN;

    const EncodeFn encode = encoder();
    if (!encode) return ALLOYB_E_CUDA;
    int dev = 0;
    const int sms = sm_count_of_device(dev);
    if (!sms) { set_cuda_error(cudaErrorInvalidValue); return ALLOYB_E_CUDA; }

    const int BM = M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256));
    // `tail`: a second matrix of the same format whose rows follow seg's in memory (the caller has checked
    // that, and that seg.N is a whole number of row tiles); no residual, no gate/up pair, not Q8_0
    if (tail && (residual || up || q8 || seg.N % BN)) return ALLOYB_NOT_TAKEN;
    const int n_rows = seg.N + (tail ? tail->N : 0);
    const int tiles_n = (n_rows + BN - 1) / BN, tiles_m = (M + BM - 1) / BM, nsb = K / QK_K;
    // too few row tiles for the SMs and one token tile: split K (the sums live in a fixed scratch)
    int splits = 1;
    if (tiles_m == 1 && BM <= SPLIT_MAX_BM && tiles_n <= SPLIT_MAX_TILES && 2 * tiles_n <= sms) {
        splits = sms / tiles_n;
        if (splits > nsb) splits = nsb;
    }

    Maps maps;
    bool ok = map2d(encode, &maps.x, dtype == ALLOYB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                    x, K, M, static_cast<uint64_t>(K) * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    // the packed rows as bytes: one box = one super-block of 128 rows
    const void* mats[2] = {seg.data, up ? up : seg.data};
    const void* scs[2] = {seg.scales, up ? up_scales : seg.scales};
    for (int i = 0; i < 2 && ok; ++i) {
        if (q8) {
            ok = map2d(encode, &maps.w[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, mats[i], K, seg.N, seg.row_bytes, 128,
                       PACK_BOX_ROWS, CU_TENSOR_MAP_SWIZZLE_128B) &&
                 map2d(encode, &maps.s[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, scs[i], static_cast<uint64_t>(K / Q8_BLOCK) * 2,
                       seg.N, static_cast<uint64_t>(K / Q8_BLOCK) * 2, 16, PACK_BOX_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
        } else {
            ok = map2d(encode, &maps.w[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, mats[i], seg.row_bytes, n_rows, seg.row_bytes,
                       seg.format == ALLOYB_Q4_K ? Q4_ROW : Q6_ROW, PACK_BOX_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
            maps.s[i] = maps.w[i];
        }
    }
    if (!ok) {
        set_cuda_error(cudaErrorInvalidValue);
        return ALLOYB_E_CUDA;
    }
    Params P;
    P.format = seg.format;
    P.y = seg.y;
    const bool add_after = residual && M > GEMM_FUSED_RESIDUAL_MAX_M;
    P.residual = add_after ? nullptr : residual;
    P.ldy = seg.ldy;
    P.M = M;
    P.N = n_rows;
    P.n_split = tail ? seg.N : INT_MAX;
    P.y2 = tail ? tail->y : nullptr;
    P.ldy2 = tail ? tail->ldy : 0;
    P.K = K;
    P.splits = splits;
    P.gated = up ? 1 : 0;
    P.act = act;

    // persistent: one CTA per SM walks the items (weight-row tile fastest, so neighbours share a token tile)
    const int n_items = tiles_n * tiles_m * splits;
    const int grid = n_items < sms ? n_items : sms;
    const int rc = dtype == ALLOYB_BF16 ? launch_bm<true>(BM, maps, P, grid, dev, st) : launch_bm<false>(BM, maps, P, grid, dev, st);
    if (rc != ALLOYB_OK || !add_after) return rc;
    return gemm_tc_residual_add(seg.y, residual, M, seg.N, seg.ldy, dtype, st);
}

}  // namespace alloyb

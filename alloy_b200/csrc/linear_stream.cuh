// Building blocks of the one-token streaming dequant-GEMV (fp16 activations, Q4_K / Q6_K weights):
// slot geometries, the parameter block, the row cursor, PTX helpers and the per-super-block
// arithmetic.  Used by the stand-alone streaming kernel (linear_stream.cu) and by the decode-layer
// kernel (decode_layer.cu), which runs the same phases back to back inside one launch.
#pragma once
#include <cuda.h>

#include <type_traits>

#include "linear.cuh"
#include "linear_rows.cuh"

namespace alloyb {
namespace st {

constexpr int WARPS = 16;                    // warps per CTA
// Warps per group (= K slices per tile) is a kernel template parameter GW: 8 when an SM owns few
// tiles (the K split is what keeps all its warps busy; 16 when it owns one or three, so that no
// group is a tile short; 4 for rows of only 4-7 super-blocks), 1 when it owns at least two tiles
// per warp (every warp then runs whole tiles on its own, with no reduction and no barrier at all).
constexpr int MAX_D = 4;                     // ring slots per warp (upper bound)
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int MAX_SEG = MAX_SEGS;
constexpr int MAX_DEVICES = 64;

// Slot geometries.  A slot holds 16 rows of one stage; its row pitch is chosen so that the lanes'
// shared-memory reads fall on 32 different banks.
//   Q4x1: one 144-byte Q4_K super-block per row; pitch 144 (16 mod 32 bytes: 128-bit reads of two
//         rows x four lanes are conflict-free).
//   Q4x2: two super-blocks per row; pitch 288 + 16 spare bytes (again 16 mod 32).
//   Q6:   one 210-byte Q6_K super-block per row.  Blocks are only 2-byte aligned, copies need 16:
//         the slot row is the 16-byte-aligned window [floor16(210 sb), +240) and the block sits
//         at offset (210 sb) mod 16 inside it; pitch 240 = 60 words (28 mod 32: 32-bit reads of
//         eight rows x four lanes are conflict-free).
//   QMIX: Q4_K matrices (as Q4x2) followed by Q6_K matrices in one launch (q/k and v of a decode step);
//         a slot is as large as the larger of the two, every tile uses its own format's geometry.
enum Kind { Q4x1 = 0, Q4x2 = 1, Q6 = 2, QMIX = 3 };
template <int KIND> struct Geom;
template <> struct Geom<Q4x1> { static constexpr int SBS = 1, PITCH = 144, BLK = Q4K_BYTES; };
template <> struct Geom<Q4x2> { static constexpr int SBS = 2, PITCH = 304, BLK = Q4K_BYTES; };
template <> struct Geom<Q6> { static constexpr int SBS = 1, PITCH = 240, BLK = Q6K_BYTES; };
template <> struct Geom<QMIX> { static constexpr int SBS = 2, PITCH = 304, BLK = Q4K_BYTES; };
// What a Q6_K row costs next to a Q4_K row (instructions and bytes) when a mixed launch shares its rows out.
constexpr int Q6_ROW_COST = 2;

static __device__ int g_error = 0;           // sticky: a bounded wait ran out (one word per translation unit)

// Row-parallel (K-sharded) linear with the all-reduce inside the launch.  Every rank owns an
// exchange buffer that all ranks have mapped (peer[r] = rank r's buffer as seen from here):
//   +0     uint32 epoch (local), +4 uint32 finished-CTA counter (local)
//   +256   uint32 flags[8 ranks][256 CTAs]: rank r's CTA c has delivered its rows for epoch >= value
//   +8448  float  slots[2 sets][8 ranks][max_n]: the partial outputs, set = epoch parity
struct TpArgs {
    int world, rank, max_n;
    uint32_t spin;                           // polls of a peer's flag before the wait gives up
    uint8_t* peer[8];
};
constexpr int TP_FLAGS_OFF = 256, TP_SLOTS_OFF = 8448;

struct Seg {
    const uint8_t* data;
    int64_t row_bytes;
    void* y;
    int n_rows;
    int row_base;                            // first row of this matrix in the launch's stacked row space
    int q6;                                  // mixed launches: 1 = Q6_K rows (stacked space in cost units)
};
struct Params {
    const __half* x;
    const __half* residual;
    const __half* norm_w;                    // non-null: RMSNorm(x; norm_w, eps) is applied on the way in
    float eps;
    Seg seg[MAX_SEG];
    int n_seg;                               // matrices walked row-wise (1 for a gate/up pair)
    int total_rows;
    int nsb;
    int gated;                               // seg[0] = gate, seg[1] = up, y = act(gate) * up
    int act;
    int depth;                               // ring slots per warp
    TpArgs tp;                               // world == 0: plain linear
};
struct Maps {
    CUtensorMap m[MAX_SEG];                  // (row_bytes / 4, n_rows) uint32, box PITCH/4 x 16
};

// Position in a CTA's row range: matrix, local row, local end of the range inside that matrix.
struct Cursor {
    int seg, row, lim;
};
// COST: the stacked space counts a Q6_K row Q6_ROW_COST times (mixed launches); a row belongs to the range
// its first unit falls into.
template <bool COST = false>
__device__ __forceinline__ void cursor_enter(Cursor& c, const Params& P, int lo, int hi) {
    while (c.seg < P.n_seg) {
        const int base = P.seg[c.seg].row_base, n = P.seg[c.seg].n_rows;
        int a = lo > base ? lo - base : 0;
        int b = hi - base;
        if (COST && P.seg[c.seg].q6) {
            a = (a + Q6_ROW_COST - 1) / Q6_ROW_COST;
            b = b > 0 ? (b + Q6_ROW_COST - 1) / Q6_ROW_COST : 0;
        }
        if (b > n) b = n;
        if (a < b) {
            c.row = a;
            c.lim = b;
            return;
        }
        ++c.seg;
    }
}
template <bool COST = false>
__device__ __forceinline__ void cursor_next(Cursor& c, const Params& P, int lo, int hi, int steps) {
    for (int i = 0; i < steps && c.seg < P.n_seg; ++i) {
        c.row += 16;
        if (c.row >= c.lim) {
            ++c.seg;
            cursor_enter<COST>(c, P, lo, hi);
        }
    }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 32) __nanosleep(32);
    }
    atomicExch(&g_error, 1);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
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
// 32 bits at a shared address that is 4-byte aligned (AL) or 2 bytes past a 4-byte boundary.
template <bool AL> __device__ __forceinline__ uint32_t lds32_u(uint32_t addr) {
    if (AL) return lds32(addr);
    return __funnelshift_r(lds32(addr - 2u), lds32(addr + 2u), 16);
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mma_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("{\n\t.reg .f32 z;\n\tmov.f32 z, 0f00000000;\n\t"
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {z,z,z,z};\n\t}"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// B fragments of one super-block of the token: lane (g, t) holds sub-block g's 32 activations when
// it owns that sub-block's k slots (g >> 1 == t), zero otherwise; sx = per-sub-block sums (columns
// 2t, 2t+1) from eight MMAs with A = 1.
struct XFrag {
    uint32_t b[8][2];
    float sx0, sx1;
};
__device__ __forceinline__ void load_xfrag(XFrag& f, const __half* x, int sb, int g, int t) {
#pragma unroll
    for (int j = 0; j < 8; ++j) f.b[j][0] = f.b[j][1] = 0u;
    if ((g >> 1) == t) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + sb * QK_K + 32 * g);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = xp[q];
            f.b[2 * q][0] = prmt(v.x, v.y, 0x5410u);          // (x[4j], x[4j+2])
            f.b[2 * q][1] = prmt(v.x, v.y, 0x7632u);          // (x[4j+1], x[4j+3])
            f.b[2 * q + 1][0] = prmt(v.z, v.w, 0x5410u);
            f.b[2 * q + 1][1] = prmt(v.z, v.w, 0x7632u);
        }
    }
    constexpr uint32_t ONE2 = 0x3C003C00u;
    float s[4];
    mma_zero(s, ONE2, ONE2, ONE2, ONE2, f.b[0][0], f.b[0][1]);
#pragma unroll
    for (int j = 1; j < 8; ++j) mma_acc(s, ONE2, ONE2, ONE2, ONE2, f.b[j][0], f.b[j][1]);
    f.sx0 = s[0];
    f.sx1 = s[1];
}

// Lane-invariant constants of the 6-bit scale decode (sub-blocks 2t, 2t+1 of rows g and g+8 at once).
struct ScaleSel {
    uint32_t sel;        // PRMT selector: bytes 2(t&1), 2(t&1)+1 of row g | the same of row g+8
    uint32_t m_a, m_b;   // t < 2: 0x3f3f3f3f, 0;  t >= 2: 0x0f0f0f0f, 0x30303030
    bool high;           // t >= 2
};
__device__ __forceinline__ ScaleSel make_scale_sel(int t) {
    ScaleSel s;
    const uint32_t b = 2u * (t & 1);
    s.sel = b | ((b + 1u) << 4) | ((b + 4u) << 8) | ((b + 5u) << 12);
    s.high = t >= 2;
    s.m_a = s.high ? 0x0f0f0f0fu : 0x3f3f3f3fu;
    s.m_b = s.high ? 0x30303030u : 0u;
    return s;
}

// One super-block of 16 rows at `blk` (row pitch PITCH): adds this lane's share of rows g and g+8.
template <int PITCH>
__device__ __forceinline__ void unit_q4k(uint32_t blk, const XFrag& f, const ScaleSel& ss, int g, int t, float& a0,
                                         float& a1) {
    const uint32_t rb = blk + g * PITCH;
    const uint4 p0 = lds128(rb + 16 + 32 * t), p1 = lds128(rb + 32 + 32 * t);
    const uint4 r0 = lds128(rb + 8 * PITCH + 16 + 32 * t), r1 = lds128(rb + 8 * PITCH + 32 + 32 * t);
    const uint4 h0 = lds128(rb), h1 = lds128(rb + 8 * PITCH);
    const uint32_t wg[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    const uint32_t wh[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    float clo[4], chi[4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t ug = wg[j] >> 8, uh = wh[j] >> 8;
        if (j == 0) {
            mma_zero(clo, wg[j] & 0x000f000fu, wh[j] & 0x000f000fu, ug & 0x000f000fu, uh & 0x000f000fu, f.b[j][0],
                     f.b[j][1]);
            mma_zero(chi, wg[j] & 0x00f000f0u, wh[j] & 0x00f000f0u, ug & 0x00f000f0u, uh & 0x00f000f0u, f.b[j][0],
                     f.b[j][1]);
        } else {
            mma_acc(clo, wg[j] & 0x000f000fu, wh[j] & 0x000f000fu, ug & 0x000f000fu, uh & 0x000f000fu, f.b[j][0],
                    f.b[j][1]);
            mma_acc(chi, wg[j] & 0x00f000f0u, wh[j] & 0x00f000f0u, ug & 0x00f000f0u, uh & 0x00f000f0u, f.b[j][0],
                    f.b[j][1]);
        }
    }
    // 6-bit scales / mins (llama.cpp's get_scale_min_k4) of both rows in one register each:
    // bytes = {row g: 2t, 2t+1; row g+8: 2t, 2t+1}
    const uint32_t Y = prmt(h0.y, h1.y, ss.sel), Z = prmt(h0.z, h1.z, ss.sel), Wd = prmt(h0.w, h1.w, ss.sel);
    const uint32_t sc4 = ((ss.high ? Wd : Y) & ss.m_a) | ((Y >> 2) & ss.m_b);
    const uint32_t mn4 = ((ss.high ? (Wd >> 4) : Z) & ss.m_a) | ((Z >> 2) & ss.m_b);
    const float2 dm0 = __half22float2(*reinterpret_cast<const __half2*>(&h0.x));
    const float2 dm1 = __half22float2(*reinterpret_cast<const __half2*>(&h1.x));
    // low nibbles entered as n * 2^-24, high ones as 16 n * 2^-24
    float a = static_cast<float>(sc4 & 0xffu) * clo[0];
    a = fmaf(static_cast<float>((sc4 >> 8) & 0xffu) * 0.0625f, chi[1], a);
    float m = static_cast<float>(mn4 & 0xffu) * f.sx0;
    m = fmaf(static_cast<float>((mn4 >> 8) & 0xffu), f.sx1, m);
    a0 = fmaf(dm0.x * 16777216.0f, a, fmaf(-dm0.y, m, a0));
    float b = static_cast<float>((sc4 >> 16) & 0xffu) * clo[2];
    b = fmaf(static_cast<float>(sc4 >> 24) * 0.0625f, chi[3], b);
    float n = static_cast<float>((mn4 >> 16) & 0xffu) * f.sx0;
    n = fmaf(static_cast<float>(mn4 >> 24), f.sx1, n);
    a1 = fmaf(dm1.x * 16777216.0f, b, fmaf(-dm1.y, n, a1));
}

// ---- Q6_K ------------------------------------------------------------------------------------
// A Q6_K super-block has 16 sub-blocks of 16 weights (int8 scale each), in two halves of 128.
// Within a half, ql byte l (l < 32) holds codes l (low nibble, "plane" 0) and l + 64 (high nibble,
// plane 2), ql byte 32 + l holds l + 32 (plane 1) and l + 96 (plane 3), qh byte l holds the four
// codes' bits 4-5; sub-block 2p + i of the half is plane p, l in [16 i, 16 i + 16).
//
// MMA mapping for one token: the eight columns are the eight sub-blocks of a half.  MMA (p, i)
// covers sub-block 2p + i: lane t supplies l = 16 i + 4t + {0, 2 | 1, 3} (bytes 0, 2 and 1, 3 of
// one 32-bit word per row), so lane (g, t) of the B operand holds x[128 h + 16 g + 4t ..+3] --
// each lane its own four activations -- for the MMA with 2p + i == g and zero for the other
// seven.  Codes enter as fp16 bit patterns: planes 0/1 as code * 2^-24, planes 2/3 as
// 16 code * 2^-24 (the high nibble stays in place, its two high bits go to bits 8-9); the -32
// offset is applied through the per-sub-block activation sums (one MMA with A = 1 per half).
struct XFrag6 {
    uint32_t b[2][2];        // [half][k slots (0, 2) | (1, 3)]
    float sx[2][2];          // [half][sub-block 2t, 2t+1 of the half]
};
// The lane's eight activations of super-block sb as loaded (two 8-byte loads), and the fragments from them:
// the loads are issued a super-block ahead of their use.
__device__ __forceinline__ void load_xraw6(uint2 (&r)[2], const __half* x, int sb, int g, int t) {
#pragma unroll
    for (int h = 0; h < 2; ++h) r[h] = *reinterpret_cast<const uint2*>(x + sb * QK_K + 128 * h + 16 * g + 4 * t);
}
__device__ __forceinline__ void build_xfrag6(XFrag6& f, const uint2 (&r)[2]) {
    constexpr uint32_t ONE2 = 0x3C003C00u;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint2 v = r[h];
        f.b[h][0] = prmt(v.x, v.y, 0x5410u);
        f.b[h][1] = prmt(v.x, v.y, 0x7632u);
        float s[4];
        mma_zero(s, ONE2, ONE2, ONE2, ONE2, f.b[h][0], f.b[h][1]);
        f.sx[h][0] = s[0];
        f.sx[h][1] = s[1];
    }
}
__device__ __forceinline__ void load_xfrag6(XFrag6& f, const __half* x, int sb, int g, int t) {
    uint2 r[2];
    load_xraw6(r, x, sb, g, t);
    build_xfrag6(f, r);
}

// One super-block of 16 rows; `blk` = slot + the block's offset inside the aligned window.
template <bool AL>
__device__ __forceinline__ void unit_q6k(uint32_t blk, const XFrag6& f, int g, int t, float& a0, float& a1) {
    constexpr int PITCH = Geom<Q6>::PITCH;
    const uint32_t rb = blk + g * PITCH + 4 * t;
    const float fscale = t >= 2 ? 1048576.0f : 16777216.0f;          // planes 2, 3 carry a factor 16
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float c[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t qa[2], qb[2], qh[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const uint32_t r = rb + rr * 8 * PITCH + 16 * i;
                qa[rr] = lds32_u<AL>(r + 64 * h);
                qb[rr] = lds32_u<AL>(r + 64 * h + 32);
                qh[rr] = lds32_u<AL>(r + 128 + 32 * h);
            }
            uint32_t A[4][4];                                          // [plane][a0..a3]
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const uint32_t qa8 = qa[rr] >> 8, qb8 = qb[rr] >> 8;
                const uint32_t u0 = qh[rr] << 4, v0 = qh[rr] << 2, u1 = qh[rr] >> 4, v1 = qh[rr] >> 6;
                A[0][rr] = (qa[rr] & 0x000f000fu) | (u0 & 0x00300030u);
                A[0][rr + 2] = (qa8 & 0x000f000fu) | (u1 & 0x00300030u);
                A[1][rr] = (qb[rr] & 0x000f000fu) | (v0 & 0x00300030u);
                A[1][rr + 2] = (qb8 & 0x000f000fu) | (v1 & 0x00300030u);
                A[2][rr] = (qa[rr] & 0x00f000f0u) | (u0 & 0x03000300u);
                A[2][rr + 2] = (qa8 & 0x00f000f0u) | (u1 & 0x03000300u);
                A[3][rr] = (qb[rr] & 0x00f000f0u) | (v0 & 0x03000300u);
                A[3][rr + 2] = (qb8 & 0x00f000f0u) | (v1 & 0x03000300u);
            }
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const bool mine = g == 2 * p + i;
                const uint32_t b0 = mine ? f.b[h][0] : 0u, b1 = mine ? f.b[h][1] : 0u;
                if (i == 0 && p == 0) mma_zero(c, A[p][0], A[p][1], A[p][2], A[p][3], b0, b1);
                else mma_acc(c, A[p][0], A[p][1], A[p][2], A[p][3], b0, b1);
            }
        }
        // int8 scales of sub-blocks 8h + 2t, 8h + 2t + 1 and the block scale, rows g and g+8
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const uint32_t base = blk + (g + 8 * rr) * PITCH;
            const uint32_t s2 = lds16(base + 192 + 8 * h + 2 * t);
            const float d = half_bits_to_f32(lds16(base + 208));
            const float s0 = static_cast<float>(static_cast<int8_t>(s2 & 0xffu));
            const float s1 = static_cast<float>(static_cast<int8_t>(s2 >> 8));
            const float e0 = fmaf(c[2 * rr], fscale, -32.0f * f.sx[h][0]);
            const float e1 = fmaf(c[2 * rr + 1], fscale, -32.0f * f.sx[h][1]);
            const float v = fmaf(s1, e1, s0 * e0);
            if (rr == 0) a0 = fmaf(d, v, a0);
            else a1 = fmaf(d, v, a1);
        }
    }
}

}  // namespace st
}  // namespace alloyb

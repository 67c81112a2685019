// Dequant-GEMV / skinny GEMM for 2..128 tokens (32 per pass) and for the one-token shapes the
// persistent streaming kernel (linear_stream.cu) does not take (bf16, K not a multiple of 1024).
//
// Why tensor cores on a memory-bound op: at HBM speed a B200 streams ~11.5e12
// Q4_K weights per second but issues only ~1.1e12 warp instructions per second,
// so a kernel may spend at most ~3 thread-instructions per weight.  Converting a
// nibble to float and multiplying it on the CUDA cores costs about that per
// weight per token, which caps a CUDA-core GEMV near half of the HBM roofline at
// M = 1 and far below it for M >= 4.  Here the CUDA cores only unpack bits; the
// multiply-adds run as mma.sync.m16n8k16 with the 16 weight rows as the M
// dimension and up to 8 tokens as N.
//
// Exactness: the A operand holds the raw quants (nibble, or q6-32) which are
// exact in fp16/bf16; the products with the fp16/bf16 activations are exact in
// fp32 and are accumulated in fp32; the per-sub-block scale d*sc (exact in
// fp32) multiplies the sub-block's sum afterwards.  That is the factored form
// sum_g d*sc_g * (sum_k nib*x) - dmin*m_g * (sum_k x) the reference's GEMV uses
// (metal/std/quant.py:1312-1347), not an fp16 dequantisation of the weights.
//
// Data movement: a CTA owns 16 (or 2x16 for gate/up) weight rows and walks K in
// chunks of 8 super-blocks.  A producer warp copies each row's chunk with
// cp.async.bulk into a ring of shared-memory stages guarded by mbarriers; eight
// consumer warps take one super-block each of a chunk.  Weight copies do not depend on
// the previous kernel, so they are issued BEFORE griddepcontrol.wait: with
// programmatic dependent launch the next layer's weights are already in flight
// while the previous kernel drains.
#include <type_traits>

#include "kv.cuh"
#include "linear.cuh"
#include "linear_rows.cuh"

namespace alloyb {

constexpr int MMA_CONSUMERS = 8;                 // consumer warps per CTA (one super-block each per stage)
constexpr int MMA_THREADS = (MMA_CONSUMERS + 1) * 32;
constexpr int MMA_CH = 8;                        // super-blocks per stage
constexpr int MMA_STAGES = 4;                    // ring depth upper bound (barrier slots)
constexpr int MMA_SMEM_TARGET = 72 * 1024;       // keeps three CTAs resident per SM
constexpr int Q4_CHUNK = MMA_CH * Q4K_BYTES;     // 1152
constexpr int Q6_CHUNK = MMA_CH * Q6K_BYTES;     // 1680
constexpr int Q4_STRIDE = Q4_CHUNK + 32;         // words/row = 8 mod 32: conflict-free 64-bit reads
constexpr int Q6_STRIDE = Q6_CHUNK;              // words/row = 4 mod 32: conflict-free 32-bit reads
constexpr int Q4_STRIDE_SB = Q4_CHUNK + 16;      // one-token path: 16 mod 128 bytes, conflict-free 128-bit reads
constexpr uint32_t SPIN_LIMIT = 1u << 22;

__device__ int g_device_error = 0;               // sticky; read by alloyb_device_error()

struct MmaSeg {
    int format;
    int n_rows;
    const uint8_t* data;
    int64_t row_bytes;
    void* y;
    int64_t ldy;
    int tile0;            // index of this matrix's first 16-row tile in the grid
};

struct MmaParams {
    const void* x;
    int M;
    int K;
    MmaSeg seg[MAX_SEGS];
    int n_seg;
    const void* residual;
    int gated;            // 1: seg[0] = gate, seg[1] = up, y = act(gate) * up into seg[0].y
    int act;
    int stage_bytes;
    int n_stages;         // ring depth actually used (<= MMA_STAGES)
};

// ------------------------------------------------------------------------------- PTX helpers

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false (and the sticky device error set) if the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    atomicExch(&g_device_error, 1);
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(MMA_CONSUMERS * 32) : "memory");
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
// 32 bits at a 2-byte-aligned shared address.
__device__ __forceinline__ uint32_t lds32_align2(uint32_t addr) {
    if (addr & 2u) {
        const uint32_t lo = lds32(addr - 2u), hi = lds32(addr + 2u);
        return __funnelshift_r(lo, hi, 16);
    }
    return lds32(addr);
}

template <typename XT>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                 uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4],
                                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Element-type constants of the A operand.
template <typename XT> struct QuantEnc;
template <> struct QuantEnc<__half> {
    static constexpr uint32_t ONE2 = 0x3C003C00u;      // (1.0, 1.0)
    static constexpr uint32_t MAGIC_BYTES = 0x64646464u;   // 0x64xx = 1024 + xx
    __device__ static __forceinline__ uint32_t sub(uint32_t v, float off) {
        const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&v), __float2half2_rn(off));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
    static constexpr float MAGIC_BASE = 1024.0f;
};
template <> struct QuantEnc<__nv_bfloat16> {
    static constexpr uint32_t ONE2 = 0x3F803F80u;
    static constexpr uint32_t MAGIC_BYTES = 0x43434343u;   // 0x43xx = 128 + xx (xx < 128)
    __device__ static __forceinline__ uint32_t sub(uint32_t v, float off) {
        const __nv_bfloat162 r =
            __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v), __float2bfloat162_rn(off));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
    static constexpr float MAGIC_BASE = 128.0f;
};

// ------------------------------------------------------------------------------- consumers

// Activation fragment loads: token column g of group nt, 4 or 8 consecutive elements.
template <typename XT>
__device__ __forceinline__ uint4 ldx8(const XT* x, int M, int K, int tok, int k) {
    if (tok < M) return __ldg(reinterpret_cast<const uint4*>(x + static_cast<int64_t>(tok) * K + k));
    return make_uint4(0u, 0u, 0u, 0u);
}
template <typename XT>
__device__ __forceinline__ uint2 ldx4(const XT* x, int M, int K, int tok, int k) {
    if (tok < M) return __ldg(reinterpret_cast<const uint2*>(x + static_cast<int64_t>(tok) * K + k));
    return make_uint2(0u, 0u);
}

// One Q4_K super-block for RT row tiles and NT token groups.
//   stage: shared address of the stage (rows rt*16.. at stride Q4_STRIDE), sb: block within the chunk
//   tbl:   this warp's scale table, RT*16 rows x 4 pairs x float4 {dsc_lo, dsc_hi, dm_lo, dm_hi}
template <typename XT, int RT, int NT, bool SUBNORMAL>
__device__ __forceinline__ void q4k_superblock(uint32_t stage, int sb, float4* tbl, const XT* x, int M,
                                               int K, int kbase, float (&acc)[RT][NT][4]) {
    using E = QuantEnc<XT>;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // ---- scale table: lane -> row (lane>>1), sub-block pairs 2*(lane&1), 2*(lane&1)+1
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
        const int r = rt * 16 + (lane >> 1);
        const uint4 hdr = lds128(stage + r * Q4_STRIDE + sb * Q4K_BYTES);
        const float d = half_bits_to_f32(hdr.x & 0xffffu);
        const float dmin = half_bits_to_f32(hdr.x >> 16);
        uint32_t scw, mw;
        if ((lane & 1) == 0) {
            scw = hdr.y & 0x3f3f3f3fu;
            mw = hdr.z & 0x3f3f3f3fu;
        } else {
            scw = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
            mw = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
        }
        // SUBNORMAL: low nibbles enter the MMA as n*2^-24, high nibbles as 16n*2^-24
        const float lo_mul = SUBNORMAL ? 16777216.0f : 1.0f;
        const float hi_mul = SUBNORMAL ? 1048576.0f : 1.0f;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            float4 e;
            e.x = d * static_cast<float>((scw >> (16 * p)) & 0xffu) * lo_mul;
            e.y = d * static_cast<float>((scw >> (16 * p + 8)) & 0xffu) * hi_mul;
            e.z = dmin * static_cast<float>((mw >> (16 * p)) & 0xffu);
            e.w = dmin * static_cast<float>((mw >> (16 * p + 8)) & 0xffu);
            tbl[r * 4 + (lane & 1) * 2 + p] = e;
        }
    }
    __syncwarp();

    const uint32_t ones[4] = {E::ONE2, E::ONE2, E::ONE2, E::ONE2};
#pragma unroll
    for (int gp = 0; gp < 4; ++gp) {
        // activations: sub-block 2gp (lo nibbles) and 2gp+1 (hi nibbles), 8 elements each per lane
        uint4 xl[NT], xh[NT];
        float sx_lo[NT][4], sx_hi[NT][4];
        const int k0 = kbase + gp * 64 + 8 * t;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            xl[nt] = ldx8<XT>(x, M, K, nt * 8 + g, k0);
            xh[nt] = ldx8<XT>(x, M, K, nt * 8 + g, k0 + 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) sx_lo[nt][i] = sx_hi[nt][i] = 0.f;
            mma16816<XT>(sx_lo[nt], ones, xl[nt].x, xl[nt].y);
            mma16816<XT>(sx_lo[nt], ones, xl[nt].z, xl[nt].w);
            mma16816<XT>(sx_hi[nt], ones, xh[nt].x, xh[nt].y);
            mma16816<XT>(sx_hi[nt], ones, xh[nt].z, xh[nt].w);
        }
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
            const uint32_t base = stage + sb * Q4K_BYTES + 16 + gp * 32 + 8 * t;
            const uint2 w0 = lds64(base + (rt * 16 + g) * Q4_STRIDE);
            const uint2 w1 = lds64(base + (rt * 16 + g + 8) * Q4_STRIDE);
            const float4 s0 = tbl[(rt * 16 + g) * 4 + gp];
            const float4 s1 = tbl[(rt * 16 + g + 8) * 4 + gp];
            uint32_t alo[2][4], ahi[2][4];     // [j][fragment register]
            const uint32_t ww[2][2] = {{w0.x, w1.x}, {w0.y, w1.y}};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {        // rr: row g / row g+8
                    const uint32_t w = ww[j][rr];
                    if (SUBNORMAL) {
                        const uint32_t p01 = prmt(w, 0u, 0x4140u), p23 = prmt(w, 0u, 0x4342u);
                        alo[j][rr] = p01 & 0x000f000fu;
                        alo[j][rr + 2] = p23 & 0x000f000fu;
                        ahi[j][rr] = p01 & 0x00f000f0u;
                        ahi[j][rr + 2] = p23 & 0x00f000f0u;
                    } else {
                        const uint32_t wl = w & 0x0f0f0f0fu, wh = (w >> 4) & 0x0f0f0f0fu;
                        alo[j][rr] = E::sub(prmt(wl, E::MAGIC_BYTES, 0x4140u), E::MAGIC_BASE);
                        alo[j][rr + 2] = E::sub(prmt(wl, E::MAGIC_BYTES, 0x4342u), E::MAGIC_BASE);
                        ahi[j][rr] = E::sub(prmt(wh, E::MAGIC_BYTES, 0x4140u), E::MAGIC_BASE);
                        ahi[j][rr + 2] = E::sub(prmt(wh, E::MAGIC_BYTES, 0x4342u), E::MAGIC_BASE);
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float cl[4] = {0.f, 0.f, 0.f, 0.f}, ch[4] = {0.f, 0.f, 0.f, 0.f};
                mma16816<XT>(cl, alo[0], xl[nt].x, xl[nt].y);
                mma16816<XT>(cl, alo[1], xl[nt].z, xl[nt].w);
                mma16816<XT>(ch, ahi[0], xh[nt].x, xh[nt].y);
                mma16816<XT>(ch, ahi[1], xh[nt].z, xh[nt].w);
                float* a = acc[rt][nt];
                a[0] += s0.x * cl[0] + s0.y * ch[0] - s0.z * sx_lo[nt][0] - s0.w * sx_hi[nt][0];
                a[1] += s0.x * cl[1] + s0.y * ch[1] - s0.z * sx_lo[nt][1] - s0.w * sx_hi[nt][1];
                a[2] += s1.x * cl[2] + s1.y * ch[2] - s1.z * sx_lo[nt][2] - s1.w * sx_hi[nt][2];
                a[3] += s1.x * cl[3] + s1.y * ch[3] - s1.z * sx_lo[nt][3] - s1.w * sx_hi[nt][3];
            }
        }
    }
    __syncwarp();
}

// fp16 MMA with the accumulator passed as separate registers, and with a zero accumulator.
__device__ __forceinline__ void mma_f16_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "{\n\t.reg .f32 z;\n\tmov.f32 z, 0f00000000;\n\t"
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{z,z,z,z};\n\t}"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One Q4_K super-block against ONE fp16 token, with the eight MMA columns used for the eight
// sub-blocks instead of for tokens.
//
// Lane (g, t) reads the 32 quant bytes of group t (sub-block 2t in the low nibbles, 2t+1 in the
// high ones) of rows g and g+8 with four 128-bit loads.  A 32-bit word gives four A registers with
// one shift and four ANDs: the nibbles of bytes (0, 2) and of bytes (1, 3), low ones as n*2^-24,
// high ones as 16n*2^-24 (fp16 subnormals, exact).  In the B operand column n carries the token's
// activations of sub-block n in the k slots of the lanes that own that sub-block and zero
// elsewhere, so that after the sixteen MMAs of a super-block C_lo[row][2t] and C_hi[row][2t+1] hold
// the per-sub-block sums  sum nib*x  (the other columns hold cross terms nobody reads).  The
// sub-block scales are then applied to eight numbers per lane instead of to every MMA's output,
// and  sum x  per sub-block comes from eight MMAs with A = 1 shared by all row tiles.
template <int RT>
__device__ __forceinline__ void q4k_superblock_sb(uint32_t stage, int sb, const __half* x, int kbase,
                                                  float (&acc)[RT][1][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    uint32_t xb[8][2];
#pragma unroll
    for (int j = 0; j < 8; ++j) xb[j][0] = xb[j][1] = 0u;
    if ((g >> 1) == t) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + kbase + 32 * g);   // sub-block g
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = __ldg(xp + q);
            xb[2 * q][0] = prmt(v.x, v.y, 0x5410u);          // (x[4j], x[4j+2])
            xb[2 * q][1] = prmt(v.x, v.y, 0x7632u);          // (x[4j+1], x[4j+3])
            xb[2 * q + 1][0] = prmt(v.z, v.w, 0x5410u);
            xb[2 * q + 1][1] = prmt(v.z, v.w, 0x7632u);
        }
    }
    constexpr uint32_t ONE2 = QuantEnc<__half>::ONE2;
    float sx[4];                                                              // sx[0], sx[1]: sub-blocks 2t, 2t+1
    mma_f16_zero(sx, ONE2, ONE2, ONE2, ONE2, xb[0][0], xb[0][1]);
#pragma unroll
    for (int j = 1; j < 8; ++j) mma_f16_acc(sx, ONE2, ONE2, ONE2, ONE2, xb[j][0], xb[j][1]);

    const int sh = 16 * (t & 1);
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
        const uint32_t rb = stage + (rt * 16 + g) * Q4_STRIDE_SB + sb * Q4K_BYTES;
        const uint4 h0 = lds128(rb), h1 = lds128(rb + 8 * Q4_STRIDE_SB);
        const uint4 p0 = lds128(rb + 16 + 32 * t), p1 = lds128(rb + 32 + 32 * t);
        const uint4 r0 = lds128(rb + 8 * Q4_STRIDE_SB + 16 + 32 * t), r1 = lds128(rb + 8 * Q4_STRIDE_SB + 32 + 32 * t);
        const uint32_t wg[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        const uint32_t wh[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        float clo[4], chi[4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t ug = wg[j] >> 8, uh = wh[j] >> 8;
            if (j == 0) {
                mma_f16_zero(clo, wg[j] & 0x000f000fu, wh[j] & 0x000f000fu, ug & 0x000f000fu, uh & 0x000f000fu,
                             xb[j][0], xb[j][1]);
                mma_f16_zero(chi, wg[j] & 0x00f000f0u, wh[j] & 0x00f000f0u, ug & 0x00f000f0u, uh & 0x00f000f0u,
                             xb[j][0], xb[j][1]);
            } else {
                mma_f16_acc(clo, wg[j] & 0x000f000fu, wh[j] & 0x000f000fu, ug & 0x000f000fu, uh & 0x000f000fu,
                            xb[j][0], xb[j][1]);
                mma_f16_acc(chi, wg[j] & 0x00f000f0u, wh[j] & 0x00f000f0u, ug & 0x00f000f0u, uh & 0x00f000f0u,
                            xb[j][0], xb[j][1]);
            }
        }
        // 6-bit scales and mins of sub-blocks 2t, 2t+1 (llama.cpp's get_scale_min_k4, two at a time)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const uint4 h = rr ? h1 : h0;
            const uint32_t wy = h.y >> sh, wz = h.z >> sh, ww = h.w >> sh;
            uint32_t scp, mp;
            if (t < 2) {
                scp = wy & 0x3f3fu;
                mp = wz & 0x3f3fu;
            } else {
                scp = (ww & 0x0f0fu) | ((wy >> 2) & 0x3030u);
                mp = ((ww >> 4) & 0x0f0fu) | ((wz >> 2) & 0x3030u);
            }
            const float d = half_bits_to_f32(h.x & 0xffffu) * 16777216.0f;     // undoes the 2^-24
            const float dmin = half_bits_to_f32(h.x >> 16);
            const float c_lo = clo[2 * rr], c_hi = chi[2 * rr + 1] * 0.0625f;
            float a = static_cast<float>(scp & 0xffu) * c_lo;
            a = fmaf(static_cast<float>(scp >> 8), c_hi, a);
            float m = static_cast<float>(mp & 0xffu) * sx[0];
            m = fmaf(static_cast<float>(mp >> 8), sx[1], m);
            acc[rt][0][2 * rr] = fmaf(d, a, fmaf(-dmin, m, acc[rt][0][2 * rr]));
        }
    }
}

// One Q6_K super-block.  tbl: RT*16 rows x 16 floats d*sc, stored [row][h][lhalf][j].
template <typename XT, int RT, int NT>
__device__ __forceinline__ void q6k_superblock(uint32_t stage, int sb, float4* tbl, const XT* x, int M,
                                               int K, int kbase, float (&acc)[RT][NT][4]) {
    using E = QuantEnc<XT>;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
        const int r = rt * 16 + (lane >> 1), h = lane & 1;
        const uint32_t blk = stage + r * Q6_STRIDE + sb * Q6K_BYTES;
        const float d = half_bits_to_f32(lds16(blk + 208));
        float s[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t two = lds16(blk + 192 + h * 8 + 2 * i);
            s[2 * i] = d * static_cast<float>(static_cast<int8_t>(two & 0xffu));
            s[2 * i + 1] = d * static_cast<float>(static_cast<int8_t>(two >> 8));
        }
        // scale index i = 2j + lhalf  ->  [h][lhalf][j]
        tbl[r * 4 + h * 2 + 0] = make_float4(s[0], s[2], s[4], s[6]);
        tbl[r * 4 + h * 2 + 1] = make_float4(s[1], s[3], s[5], s[7]);
    }
    __syncwarp();

    const float off = E::MAGIC_BASE + 32.0f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int lh = 0; lh < 2; ++lh) {
            uint2 xv[NT][4];
            const int k0 = kbase + h * 128 + lh * 16 + 4 * t;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) xv[nt][j] = ldx4<XT>(x, M, K, nt * 8 + g, k0 + j * 32);
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
                uint32_t a[4][4];                 // [j][fragment register]
                float4 sc[2];
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int r = rt * 16 + g + 8 * rr;
                    const uint32_t blk = stage + r * Q6_STRIDE + sb * Q6K_BYTES;
                    const uint32_t qla = lds32_align2(blk + h * 64 + lh * 16 + 4 * t);
                    const uint32_t qlb = lds32_align2(blk + h * 64 + 32 + lh * 16 + 4 * t);
                    const uint32_t qh = lds32_align2(blk + 128 + h * 32 + lh * 16 + 4 * t);
                    sc[rr] = tbl[r * 4 + h * 2 + lh];
                    uint32_t q[4];
                    q[0] = (qla & 0x0f0f0f0fu) | ((qh << 4) & 0x30303030u);
                    q[1] = (qlb & 0x0f0f0f0fu) | ((qh << 2) & 0x30303030u);
                    q[2] = ((qla >> 4) & 0x0f0f0f0fu) | (qh & 0x30303030u);
                    q[3] = ((qlb >> 4) & 0x0f0f0f0fu) | ((qh >> 2) & 0x30303030u);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        a[j][rr] = E::sub(prmt(q[j], E::MAGIC_BYTES, 0x4140u), off);
                        a[j][rr + 2] = E::sub(prmt(q[j], E::MAGIC_BYTES, 0x4342u), off);
                    }
                }
                const float s0[4] = {sc[0].x, sc[0].y, sc[0].z, sc[0].w};
                const float s1[4] = {sc[1].x, sc[1].y, sc[1].z, sc[1].w};
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
                        mma16816<XT>(c, a[j], xv[nt][j].x, xv[nt][j].y);
                        float* o = acc[rt][nt];
                        o[0] = fmaf(s0[j], c[0], o[0]);
                        o[1] = fmaf(s0[j], c[1], o[1]);
                        o[2] = fmaf(s1[j], c[2], o[2]);
                        o[3] = fmaf(s1[j], c[3], o[3]);
                    }
                }
            }
        }
    }
    __syncwarp();
}

// ------------------------------------------------------------------------------- kernel

struct SmemHeader {
    uint64_t full[MMA_STAGES];
    uint64_t empty[MMA_STAGES];
};

// Two CTAs per SM (nine warps each) wherever the accumulators leave the registers for it: with one, the
// warps wait on their activation loads with nobody to run meanwhile.  A gate/up pair with three or four
// token groups would spill under that limit and keeps the SM to itself.
template <typename XT, int RT, int NT, bool SB>
__global__ void __launch_bounds__(MMA_THREADS, (RT == 2 && NT >= 3) ? 1 : 2) linear_mma_kernel(const MmaParams P) {
    static_assert(!SB || (std::is_same<XT, __half>::value && NT == 1), "one-token path: fp16, one token group");
    extern __shared__ __align__(128) uint8_t smem[];
    SmemHeader* hdr = reinterpret_cast<SmemHeader*>(smem);
    float4* tbl_all = reinterpret_cast<float4*>(smem + 128);              // per consumer warp: RT KB
    float* red = reinterpret_cast<float*>(smem + 128 + MMA_CONSUMERS * RT * 1024);
    uint8_t* stages = smem + 128 + MMA_CONSUMERS * RT * 1024 + MMA_CONSUMERS * RT * 16 * 8 * NT * 4;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // which matrix / tile
    int si = 0;
    if (!P.gated) {
        while (si + 1 < P.n_seg && static_cast<int>(blockIdx.x) >= P.seg[si + 1].tile0) ++si;
    }
    const MmaSeg& sg = P.seg[si];
    const int tile = blockIdx.x - sg.tile0;
    const int row0 = tile * 16;
    const int fmt = sg.format;
    const int nsb = P.K / QK_K;
    const int nchunks = (nsb + MMA_CH - 1) / MMA_CH;
    const int blk_bytes = (fmt == ALLOYB_Q4_K) ? Q4K_BYTES : Q6K_BYTES;
    const int stride = (fmt == ALLOYB_Q4_K) ? (SB ? Q4_STRIDE_SB : Q4_STRIDE) : Q6_STRIDE;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P.n_stages; ++s) {
            mbar_init(&hdr->full[s], 1);
            mbar_init(&hdr->empty[s], MMA_CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == MMA_CONSUMERS) {
        // ---------------- producer: one row per lane (RT*16 rows), weights only -> no pdl_wait
        bool ok = true;
        for (int c = 0; c < nchunks && ok; ++c) {
            const int s = c % P.n_stages;
            if (c >= P.n_stages) ok = mbar_wait(&hdr->empty[s], ((c / P.n_stages) - 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const int sb_n = min(MMA_CH, nsb - c * MMA_CH);
            const uint32_t bytes = (static_cast<uint32_t>(sb_n * blk_bytes) + 15u) & ~15u;
            if (lane == 0) mbar_arrive_expect_tx(&hdr->full[s], bytes * RT * 16);
            __syncwarp();
            uint8_t* dst_stage = stages + static_cast<size_t>(s) * P.stage_bytes;
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
                if (lane < 16) {
                    const MmaSeg& src = P.gated ? P.seg[rt] : sg;
                    int r = row0 + lane;
                    if (r >= src.n_rows) r = src.n_rows - 1;      // tail tile: re-read the last row
                    const uint8_t* gp = src.data + static_cast<int64_t>(r) * src.row_bytes +
                                        static_cast<int64_t>(c) * MMA_CH * blk_bytes;
                    bulk_g2s(dst_stage + (rt * 16 + lane) * stride, gp, bytes, &hdr->full[s]);
                }
            }
        }
        return;
    }

    // ---------------- consumers
    float acc[RT][NT][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[rt][nt][i] = 0.f;
    float4* tbl = tbl_all + warp * RT * 64;
    const XT* x = static_cast<const XT*>(P.x);

    pdl_wait();      // activations (and the output buffer) belong to the previous kernel until here

    bool ok = true;
    for (int c = 0; c < nchunks; ++c) {
        const int s = c % P.n_stages;
        ok = mbar_wait(&hdr->full[s], (c / P.n_stages) & 1);
        if (!ok) break;
        const uint32_t stage = smem_u32(stages + static_cast<size_t>(s) * P.stage_bytes);
        const int sb_n = min(MMA_CH, nsb - c * MMA_CH);
        for (int sb = warp; sb < sb_n; sb += MMA_CONSUMERS) {
            const int kbase = (c * MMA_CH + sb) * QK_K;
            if (fmt == ALLOYB_Q4_K) {
                if constexpr (SB)
                    q4k_superblock_sb<RT>(stage, sb, x, kbase, acc);
                else if (!std::is_same<XT, __half>::value)
                    q4k_superblock<XT, RT, NT, false>(stage, sb, tbl, x, P.M, P.K, kbase, acc);
                else
                    q4k_superblock<XT, RT, NT, true>(stage, sb, tbl, x, P.M, P.K, kbase, acc);
            } else {
                q6k_superblock<XT, RT, NT>(stage, sb, tbl, x, P.M, P.K, kbase, acc);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->empty[s]);
    }
    if (!ok) {
        // A wait ran out (the sticky error word is set; results of this CTA are garbage).  Give
        // copies already in flight time to land before the CTA's shared memory is released, then
        // fall through so that the other warps are not left at the barrier below.
        for (uint32_t i = 0; i < 2048; ++i) __nanosleep(512);
    }

    // ---------------- cross-warp reduction + epilogue
    const int g = lane >> 2, t = lane & 3;
    if constexpr (SB) {
        // the one-token path keeps one partial per lane for rows g and g+8: fold the four t lanes
        // (Q6_K tiles of the same launch already hold column sums; their t > 0 columns are tokens
        // that do not exist and are never read)
        if (fmt == ALLOYB_Q4_K) {
#pragma unroll
            for (int rt = 0; rt < RT; ++rt)
#pragma unroll
                for (int i = 0; i < 4; i += 2) {
                    float v = acc[rt][0][i];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    acc[rt][0][i] = v;
                }
        }
    }
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float* o = red + ((warp * RT + rt) * 16) * (8 * NT);
            o[(g) * (8 * NT) + nt * 8 + 2 * t] = acc[rt][nt][0];
            o[(g) * (8 * NT) + nt * 8 + 2 * t + 1] = acc[rt][nt][1];
            o[(g + 8) * (8 * NT) + nt * 8 + 2 * t] = acc[rt][nt][2];
            o[(g + 8) * (8 * NT) + nt * 8 + 2 * t + 1] = acc[rt][nt][3];
        }
    consumer_sync();
    const int out_tiles = P.gated ? 1 : RT;
    const int tid = threadIdx.x;
    for (int idx = tid; idx < out_tiles * 16 * 8 * NT; idx += MMA_CONSUMERS * 32) {
        const int row = idx & 15;
        const int tok = (idx >> 4) % (8 * NT);
        const int rt = idx / (16 * 8 * NT);
        if (tok >= P.M || row0 + row >= sg.n_rows) continue;
        float v = 0.f, u = 0.f;
#pragma unroll
        for (int w = 0; w < MMA_CONSUMERS; ++w) {
            v += red[((w * RT + rt) * 16 + row) * (8 * NT) + tok];
            if (RT == 2) u += red[((w * RT + 1) * 16 + row) * (8 * NT) + tok];
        }
        const int64_t o = static_cast<int64_t>(tok) * sg.ldy + row0 + row;
        XT* y = static_cast<XT*>(sg.y);
        if (P.gated) {
            const float a = (P.act == ALLOYB_ACT_SILU) ? act_silu(v) : act_gelu_tanh(v);
            y[o] = from_f32<XT>(a * u);
        } else {
            XT r = from_f32<XT>(v);
            if (P.residual)
                r = from_f32<XT>(to_f32<XT>(static_cast<const XT*>(P.residual)[o]) + to_f32<XT>(r));
            y[o] = r;
        }
    }
}

// ------------------------------------------------------------------------------- host

template <typename XT, int RT, int NT, bool SB = false>
static int launch_mma(const MmaParams& P, int grid, int smem_bytes, cudaStream_t st) {
    static bool configured[64] = {};   // per template instance and device ordinal
    auto kern = linear_mma_kernel<XT, RT, NT, SB>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(MMA_THREADS);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, P);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

template <typename XT, int RT>
static int launch_mma_nt(MmaParams& P, int grid, int stage_rows_bytes, cudaStream_t st) {
    const int nt = (P.M + 7) / 8;
    const int NTt = nt <= 1 ? 1 : (nt == 2 ? 2 : 4);
    const int fixed = 128 + MMA_CONSUMERS * RT * 1024 + MMA_CONSUMERS * RT * 16 * 8 * NTt * 4;
    int stages = (MMA_SMEM_TARGET - fixed) / stage_rows_bytes;
    if (stages > MMA_STAGES) stages = MMA_STAGES;
    if (stages < 2) stages = 2;
    P.n_stages = stages;
    const int smem = fixed + stages * stage_rows_bytes;
    if constexpr (std::is_same<XT, __half>::value) {
        if (P.M == 1) return launch_mma<XT, RT, 1, true>(P, grid, smem, st);
    }
    switch (NTt) {
        case 1: return launch_mma<XT, RT, 1>(P, grid, smem, st);
        case 2: return launch_mma<XT, RT, 2>(P, grid, smem, st);
        default: return launch_mma<XT, RT, 4>(P, grid, smem, st);
    }
}

static bool seg_ok(const WeightSeg& s, int K) {
    if (s.format != ALLOYB_Q4_K && s.format != ALLOYB_Q6_K) return false;
    if (K % QK_K) return false;
    if (reinterpret_cast<uintptr_t>(s.data) % 16 || s.row_bytes % 16) return false;
    // a row's last chunk is copied rounded up to 16 bytes: it must stay inside the row pitch
    const int nsb = K / QK_K;
    const int bb = s.format == ALLOYB_Q4_K ? Q4K_BYTES : Q6K_BYTES;
    const int64_t need = static_cast<int64_t>((nsb - 1) / MMA_CH) * MMA_CH * bb +
                         ((static_cast<int64_t>((nsb - 1) % MMA_CH + 1) * bb + 15) & ~15LL);
    return need <= s.row_bytes;
}

int try_linear_fast(const void* x, int M, int K, int dtype, const WeightSeg* seg, int n_seg,
                    const void* residual, cudaStream_t st) {
    if (dtype != ALLOYB_F16 && dtype != ALLOYB_BF16) return ALLOYB_NOT_TAKEN;
    if (reinterpret_cast<uintptr_t>(x) % 16 || K % 8) return ALLOYB_NOT_TAKEN;
    if (M > 128) return ALLOYB_NOT_TAKEN;
    {
        const int rc = try_gemv_stream_mixed(x, M, K, dtype, seg, n_seg, residual, nullptr, 0.f, st);
        if (rc != ALLOYB_NOT_TAKEN) return rc;
    }
    int stage_bytes = 0;
    for (int i = 0; i < n_seg; ++i) {
        if (!seg_ok(seg[i], K)) return ALLOYB_NOT_TAKEN;
        const int sb = 16 * (seg[i].format == ALLOYB_Q4_K ? Q4_STRIDE : Q6_STRIDE);
        if (sb > stage_bytes) stage_bytes = sb;
    }
    const int esz = 2;
    for (int m0 = 0; m0 < M; m0 += 32) {
        MmaParams P = {};
        P.x = static_cast<const uint8_t*>(x) + static_cast<int64_t>(m0) * K * esz;
        P.M = (M - m0 < 32) ? (M - m0) : 32;
        P.K = K;
        P.n_seg = n_seg;
        P.gated = 0;
        P.stage_bytes = stage_bytes;
        int tiles = 0;
        for (int i = 0; i < n_seg; ++i) {
            MmaSeg& d = P.seg[i];
            d.format = seg[i].format;
            d.n_rows = seg[i].N;
            d.data = static_cast<const uint8_t*>(seg[i].data);
            d.row_bytes = seg[i].row_bytes;
            d.y = static_cast<uint8_t*>(seg[i].y) + static_cast<int64_t>(m0) * seg[i].ldy * esz;
            d.ldy = seg[i].ldy;
            d.tile0 = tiles;
            tiles += (seg[i].N + 15) / 16;
        }
        P.residual = residual ? static_cast<const uint8_t*>(residual) +
                                    static_cast<int64_t>(m0) * seg[0].ldy * esz
                              : nullptr;
        const int rc = (dtype == ALLOYB_F16) ? launch_mma_nt<__half, 1>(P, tiles, stage_bytes, st)
                                             : launch_mma_nt<__nv_bfloat16, 1>(P, tiles, stage_bytes, st);
        if (rc != ALLOYB_OK) return rc;
    }
    return ALLOYB_OK;
}

int try_gated_fast(const void* x, const void* gate, const void* gate_scales, const void* up,
                   const void* up_scales, void* y, int M, int N, int K, int format, int act, int dtype,
                   cudaStream_t st) {
    (void)gate_scales;
    (void)up_scales;
    if (format != ALLOYB_Q4_K) return ALLOYB_NOT_TAKEN;
    if (dtype != ALLOYB_F16 && dtype != ALLOYB_BF16) return ALLOYB_NOT_TAKEN;
    if (reinterpret_cast<uintptr_t>(x) % 16 || M > 128) return ALLOYB_NOT_TAKEN;
    WeightSeg gs = {ALLOYB_Q4_K, N, gate, nullptr, static_cast<int64_t>(K / QK_K) * Q4K_BYTES, y, N};
    WeightSeg us = gs;
    us.data = up;
    if (!seg_ok(gs, K) || !seg_ok(us, K)) return ALLOYB_NOT_TAKEN;
    {
        const WeightSeg pair[2] = {gs, us};
        const int rc = try_gemv_stream(x, M, K, dtype, pair, 2, true, act, nullptr, nullptr, 0.f, st, nullptr);
        if (rc != ALLOYB_NOT_TAKEN) return rc;
    }
    const int stage_bytes = 32 * Q4_STRIDE;
    const int esz = 2;
    for (int m0 = 0; m0 < M; m0 += 32) {
        MmaParams P = {};
        P.x = static_cast<const uint8_t*>(x) + static_cast<int64_t>(m0) * K * esz;
        P.M = (M - m0 < 32) ? (M - m0) : 32;
        P.K = K;
        P.n_seg = 2;
        P.gated = 1;
        P.act = act;
        P.stage_bytes = stage_bytes;
        for (int i = 0; i < 2; ++i) {
            MmaSeg& d = P.seg[i];
            d.format = ALLOYB_Q4_K;
            d.n_rows = N;
            d.data = static_cast<const uint8_t*>(i ? up : gate);
            d.row_bytes = gs.row_bytes;
            d.y = static_cast<uint8_t*>(y) + static_cast<int64_t>(m0) * N * esz;
            d.ldy = N;
            d.tile0 = 0;
        }
        const int tiles = (N + 15) / 16;
        const int rc = (dtype == ALLOYB_F16) ? launch_mma_nt<__half, 2>(P, tiles, stage_bytes, st)
                                             : launch_mma_nt<__nv_bfloat16, 2>(P, tiles, stage_bytes, st);
        if (rc != ALLOYB_OK) return rc;
    }
    return ALLOYB_OK;
}

}  // namespace alloyb

// Sticky device-side error word (1: a bounded mbarrier wait ran out).  Synchronises the device.
extern "C" int alloyb_device_error(int clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, alloyb::g_device_error, sizeof(int));
    if (e != cudaSuccess) { alloyb::set_cuda_error(e); return ALLOYB_E_CUDA; }
    const int v_tc = alloyb::gemm_tc_device_error(clear) | alloyb::attn_mma_device_error(clear) |
                     alloyb::gemv_stream_device_error(clear) | alloyb::decode_layer_device_error(clear);
    if (clear && v) {
        const int z = 0;
        e = cudaMemcpyToSymbol(alloyb::g_device_error, &z, sizeof(int));
        if (e != cudaSuccess) { alloyb::set_cuda_error(e); return ALLOYB_E_CUDA; }
    }
    return v | v_tc;
}

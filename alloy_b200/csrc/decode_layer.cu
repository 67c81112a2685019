// The decode step of a Llama-shape Q4_K / Q6_K model for ONE token as a single persistent launch.
//
// A decode step at batch 1 is ~190 small dependent operations (per layer: RMSNorm + q/k/v, RoPE +
// cache append + attention, o_proj + residual, RMSNorm + gate/up + SiLU, down + residual; then the
// final norm and the output head).  Launched one by one, each pays a few microseconds of launch,
// prologue and pipeline fill against one to ten microseconds of HBM time.  Here one cooperative
// grid (one CTA of sixteen warps per SM) walks a list of PHASES prepared once on the host:
//
//   * a GEMV phase is the streaming dequant-GEMV of linear_stream.cu (same slot geometries, same
//     per-super-block tensor-core arithmetic, same K split over the warps): the token is staged
//     (and normalised, when the phase carries an RMSNorm) into shared memory with loads that bypass
//     L1, together with the sums of its 16-element chunks (the Q4_K min and Q6_K offset terms);
//     every warp streams its K slice of the CTA's rows through its private TMA ring.  ONE routine
//     serves every weight format and grouping (the format is a per-matrix run-time value, so q, k
//     and v of different formats are one phase): a step touches ~200 phases and a routine per
//     variant did not fit the instruction cache;
//   * the attention phase rotates q (and the new k) in its prologue, appends the new K/V row to the
//     cache, and runs the split-K tensor-core decode attention of attn_mma.cu with sixteen warps
//     per CTA, (kv head, split) pairs dealt over the CTAs, the last CTA of a head merging the splits;
//   * phases are separated by a grid-wide barrier (an atomic counter polled with a bound) where the
//     next phase reads what the previous one wrote; a warp issues the first weight copies of the
//     NEXT phase before it goes to the barrier, so HBM stays busy across it.
//
// Row-parallel phases of a tensor-parallel model end with the same peer-memory exchange as the
// stand-alone kernel.  Every wait is bounded; a wait that runs out sets the sticky error word,
// after which the remaining barriers are passed without waiting and the results are undefined.
#include <new>
#include <vector>

#include "kv.cuh"
#include "linear_stream.cuh"

namespace alloyb {
namespace dl {

using namespace st;

constexpr int RING_WARP = 9728;                       // per-warp slot area: max over kinds of depth x 16 x pitch
constexpr int RING_BYTES = WARPS * RING_WARP;         // 155,648
constexpr int RED_BYTES = 4096;                       // per-tile partials of the K slices (double-buffered)
constexpr int BAR_BYTES = WARPS * MAX_D * 8;
constexpr int XS_HALVES = 28672;                      // the staged token: the largest K of a phase
constexpr int XS_BYTES = XS_HALVES * 2;
constexpr int SUMS_BYTES = XS_HALVES / 16 * 4;        // fp32 sum of every 16-element chunk of the token
constexpr int DESC_SLOT = 384, DESC_SLOTS = 3;        // phase descriptors cached in shared memory
constexpr int PLAN_SLOT = 64;
constexpr int OFF_RED = RING_BYTES, OFF_BAR = OFF_RED + RED_BYTES, OFF_XS = OFF_BAR + BAR_BYTES,
              OFF_SUMS = OFF_XS + XS_BYTES, OFF_NRED = OFF_SUMS + SUMS_BYTES, OFF_DESC = OFF_NRED + 128,
              OFF_PLAN = OFF_DESC + DESC_SLOTS * DESC_SLOT, SMEM_BYTES = OFF_PLAN + WARPS * PLAN_SLOT;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
constexpr uint32_t GRID_SPIN = 1u << 24;
constexpr float NEG_BIG = -1.0e30f;
constexpr float P_BIAS = 64.0f;                       // see attn_mma.cu
constexpr int AD = 128;                               // head_dim of the attention phase
constexpr int NKP = AD / 32;
constexpr int SLAB = PAGE_TOKENS * NKP * KV_BLOCK_BYTES;
constexpr int MAX_SPLITS = 64;

enum { PH_GEMV = 0, PH_ATTN = 1 };

struct GSeg {
    const uint8_t* data;
    int64_t row_bytes;
    void* y;
    int n_rows;
    int row_base;        // first row of this matrix in the phase's stacked row space
    int kind;            // st::Kind: slot geometry / weight format of this matrix
    int map;             // index of its tensor map in the step's map array
};
struct GemvDesc {
    const __half* x;
    const __half* residual;
    const __half* norm_w;        // non-null: RMSNorm(x; norm_w, eps) on the way in
    float eps;
    int n_seg;                   // matrices walked row-wise (1 for a gate/up pair)
    GSeg seg[MAX_SEG];
    int total_rows;
    int nsb;
    int gu;                      // gate/up pair: seg[0] rows to warps 0-7, seg[1] rows to warps 8-15, y = act(g) * u
    int act;
    int depth;                   // ring slots per warp
    int gw;                      // warps per K-split group: 1, 4, 8 or 16
    int sbs;                     // super-blocks per slot (the same for every matrix of the phase)
    int slot_bytes;              // ring slot stride
    int stage_x;                 // 1: stage x into shared memory; 0: the previous phase's token is still there
    int K;
    TpArgs tp;                   // world == 0: plain linear
};
struct AttnDesc {
    const __half* q;     // this step's projections, un-rotated: (H, 128), (KV_H, 128), (KV_H, 128)
    const __half* k;
    const __half* v;
    __half* out;         // (H, 128)
    int layout;          // ALLOYB_KV_F16 or ALLOYB_KV_Q8_PAGED
    KVPtrs kv;
    const int32_t* pos;
    const float* inv_freq;
    int H, KV_H, G, splits;
    float scale_log2;
    float* part_o;       // (H, splits, 128)
    float* part_lse;     // (H, splits)
    unsigned int* counters;   // (KV_H)
    int* status;
};
struct PhaseDesc {
    int type;
    int barrier_after;
    union {
        GemvDesc g;
        AttnDesc a;
    };
};
static_assert(sizeof(PhaseDesc) <= DESC_SLOT && sizeof(PhaseDesc) % 4 == 0, "descriptor slot");
struct StepDesc {
    const PhaseDesc* phases;
    int n_phases;
    const CUtensorMap* maps;
    unsigned int* barrier;       // zeroed on the stream before every launch
    unsigned long long* trace;   // optional: per (phase, CTA) four nanosecond clocks: token staged, phase done,
                                 // next phase's copies issued, barrier passed
};

struct RingState {
    uint32_t ring;       // shared address of this warp's slot area
    uint32_t bar0;       // ... of its MAX_D barriers
    uint32_t parity;     // bit s: parity the next wait on barrier s uses
    bool ok;             // false once a bounded wait of this warp ran out
};

// A warp's share of a phase.  Warp-uniform, kept in shared memory (one slot per warp).
struct Plan {
    int lo, hi, sb_lo, slice, spt, my_tiles, n_stage, issued, p_r, p_slot, tstep, grp, wg;
    int seg, row, lim;   // producer cursor
};
static_assert(sizeof(Plan) <= PLAN_SLOT, "plan slot");

__device__ __forceinline__ uint4 ldcg128(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ int kind_pitch(int kind) { return kind == Q6 ? 240 : (kind == Q4x2 ? 304 : 144); }
__device__ __forceinline__ int kind_blk(int kind) { return kind == Q6 ? Q6K_BYTES : Q4K_BYTES; }

// ------------------------------------------------------------------------------------ grid barrier

__device__ __forceinline__ void grid_sync(unsigned int* ctr, unsigned int& target) {
    __syncthreads();
    if (threadIdx.x == 0) {
        target += gridDim.x;
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
        if (*reinterpret_cast<volatile int*>(&g_error) == 0) {
            uint32_t i = 0;
            for (; i < GRID_SPIN; ++i) {
                unsigned int v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
                if (v >= target) break;
            }
            if (i == GRID_SPIN) atomicExch(&g_error, 2);
        }
    }
    __syncthreads();
}

// ------------------------------------------------------------------------------------ GEMV phases

// Row cursor over the phase's stacked matrices (as st::Cursor, on this file's descriptor).
__device__ __forceinline__ void cur_enter(int& seg, int& row, int& lim, const GemvDesc& d, int lo, int hi) {
    while (seg < d.n_seg) {
        const int base = d.seg[seg].row_base, n = d.seg[seg].n_rows;
        const int a = lo > base ? lo - base : 0;
        const int b = hi - base < n ? hi - base : n;
        if (a < b) {
            row = a;
            lim = b;
            return;
        }
        ++seg;
    }
}
__device__ __forceinline__ void cur_next(int& seg, int& row, int& lim, const GemvDesc& d, int lo, int hi, int steps) {
    for (int i = 0; i < steps && seg < d.n_seg; ++i) {
        row += 16;
        if (row >= lim) {
            ++seg;
            cur_enter(seg, row, lim, d, lo, hi);
        }
    }
}

// One stage (16 rows x sbs super-blocks of the producer cursor's tile) into the next ring slot.
__device__ __forceinline__ void gemv_issue(Plan& pl, const GemvDesc& d, const CUtensorMap* maps, const RingState& rs,
                                           int lane) {
    const GSeg& sg = d.seg[d.gu ? pl.grp : pl.seg];
    const int kind = sg.kind, pitch = kind_pitch(kind), blk = kind_blk(kind);
    const int sb = pl.sb_lo + pl.p_r * d.sbs;
    const int nvalid = pl.lim - pl.row < 16 ? pl.lim - pl.row : 16;
    const uint32_t bar = rs.bar0 + 8 * pl.p_slot, dst = rs.ring + pl.p_slot * d.slot_bytes;
    const int win = (sb * blk) & ~15;                                // 16-byte-aligned start of the stage in a row
    if (nvalid == 16) {
        if (lane == 0) {
            mbar_expect_tx(bar, 16 * pitch);
            tma_2d(dst, maps + sg.map, win / 4, pl.row, bar);
        }
    } else {
        int bytes = d.sbs * blk;
        if (kind == Q6) {
            const int left = static_cast<int>(sg.row_bytes) - win;
            bytes = left < pitch ? left : pitch;
        }
        if (lane == 0) mbar_expect_tx(bar, nvalid * bytes);
        __syncwarp();
        if (lane < nvalid) bulk_g2s(dst + lane * pitch, sg.data + (pl.row + lane) * sg.row_bytes + win, bytes, bar);
    }
    ++pl.issued;
    if (++pl.p_slot == d.depth) pl.p_slot = 0;
    if (++pl.p_r == pl.spt) {
        pl.p_r = 0;
        cur_next(pl.seg, pl.row, pl.lim, d, pl.lo, pl.hi, pl.tstep);
    }
}

// Plan this warp's share of the phase and start its first weight copies (they depend on nothing
// this step computes, so this runs BEFORE the barrier that guards the phase's input).
__device__ __noinline__ void gemv_begin(Plan& pl_out, const GemvDesc& d, const CUtensorMap* maps, const RingState& rs_in,
                                        int warp, int lane) {
    // everything is computed in registers and stored once: the plan and the descriptor are both in
    // shared memory, and stores to one would make the compiler re-read the other
    const RingState rs = rs_in;
    const int gw = d.gw, nsb = d.nsb, total_rows = d.total_rows, gu = d.gu, depth = d.depth, sbs = d.sbs;
    Plan pl;
    pl.grp = warp / gw;
    pl.wg = warp % gw;
    pl.tstep = gu ? 1 : WARPS / gw;
    pl.lo = static_cast<int>(static_cast<uint32_t>(total_rows) * blockIdx.x / gridDim.x);
    pl.hi = static_cast<int>(static_cast<uint32_t>(total_rows) * (blockIdx.x + 1) / gridDim.x);
    pl.sb_lo = (pl.wg * nsb) / gw;
    pl.slice = ((pl.wg + 1) * nsb) / gw - pl.sb_lo;
    pl.spt = pl.slice / sbs;
    int tiles = 0;
    {
        int seg = 0, row = 0, lim = 0;
        cur_enter(seg, row, lim, d, pl.lo, pl.hi);
        cur_next(seg, row, lim, d, pl.lo, pl.hi, gu ? 0 : pl.grp);
        while (seg < d.n_seg) {
            ++tiles;
            cur_next(seg, row, lim, d, pl.lo, pl.hi, pl.tstep);
        }
    }
    pl.my_tiles = tiles;
    pl.n_stage = tiles * pl.spt;
    pl.seg = pl.row = pl.lim = 0;
    cur_enter(pl.seg, pl.row, pl.lim, d, pl.lo, pl.hi);
    cur_next(pl.seg, pl.row, pl.lim, d, pl.lo, pl.hi, gu ? 0 : pl.grp);
    pl.issued = pl.p_r = pl.p_slot = 0;
    if (rs.ok)
        while (pl.issued < pl.n_stage && pl.issued < depth) gemv_issue(pl, d, maps, rs, lane);
    pl_out = pl;
}

// The token of a phase -> shared memory (fp16) plus the fp32 sum of each 16-element chunk, read past
// L1 (another SM wrote it earlier in this launch) in ONE round trip: a thread keeps its chunks in
// registers between the sum of squares and the scaling.  RMSNorm arithmetic as the stand-alone
// kernels: fp32 sum of squares, x * r narrowed to fp16, then times the fp16 weight.
constexpr int STAGE_CHUNKS = XS_HALVES / 8 / (WARPS * 32);          // 16-byte chunks per thread at the largest K
__device__ __noinline__ void stage_token(const GemvDesc& d, __half* xs, float* sums, float* nred) {
    const int K = d.K, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const __half* x = d.x;
    const __half* norm_w = d.norm_w;
    uint4 xv[STAGE_CHUNKS], wv[STAGE_CHUNKS];
#pragma unroll
    for (int c = 0; c < STAGE_CHUNKS; ++c) {
        const int i = (c * WARPS * 32 + threadIdx.x) * 8;
        xv[c] = make_uint4(0u, 0u, 0u, 0u);
        wv[c] = xv[c];
        if (i < K) {
            xv[c] = ldcg128(x + i);
            if (norm_w) wv[c] = __ldg(reinterpret_cast<const uint4*>(norm_w + i));
        }
    }
    if (norm_w) {
        float ssq = 0.f;
#pragma unroll
        for (int c = 0; c < STAGE_CHUNKS; ++c) {
            const __half2* h2 = reinterpret_cast<const __half2*>(&xv[c]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f2 = __half22float2(h2[j]);
                ssq = fmaf(f2.x, f2.x, ssq);
                ssq = fmaf(f2.y, f2.y, ssq);
            }
        }
        ssq = warp_sum(ssq);
        if (lane == 0) nred[warp] = ssq;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < WARPS; ++i) tot += nred[i];
        const float r = rsqrtf(tot / static_cast<float>(K) + d.eps);
#pragma unroll
        for (int c = 0; c < STAGE_CHUNKS; ++c) {
            const __half* hv = reinterpret_cast<const __half*>(&xv[c]);
            const __half* hw = reinterpret_cast<const __half*>(&wv[c]);
            uint4 o;
            __half* ho = reinterpret_cast<__half*>(&o);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const __half normed = __float2half_rn(__half2float(hv[j]) * r);
                ho[j] = __float2half_rn(__half2float(hw[j]) * __half2float(normed));
            }
            xv[c] = o;
        }
    }
#pragma unroll
    for (int c = 0; c < STAGE_CHUNKS; ++c) {
        const int i = (c * WARPS * 32 + threadIdx.x) * 8;
        const __half2* h2 = reinterpret_cast<const __half2*>(&xv[c]);
        float s8 = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f2 = __half22float2(h2[j]);
            s8 += f2.x + f2.y;
        }
        s8 += __shfl_xor_sync(0xffffffffu, s8, 1);                   // lanes 2k, 2k+1 hold one 16-element chunk
        if (i < K) {
            *reinterpret_cast<uint4*>(xs + i) = xv[c];
            if ((lane & 1) == 0) sums[i >> 4] = s8;
        }
    }
    __syncthreads();
}

// B fragments of one super-block of the staged token (see st::load_xfrag); the per-sub-block sums
// come from the staged chunk sums instead of eight extra MMAs.
__device__ __forceinline__ void load_xfrag_s(XFrag& f, const __half* xs, const float* sums, int sb, int g, int t) {
#pragma unroll
    for (int j = 0; j < 8; ++j) f.b[j][0] = f.b[j][1] = 0u;
    if ((g >> 1) == t) {
        const uint4* xp = reinterpret_cast<const uint4*>(xs + sb * QK_K + 32 * g);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = xp[q];
            f.b[2 * q][0] = prmt(v.x, v.y, 0x5410u);
            f.b[2 * q][1] = prmt(v.x, v.y, 0x7632u);
            f.b[2 * q + 1][0] = prmt(v.z, v.w, 0x5410u);
            f.b[2 * q + 1][1] = prmt(v.z, v.w, 0x7632u);
        }
    }
    const float4 s4 = *reinterpret_cast<const float4*>(sums + sb * 16 + 4 * t);       // sub-blocks 2t, 2t+1
    f.sx0 = s4.x + s4.y;
    f.sx1 = s4.z + s4.w;
}
__device__ __forceinline__ void load_xfrag6_s(XFrag6& f, const __half* xs, const float* sums, int sb, int g, int t) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint2 v = *reinterpret_cast<const uint2*>(xs + sb * QK_K + 128 * h + 16 * g + 4 * t);
        f.b[h][0] = prmt(v.x, v.y, 0x5410u);
        f.b[h][1] = prmt(v.x, v.y, 0x7632u);
        const float2 s2 = *reinterpret_cast<const float2*>(sums + sb * 16 + 8 * h + 2 * t);
        f.sx[h][0] = s2.x;
        f.sx[h][1] = s2.y;
    }
}

// st::unit_q4k with the slot's row pitch as a run-time value (one routine for both Q4_K geometries).
__device__ __forceinline__ void unit_q4k_rt(uint32_t blk, int pitch, const XFrag& f, const ScaleSel& ss, int g, int t,
                                            float& a0, float& a1) {
    const uint32_t rb = blk + g * pitch, rb8 = rb + 8 * pitch;
    const uint4 p0 = lds128(rb + 16 + 32 * t), p1 = lds128(rb + 32 + 32 * t);
    const uint4 r0 = lds128(rb8 + 16 + 32 * t), r1 = lds128(rb8 + 32 + 32 * t);
    const uint4 h0 = lds128(rb), h1 = lds128(rb8);
    const uint32_t wg[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    const uint32_t wh[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    float clo[4], chi[4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t ug = wg[j] >> 8, uh = wh[j] >> 8;
        if (j == 0) {
            mma_zero(clo, wg[j] & 0x000f000fu, wh[j] & 0x000f000fu, ug & 0x000f000fu, uh & 0x000f000fu, f.b[j][0], f.b[j][1]);
            mma_zero(chi, wg[j] & 0x00f000f0u, wh[j] & 0x00f000f0u, ug & 0x00f000f0u, uh & 0x00f000f0u, f.b[j][0], f.b[j][1]);
        } else {
            mma_acc(clo, wg[j] & 0x000f000fu, wh[j] & 0x000f000fu, ug & 0x000f000fu, uh & 0x000f000fu, f.b[j][0], f.b[j][1]);
            mma_acc(chi, wg[j] & 0x00f000f0u, wh[j] & 0x00f000f0u, ug & 0x00f000f0u, uh & 0x00f000f0u, f.b[j][0], f.b[j][1]);
        }
    }
    const uint32_t Y = prmt(h0.y, h1.y, ss.sel), Z = prmt(h0.z, h1.z, ss.sel), Wd = prmt(h0.w, h1.w, ss.sel);
    const uint32_t sc4 = ((ss.high ? Wd : Y) & ss.m_a) | ((Y >> 2) & ss.m_b);
    const uint32_t mn4 = ((ss.high ? (Wd >> 4) : Z) & ss.m_a) | ((Z >> 2) & ss.m_b);
    const float2 dm0 = __half22float2(*reinterpret_cast<const __half2*>(&h0.x));
    const float2 dm1 = __half22float2(*reinterpret_cast<const __half2*>(&h1.x));
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

__device__ __noinline__ void gemv_run(const Plan& pl_in, const GemvDesc& d, const CUtensorMap* maps, RingState& rs_io,
                                      const __half* xs, const float* sums, float* red_all, int warp, int lane) {
    Plan pl = pl_in;                                   // registers: nothing below stores to the shared copy
    RingState rs = rs_io;
    const int g = lane >> 2, t = lane & 3;
    const int GW = d.gw, grp = pl.grp, wg = pl.wg, D = d.depth, gu = d.gu, sbs = d.sbs, slot_bytes = d.slot_bytes;
    float* red = red_all + grp * (2 * GW * 16);
    const int tp_world = gu ? 0 : d.tp.world, tp_rank = d.tp.rank, tp_max_n = d.tp.max_n, act = d.act;
    const __half* residual = d.residual;

    uint32_t tp_next = 0;
    if (tp_world) tp_next = *reinterpret_cast<volatile uint32_t*>(d.tp.peer[tp_rank]) + 1u;
    const ScaleSel ss = make_scale_sel(t);

    int c_slot = 0;
    int cseg = 0, crow = 0, clim = 0;
    cur_enter(cseg, crow, clim, d, pl.lo, pl.hi);
    cur_next(cseg, crow, clim, d, pl.lo, pl.hi, gu ? 0 : grp);
    const int my_tiles = pl.my_tiles, sb_lo = pl.sb_lo, sb_hi = pl.sb_lo + pl.slice;
    for (int it = 0; it < my_tiles; ++it) {
        const int kind = d.seg[gu ? grp : cseg].kind, pitch = kind_pitch(kind);
        float acc0 = 0.f, acc1 = 0.f;
        for (int sb = sb_lo; sb < sb_hi; sb += sbs) {
            const uint32_t slot = rs.ring + c_slot * slot_bytes;
            if (rs.ok) rs.ok = mbar_wait(rs.bar0 + 8 * c_slot, (rs.parity >> c_slot) & 1u);
            rs.parity ^= 1u << c_slot;
            if (++c_slot == D) c_slot = 0;
            rs.ok = __all_sync(0xffffffffu, rs.ok);
            if (rs.ok) {
                if (kind == Q6) {
                    XFrag6 f;
                    load_xfrag6_s(f, xs, sums, sb, g, t);
                    const uint32_t off = static_cast<uint32_t>(sb * Q6K_BYTES) & 15u;
                    if (off & 2u) unit_q6k<false>(slot + off, f, g, t, acc0, acc1);
                    else unit_q6k<true>(slot + off, f, g, t, acc0, acc1);
                } else {
                    for (int i = 0; i < sbs; ++i) {
                        XFrag f;
                        load_xfrag_s(f, xs, sums, sb + i, g, t);
                        unit_q4k_rt(slot + i * Q4K_BYTES, pitch, f, ss, g, t, acc0, acc1);
                    }
                }
            }
            __syncwarp();
            if (rs.ok && pl.issued < pl.n_stage) gemv_issue(pl, d, maps, rs, lane);      // refills the slot just drained
        }
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
        auto store = [&](int tl, float v, float u) {
            if (crow + tl >= clim) return;
            const int row = crow + tl;
            __half* y = static_cast<__half*>(d.seg[cseg].y);
            if (gu) {
                const float a = (act == ALLOYB_ACT_SILU) ? act_silu(v) : act_gelu_tanh(v);
                y[row] = __float2half_rn(a * u);
            } else if (tp_world) {
                const size_t off = TP_SLOTS_OFF + (static_cast<size_t>((tp_next & 1u) * 8 + tp_rank) * tp_max_n + row) * 4;
                for (int p = 0; p < tp_world; ++p) *reinterpret_cast<float*>(d.tp.peer[p] + off) = v;
            } else {
                __half r = __float2half_rn(v);
                if (residual) r = __float2half_rn(__half2float(__ldcg(residual + row)) + __half2float(r));
                y[row] = r;
            }
        };
        if (gu) {
            float* rbuf = red_all + (it & 1) * (WARPS * 16);
            if (t == 0) {
                rbuf[warp * 16 + g] = acc0;
                rbuf[warp * 16 + g + 8] = acc1;
            }
            __syncthreads();
            if (threadIdx.x < 16) {
                float v = 0.f, u = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    v += rbuf[w * 16 + threadIdx.x];
                    u += rbuf[(8 + w) * 16 + threadIdx.x];
                }
                store(threadIdx.x, v, u);
            }
        } else if (GW == 1) {
            if (t == 0) {
                store(g, acc0, 0.f);
                store(g + 8, acc1, 0.f);
            }
        } else {
            float* rbuf = red + (it & 1) * (GW * 16);
            if (t == 0) {
                rbuf[wg * 16 + g] = acc0;
                rbuf[wg * 16 + g + 8] = acc1;
            }
            asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(GW * 32) : "memory");
            const int tl = threadIdx.x - grp * GW * 32;
            if (tl < 16) {
                float v = 0.f;
                for (int w = 0; w < GW; ++w) v += rbuf[w * 16 + tl];
                store(tl, v, 0.f);
            }
        }
        cur_next(cseg, crow, clim, d, pl.lo, pl.hi, pl.tstep);
    }
    if (tp_world) {
        // all-reduce of this CTA's rows over the ranks (see linear_stream.cu)
        const int lo = pl.lo, hi = pl.hi;
        const uint32_t spin = d.tp.spin;
        __syncthreads();
        uint8_t* mine = d.tp.peer[tp_rank];
        if (threadIdx.x >= 32 && threadIdx.x < 32 + tp_world) {
            const int p = threadIdx.x - 32;
            uint32_t* f = reinterpret_cast<uint32_t*>(d.tp.peer[p] + TP_FLAGS_OFF) + tp_rank * 256 + blockIdx.x;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(tp_next) : "memory");
        }
        if (threadIdx.x < tp_world) {
            const uint32_t* f = reinterpret_cast<const uint32_t*>(mine + TP_FLAGS_OFF) + threadIdx.x * 256 + blockIdx.x;
            uint32_t v = 0, i = 0;
            for (; i < spin; ++i) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                if (static_cast<int32_t>(v - tp_next) >= 0) break;
                if (i > 64) __nanosleep(64);
            }
            if (i == spin) atomicExch(&g_error, 1);
        }
        __syncthreads();
        const float* slots = reinterpret_cast<const float*>(mine + TP_SLOTS_OFF) +
                             static_cast<size_t>(tp_next & 1u) * 8 * tp_max_n;
        __half* y = static_cast<__half*>(d.seg[0].y);
        for (int row = lo + threadIdx.x; row < hi; row += blockDim.x) {
            float v = 0.f;
            for (int r = 0; r < tp_world; ++r) v += __ldcg(slots + static_cast<size_t>(r) * tp_max_n + row);
            __half o = __float2half_rn(v);
            if (residual) o = __float2half_rn(__half2float(__ldcg(residual + row)) + __half2float(o));
            y[row] = o;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t* ctr = reinterpret_cast<uint32_t*>(mine + 4);
            __threadfence();
            if (atomicAdd(ctr, 1u) == gridDim.x - 1) {
                *ctr = 0u;
                __threadfence();
                *reinterpret_cast<volatile uint32_t*>(mine) = tp_next;
            }
        }
    }
    rs_io = rs;
}

// ------------------------------------------------------------------------------------ attention phase

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
__device__ __forceinline__ void mma8(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    // rows 8..15 of A are zero (at most 8 query heads per KV head)
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lds32g(const void* p) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ uint32_t lds16g(const void* p) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ void lds_words_align2(const uint8_t* p, uint32_t& w0, uint32_t& w1, bool two) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint8_t* base = reinterpret_cast<const uint8_t*>(a & ~uintptr_t(3));
    const uint32_t x0 = lds32g(base), x1 = lds32g(base + 4);
    if (a & 2u) {
        w0 = __funnelshift_r(x0, x1, 16);
        if (two) w1 = __funnelshift_r(x1, lds32g(base + 8), 16);
    } else {
        w0 = x0;
        if (two) w1 = x1;
    }
}

struct Q8Out {
    int code;
    __half scale;
};
// the block quantiser of kv.cu: all 32 lanes hold one element each of the same block
__device__ __forceinline__ Q8Out quantize_block(float x) {
    const float m = warp_max(fabsf(x));
    const float inv = (m > 0.f) ? __fdiv_rn(127.0f, m) : 0.f;
    const float q = __fmul_rn(x, inv);
    const float mag = floorf(__fadd_rn(fabsf(q), 0.5f));
    Q8Out r;
    r.code = static_cast<int>(copysignf(mag, q));
    r.scale = __float2half_rn(__fdiv_rn(m, 127.0f));
    return r;
}

struct AttnSmem {                    // lives in the token-staging area
    __half q[8][AD];                 // rotated queries of the CTA's KV head
    __half k[AD];                    // the new token's rotated K row and its V row
    __half v[AD];
    uint8_t k8[NKP * KV_BLOCK_BYTES + 8];    // ... as q8_0 blocks (paged layout)
    uint8_t v8[NKP * KV_BLOCK_BYTES + 8];
    float m[WARPS][8], l[WARPS][8];
    float wgt[8 * MAX_SPLITS];
    int last;
};

template <int LAYOUT>
__device__ __noinline__ void attn_phase(const AttnDesc& A, RingState& rs, uint8_t* ring_area, AttnSmem* S,
                                           int warp, int lane) {
    constexpr bool PAGED = LAYOUT == ALLOYB_KV_Q8_PAGED;
    const int g = lane >> 2, t = lane & 3;
    const int G = A.G;
    const int item = blockIdx.x;
    if (item >= A.KV_H * A.splits) return;             // this CTA has no (head, split) pair
    const int kvh = item / A.splits, split = item - kvh * A.splits;
    int pos = __ldcg(A.pos);
    if (pos >= A.kv.S_max || pos < 0) {
        if (threadIdx.x == 0 && A.status) atomicOr(A.status, KV_STATUS_POS_RANGE);
        pos = pos < 0 ? 0 : A.kv.S_max - 1;
    }
    const int len = pos + 1;
    int chunk = (len + A.splits - 1) / A.splits;
    chunk = (chunk + 15) & ~15;
    const int t0 = split * chunk;
    const int t1 = min(len, t0 + chunk);
    const int n_tiles = t1 > t0 ? (t1 - t0 + 15) / 16 : 0;
    const bool owner = pos >= t0 && pos < t1;          // this CTA's range holds the new token

    // ---- prologue: rotate q (all CTAs of the head) and k (owner), append the new row (owner)
    __syncthreads();
    {
        const int half = AD / 2;
        for (int i = threadIdx.x; i < (G + 1) * half; i += WARPS * 32) {
            const int hh = i / half, j = i - hh * half;
            if (hh == G && !owner) continue;
            const __half* src = hh < G ? A.q + static_cast<int64_t>(kvh * G + hh) * AD : A.k + static_cast<int64_t>(kvh) * AD;
            const float angle = static_cast<float>(pos) * A.inv_freq[j];
            float sn, cs;
            sincosf(angle, &sn, &cs);
            const float x1 = __half2float(__ldcg(src + j)), x2 = __half2float(__ldcg(src + j + half));
            const __half r1 = __float2half_rn(__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn)));
            const __half r2 = __float2half_rn(__fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn)));
            __half* dst = hh < G ? S->q[hh] : S->k;
            dst[j] = r1;
            dst[j + half] = r2;
        }
        if (owner)
            for (int i = threadIdx.x; i < AD; i += WARPS * 32) S->v[i] = __ldcg(A.v + static_cast<int64_t>(kvh) * AD + i);
    }
    __syncthreads();
    if (owner) {
        if (!PAGED) {
            const int64_t row = (static_cast<int64_t>(kvh) * A.kv.S_max + pos) * AD;       // batch 0
            for (int i = threadIdx.x; i < 2 * AD; i += WARPS * 32) {
                if (i < AD) static_cast<__half*>(A.kv.k0)[row + i] = S->k[i];
                else static_cast<__half*>(A.kv.v0)[row + i - AD] = S->v[i - AD];
            }
        } else if (warp < 2 * NKP) {
            // warps 0-3: K blocks, warps 4-7: V blocks
            const int which = warp / NKP, blk = warp % NKP;
            const Q8Out qb = quantize_block(__half2float((which ? S->v : S->k)[blk * 32 + lane]));
            uint8_t* row8 = which ? S->v8 : S->k8;
            if (lane == 0) *reinterpret_cast<__half*>(row8 + blk * KV_BLOCK_BYTES) = qb.scale;
            reinterpret_cast<int8_t*>(row8 + blk * KV_BLOCK_BYTES + 2)[lane] = static_cast<int8_t>(qb.code);
            const int32_t* table = static_cast<const int32_t*>(A.kv.k1);
            const int64_t page = table[pos / PAGE_TOKENS];
            if (page < 0 || page >= A.kv.num_pages) {
                if (lane == 0 && A.status) atomicOr(A.status, KV_STATUS_PAGE_RANGE);
            } else {
                uint8_t* dst = static_cast<uint8_t*>(A.kv.k0) +
                               paged_row_offset(page, which, kvh, pos % PAGE_TOKENS, A.KV_H, AD) + blk * KV_BLOCK_BYTES;
                if (lane == 0) *reinterpret_cast<__half*>(dst) = qb.scale;
                reinterpret_cast<int8_t*>(dst + 2)[lane] = static_cast<int8_t>(qb.code);
            }
        }
        __syncthreads();
    }

    // ---- Q fragments (rows = heads of this group; rows >= G are zero) and per-block sums of q
    uint32_t qa[NKP][2][2];
    float qsum[NKP];
#pragma unroll
    for (int kp = 0; kp < NKP; ++kp) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (g < G) v = *reinterpret_cast<const uint4*>(&S->q[g][32 * kp + 8 * t]);
        qa[kp][0][0] = v.x;
        qa[kp][0][1] = v.y;
        qa[kp][1][0] = v.z;
        qa[kp][1][1] = v.w;
        const float2 a = unpack_h2(v.x), b2 = unpack_h2(v.y), c = unpack_h2(v.z), d2 = unpack_h2(v.w);
        float s = ((a.x + a.y) + (b2.x + b2.y)) + ((c.x + c.y) + (d2.x + d2.y));
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        qsum[kp] = s;
    }

    float m_run = NEG_BIG, l_run = 0.f;
    float o[NKP * 4][2];
    float ocorr[NKP];
    float zz2 = 0.f, zz3 = 0.f;
#pragma unroll
    for (int i = 0; i < NKP * 4; ++i) o[i][0] = o[i][1] = 0.f;
#pragma unroll
    for (int kp = 0; kp < NKP; ++kp) ocorr[kp] = 0.f;

    const int64_t head_row = static_cast<int64_t>(kvh) * A.kv.S_max;
    uint8_t* stage = ring_area + warp * RING_WARP;        // paged: [2 slots][K slab | V slab]
    const int32_t* table = static_cast<const int32_t*>(A.kv.k1);

    auto issue_page = [&](int tile_idx, int slot) {
        const int tok0 = t0 + tile_idx * 16;
        int64_t page = table[tok0 / PAGE_TOKENS];
        if (page < 0 || page >= A.kv.num_pages) {
            if (A.status) atomicOr(A.status, KV_STATUS_PAGE_RANGE);
            page = 0;
        }
        const uint8_t* pool = static_cast<const uint8_t*>(A.kv.k0);
        const uint32_t bar = rs.bar0 + 8 * slot, dst = rs.ring + slot * (2 * SLAB);
        mbar_expect_tx(bar, 2 * SLAB);
        bulk_g2s(dst, pool + paged_row_offset(page, 0, kvh, 0, A.KV_H, AD), SLAB, bar);
        bulk_g2s(dst + SLAB, pool + paged_row_offset(page, 1, kvh, 0, A.KV_H, AD), SLAB, bar);
    };

    int n_mine = 0;
    if (PAGED && warp < n_tiles && lane == 0 && rs.ok) issue_page(warp, 0);
    for (int tile = warp; tile < n_tiles; tile += WARPS, ++n_mine) {
        const int tok0 = t0 + tile * 16;
        const int slot = n_mine & 1;
        const uint8_t* kslab = stage + slot * (2 * SLAB);
        const uint8_t* vslab = kslab + SLAB;
        if (PAGED) {
            if (tile + WARPS < n_tiles && lane == 0 && rs.ok) issue_page(tile + WARPS, slot ^ 1);
            if (rs.ok) rs.ok = mbar_wait(rs.bar0 + 8 * slot, (rs.parity >> slot) & 1u);
            rs.parity ^= 1u << slot;
            rs.ok = __all_sync(0xffffffffu, rs.ok);
            if (!rs.ok) continue;
            if (owner && pos >= tok0 && pos < tok0 + 16) {
                // the page was copied while (or before) the new row was written: take the row from shared memory
                uint8_t* kr = const_cast<uint8_t*>(kslab) + (pos - tok0) * (NKP * KV_BLOCK_BYTES);
                uint8_t* vr = const_cast<uint8_t*>(vslab) + (pos - tok0) * (NKP * KV_BLOCK_BYTES);
                for (int i = lane; i < NKP * KV_BLOCK_BYTES / 2; i += 32) {
                    reinterpret_cast<uint16_t*>(kr)[i] = reinterpret_cast<const uint16_t*>(S->k8)[i];
                    reinterpret_cast<uint16_t*>(vr)[i] = reinterpret_cast<const uint16_t*>(S->v8)[i];
                }
                __syncwarp();
            }
        }
        // ---------------- S = Q K^T
        float s[2][2];
#pragma unroll
        for (int tb = 0; tb < 2; ++tb) {
            const int tok = min(tok0 + 8 * tb + g, t1 - 1);
            float sc[2] = {0.f, 0.f};
            if (!PAGED) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                const __half* krow = (owner && tok == pos) ? S->k : static_cast<const __half*>(A.kv.k0) + (head_row + tok) * AD;
                const uint4* kr = reinterpret_cast<const uint4*>(krow) + t;
#pragma unroll
                for (int kp = 0; kp < NKP; ++kp) {
                    const uint4 kv = kr[kp * 4];
                    mma8(c, qa[kp][0][0], qa[kp][0][1], kv.x, kv.y);
                    mma8(c, qa[kp][1][0], qa[kp][1][1], kv.z, kv.w);
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
                    lds_words_align2(kslab + (8 * tb + g) * (NKP * KV_BLOCK_BYTES) + kp * KV_BLOCK_BYTES + 2 + 8 * t, w0, w1, true);
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        ks[e] = tok0 + 8 * tb + 2 * t + e < t1
                                    ? half_bits_to_f32(lds16g(kslab + (8 * tb + 2 * t + e) * (NKP * KV_BLOCK_BYTES) + kp * KV_BLOCK_BYTES))
                                    : 0.f;
                    const uint32_t u0 = w0 ^ 0x80808080u, u1 = w1 ^ 0x80808080u;
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma8(c, qa[kp][0][0], qa[kp][0][1], prmt(u0, 0u, 0x4140u), prmt(u0, 0u, 0x4342u));
                    mma8(c, qa[kp][1][0], qa[kp][1][1], prmt(u1, 0u, 0x4140u), prmt(u1, 0u, 0x4342u));
                    sc[0] = fmaf(ks[0], fmaf(c[0], 16777216.0f, -128.0f * qsum[kp]), sc[0]);
                    sc[1] = fmaf(ks[1], fmaf(c[1], 16777216.0f, -128.0f * qsum[kp]), sc[1]);
                    zz2 = c[2];
                    zz3 = c[3];
                }
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool valid = tok0 + 8 * tb + 2 * t + e < t1;
                s[tb][e] = valid ? sc[e] * A.scale_log2 : NEG_BIG;
            }
        }
        // ---------------- online softmax for head g
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
                p[tb][e] = s[tb][e] > 0.5f * NEG_BIG ? exp2f(s[tb][e] - m_new) : 0.f;
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
        int vtok[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) vtok[i] = min(tok0 + (i >> 1) * 8 + 2 * t + (i & 1), t1 - 1);
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
            uint32_t b0[4], b1[4];
            if (!PAGED) {
                uint2 w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half* vrow = (owner && vtok[i] == pos) ? S->v : static_cast<const __half*>(A.kv.v0) + (head_row + vtok[i]) * AD;
                    w[i] = *reinterpret_cast<const uint2*>(vrow + 32 * kp + 4 * g);
                }
                b0[0] = prmt(w[0].x, w[1].x, 0x5410u); b0[1] = prmt(w[0].x, w[1].x, 0x7632u);
                b0[2] = prmt(w[0].y, w[1].y, 0x5410u); b0[3] = prmt(w[0].y, w[1].y, 0x7632u);
                b1[0] = prmt(w[2].x, w[3].x, 0x5410u); b1[1] = prmt(w[2].x, w[3].x, 0x7632u);
                b1[2] = prmt(w[2].y, w[3].y, 0x5410u); b1[3] = prmt(w[2].y, w[3].y, 0x7632u);
            } else {
                uint32_t w[4];
                float vs[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint8_t* row = vslab + ((i >> 1) * 8 + 2 * t + (i & 1)) * (NKP * KV_BLOCK_BYTES) + kp * KV_BLOCK_BYTES;
                    uint32_t dummy;
                    lds_words_align2(row + 2 + 4 * g, w[i], dummy, false);
                    vs[i] = tok0 + (i >> 1) * 8 + 2 * t + (i & 1) < t1 ? half_bits_to_f32(lds16g(row)) : 0.f;
                    w[i] ^= 0x80808080u;
                }
                const uint32_t lo01 = prmt(w[0], w[1], 0x5140u), hi01 = prmt(w[0], w[1], 0x7362u);
                const uint32_t lo23 = prmt(w[2], w[3], 0x5140u), hi23 = prmt(w[2], w[3], 0x7362u);
                const uint32_t T[4] = {prmt(lo01, lo23, 0x5410u), prmt(lo01, lo23, 0x7632u),
                                       prmt(hi01, hi23, 0x5410u), prmt(hi01, hi23, 0x7632u)};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    b0[e] = prmt(T[e], 0u, 0x4140u);
                    b1[e] = prmt(T[e], 0u, 0x4342u);
                }
                const float f0 = pb[0] * vs[0], f1 = pb[1] * vs[1], f2 = pb[2] * vs[2], f3 = pb[3] * vs[3];
                pa0 = pack_h2(f0, f1);
                pa2 = pack_h2(f2, f3);
                const float2 r0 = unpack_h2(pa0), r2 = unpack_h2(pa2);
                pl0 = pack_h2(f0 - r0.x, f1 - r0.y);
                pl2 = pack_h2(f2 - r2.x, f3 - r2.y);
                const float2 q0 = unpack_h2(pl0), q2 = unpack_h2(pl2);
                ocorr[kp] += ((r0.x + r0.y) + (r2.x + r2.y)) + ((q0.x + q0.y) + (q2.x + q2.y));
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (PAGED) {
                    float c[4] = {0.f, 0.f, zz2, zz3};
                    mma8(c, pa0, pa2, b0[e], b1[e]);
                    mma8(c, pl0, pl2, b0[e], b1[e]);
                    o[kp * 4 + e][0] += c[0];
                    o[kp * 4 + e][1] += c[1];
                    zz2 = c[2];
                    zz3 = c[3];
                } else {
                    float c[4] = {o[kp * 4 + e][0], o[kp * 4 + e][1], zz2, zz3};
                    mma8(c, pa0, pa2, b0[e], b1[e]);
                    mma8(c, pl0, pl2, b0[e], b1[e]);
                    o[kp * 4 + e][0] = c[0];
                    o[kp * 4 + e][1] = c[1];
                    zz2 = c[2];
                    zz3 = c[3];
                }
            }
        }
        __syncwarp();
    }

    // ---- this warp's state -> shared memory
    if (PAGED) {
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
    __syncthreads();                                   // every warp is done with its page stages
    float (*sm_o)[8][AD] = reinterpret_cast<float (*)[8][AD]>(ring_area);      // [WARPS][8][128] floats = 64 KB
    if (t == 0) { S->m[warp][g] = m_run; S->l[warp][g] = l_run; }
#pragma unroll
    for (int kp = 0; kp < NKP; ++kp)
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int c = 0; c < 2; ++c) sm_o[warp][g][32 * kp + 4 * (2 * t + c) + e] = o[kp * 4 + e][c];
    __syncthreads();

    // ---- merge the warps, write the split's partial, let the last CTA of the head combine the splits
    if (threadIdx.x < G) {
        const int hg = threadIdx.x;
        float mx = NEG_BIG;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, S->m[w][hg]);
        float sc[WARPS], lt = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            sc[w] = exp2f(S->m[w][hg] - mx);
            lt = fmaf(S->l[w][hg], sc[w], lt);
        }
        const float inv = lt > 0.f ? 1.0f / lt : 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) S->l[w][hg] = sc[w] * inv;
        A.part_lse[static_cast<int64_t>(kvh * G + hg) * A.splits + split] = lt > 0.f ? mx + log2f(lt) : NEG_BIG;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * (AD / 4); i += WARPS * 32) {
        const int hg = i / (AD / 4), dd = (i - hg * (AD / 4)) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = S->l[w][hg];
            const float4 v = *reinterpret_cast<const float4*>(&sm_o[w][hg][dd]);
            acc.x = fmaf(v.x, f, acc.x);
            acc.y = fmaf(v.y, f, acc.y);
            acc.z = fmaf(v.z, f, acc.z);
            acc.w = fmaf(v.w, f, acc.w);
        }
        const int64_t pi = static_cast<int64_t>(kvh * G + hg) * A.splits + split;
        *reinterpret_cast<float4*>(A.part_o + pi * AD + dd) = acc;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(A.counters + kvh, 1u);
        S->last = (prev == static_cast<unsigned int>(A.splits) - 1u);
        if (S->last) A.counters[kvh] = 0u;
    }
    __syncthreads();
    if (!S->last) return;
    __threadfence();
    for (int hg = warp; hg < G; hg += WARPS) {
        const float* lse = A.part_lse + static_cast<int64_t>(kvh * G + hg) * A.splits;
        const float l0 = lane < A.splits ? __ldcg(lse + lane) : NEG_BIG;
        const float l1 = lane + 32 < A.splits ? __ldcg(lse + lane + 32) : NEG_BIG;
        const float mx = warp_max(fmaxf(l0, l1));
        const float e0 = l0 > 0.5f * NEG_BIG ? exp2f(l0 - mx) : 0.f;
        const float e1 = l1 > 0.5f * NEG_BIG ? exp2f(l1 - mx) : 0.f;
        const float sum = warp_sum(e0 + e1);
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
        if (lane < A.splits) S->wgt[hg * A.splits + lane] = e0 * inv;
        if (lane + 32 < A.splits) S->wgt[hg * A.splits + lane + 32] = e1 * inv;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * (AD / 4); i += WARPS * 32) {
        const int hg = i / (AD / 4), dd = (i - hg * (AD / 4)) * 4;
        const int h = kvh * G + hg;
        const float4* po = reinterpret_cast<const float4*>(A.part_o + static_cast<int64_t>(h) * A.splits * AD + dd);
        const float* w = S->wgt + hg * A.splits;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int s2 = 0;
        for (; s2 + 8 <= A.splits; s2 += 8) {              // eight independent loads in flight
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(po + static_cast<int64_t>(s2 + u) * (AD / 4));
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                acc.x = fmaf(w[s2 + u], v[u].x, acc.x);
                acc.y = fmaf(w[s2 + u], v[u].y, acc.y);
                acc.z = fmaf(w[s2 + u], v[u].z, acc.z);
                acc.w = fmaf(w[s2 + u], v[u].w, acc.w);
            }
        }
        for (; s2 < A.splits; ++s2) {
            const float4 v = __ldcg(po + static_cast<int64_t>(s2) * (AD / 4));
            acc.x = fmaf(w[s2], v.x, acc.x);
            acc.y = fmaf(w[s2], v.y, acc.y);
            acc.z = fmaf(w[s2], v.z, acc.z);
            acc.w = fmaf(w[s2], v.w, acc.w);
        }
        __half2* dst = reinterpret_cast<__half2*>(A.out + static_cast<int64_t>(h) * AD + dd);
        dst[0] = __floats2half2_rn(acc.x, acc.y);
        dst[1] = __floats2half2_rn(acc.z, acc.w);
    }
}

// ------------------------------------------------------------------------------------ the kernel

__global__ void __launch_bounds__(WARPS * 32, 1) decode_layers_kernel(const StepDesc sd) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* red_all = reinterpret_cast<float*>(smem + OFF_RED);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    __half* xs = reinterpret_cast<__half*>(smem + OFF_XS);
    float* sums = reinterpret_cast<float*>(smem + OFF_SUMS);
    float* nred = reinterpret_cast<float*>(smem + OFF_NRED);
    RingState rs;
    rs.ring = smem_u32(smem + warp * RING_WARP);
    rs.bar0 = smem_u32(bars + warp * MAX_D);
    rs.parity = 0u;
    rs.ok = true;
    if (lane == 0) {
        for (int s = 0; s < MAX_D; ++s) mbar_init(rs.bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    pdl_launch_dependents();

    // Phase descriptors live in global memory; a CTA works from copies in shared memory (three slots):
    // the row cursors and the copy issue read them all the time, and with this much shared memory in
    // use L1 is too small to serve that.  A descriptor is loaded two phases ahead (one word per
    // thread, held in a register) and stored one phase ahead, so the load's latency is never waited for.
    constexpr int DESC_WORDS = static_cast<int>(sizeof(PhaseDesc) / 4);
    auto slot_of = [&](int ph) { return reinterpret_cast<const PhaseDesc*>(smem + OFF_DESC + (ph % DESC_SLOTS) * DESC_SLOT); };
    auto load_word = [&](int ph) -> uint32_t {
        return (ph < sd.n_phases && threadIdx.x < DESC_WORDS) ? __ldg(reinterpret_cast<const uint32_t*>(sd.phases + ph) + threadIdx.x) : 0u;
    };
    auto store_word = [&](int ph, uint32_t w) {
        if (ph < sd.n_phases && threadIdx.x < DESC_WORDS)
            reinterpret_cast<uint32_t*>(smem + OFF_DESC + (ph % DESC_SLOTS) * DESC_SLOT)[threadIdx.x] = w;
    };
    unsigned int target = 0;
    Plan& pl = *reinterpret_cast<Plan*>(smem + OFF_PLAN + warp * PLAN_SLOT);
    store_word(0, load_word(0));
    store_word(1, load_word(1));
    uint32_t pending = load_word(2);
    __syncthreads();
    if (slot_of(0)->type == PH_GEMV) gemv_begin(pl, slot_of(0)->g, sd.maps, rs, warp, lane);
    pdl_wait();
    for (int ph = 0; ph < sd.n_phases; ++ph) {
        __syncthreads();                               // every warp has left phase ph - 1
        if (ph >= 1) {
            store_word(ph + 1, pending);
            pending = load_word(ph + 2);
        }
        const PhaseDesc& pd = *slot_of(ph);
        auto stamp = [&](int k) {
            if (sd.trace && threadIdx.x == 0) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                sd.trace[(static_cast<size_t>(ph) * gridDim.x + blockIdx.x) * 4 + k] = t;
            }
        };
        if (pd.type == PH_GEMV) {
            if (pd.g.stage_x) stage_token(pd.g, xs, sums, nred);
            else __syncthreads();
            // the descriptor of phase ph + 1 is readable now: let the TMA unit fetch its tensor maps
            // ahead of the first copy (they live in global memory; an un-fetched map stalls the issue)
            if (ph + 1 < sd.n_phases && threadIdx.x < MAX_SEG) {
                const PhaseDesc& nx = *slot_of(ph + 1);
                if (nx.type == PH_GEMV && nx.g.seg[threadIdx.x].data)
                    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(sd.maps + nx.g.seg[threadIdx.x].map)) : "memory");
            }
            stamp(0);
            gemv_run(pl, pd.g, sd.maps, rs, xs, sums, red_all, warp, lane);
        } else {
            __syncthreads();
            if (ph + 1 < sd.n_phases && threadIdx.x < MAX_SEG) {
                const PhaseDesc& nx = *slot_of(ph + 1);
                if (nx.type == PH_GEMV && nx.g.seg[threadIdx.x].data)
                    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(sd.maps + nx.g.seg[threadIdx.x].map)) : "memory");
            }
            stamp(0);
            AttnSmem* S = reinterpret_cast<AttnSmem*>(xs);
            if (pd.a.layout == ALLOYB_KV_F16) attn_phase<ALLOYB_KV_F16>(pd.a, rs, smem, S, warp, lane);
            else attn_phase<ALLOYB_KV_Q8_PAGED>(pd.a, rs, smem, S, warp, lane);
        }
        const int barrier_after = pd.barrier_after;
        stamp(1);
        if (ph + 1 < sd.n_phases) {
            const PhaseDesc& nx = *slot_of(ph + 1);
            if (nx.type == PH_GEMV) {
                // the next phase's first weight copies go out before the barrier (the attention phase
                // uses the ring area for its own staging, so nothing is prefetched across it)
                if (pd.type == PH_ATTN) __syncthreads();
                gemv_begin(pl, nx.g, sd.maps, rs, warp, lane);
            }
        }
        stamp(2);
        if (barrier_after) grid_sync(sd.barrier, target);
        stamp(3);
    }
}

}  // namespace dl
}  // namespace alloyb

// ------------------------------------------------------------------------------------ host side

namespace alloyb {
namespace dl {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn encoder() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
            qr != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

struct Decoder {
    int device = 0;
    int sms = 0;
    StepDesc step = {};
    void* dev_block = nullptr;           // one allocation: phases | maps | scratch
    int n_phases = 0;
    int32_t* status = nullptr;
    unsigned long long* trace = nullptr;   // 2 * n_phases timestamps, filled when tracing is on
};

struct Builder {
    std::vector<PhaseDesc> phases;
    std::vector<CUtensorMap> maps;
    int sms;
    int rc = ALLOYB_OK;

    // One GEMV phase over matrices (Q4_K and Q6_K may be mixed) that share the token x (K elements).
    void gemv(const __half* x, int K, const __half* norm_w, float eps, const alloyb_matrix* const* m, void* const* y,
              int n_m, bool gated, const __half* residual, const alloyb_tp* tp, bool stage_x, bool barrier_after) {
        if (rc != ALLOYB_OK) return;
        PhaseDesc pd = {};
        pd.type = PH_GEMV;
        pd.barrier_after = barrier_after ? 1 : 0;
        GemvDesc& g = pd.g;
        if (K % QK_K || K > XS_HALVES || n_m < 1 || n_m > MAX_SEG) { rc = ALLOYB_E_SHAPE; return; }
        const int nsb = K / QK_K;
        int64_t rows = 0;
        bool any_q6 = false;
        for (int i = 0; i < n_m; ++i) {
            if (m[i]->format != ALLOYB_Q4_K && m[i]->format != ALLOYB_Q6_K) { rc = ALLOYB_E_SHAPE; return; }
            any_q6 |= m[i]->format == ALLOYB_Q6_K;
            if (!gated || i == 0) rows += m[i]->N;
        }
        // the grouping rules of the stand-alone streaming kernel (linear_stream.cu)
        int gw = (rows / 16 >= static_cast<int64_t>(2) * WARPS * sms) ? 1 : (nsb >= 8 ? 8 : (nsb >= 4 ? 4 : 0));
        const int tiles_per_cta = static_cast<int>((rows + 16 * sms - 1) / (16 * sms));
        if (gw == 8 && !gated && nsb >= 16 && nsb % 16 == 0 && (tiles_per_cta == 1 || tiles_per_cta == 3)) gw = 16;
        if (gw == 0 || (gated && (gw != 8 || any_q6 || n_m != 2 || m[0]->N != m[1]->N))) { rc = ALLOYB_E_SHAPE; return; }
        if (tp && (gated || n_m != 1)) { rc = ALLOYB_E_SHAPE; return; }
        const int sbs = (!any_q6 && nsb % (2 * gw) == 0) ? 2 : 1;
        g.x = x;
        g.residual = residual;
        g.norm_w = norm_w;
        g.eps = eps;
        g.n_seg = gated ? 1 : n_m;
        g.nsb = nsb;
        g.gu = gated ? 1 : 0;
        g.act = ALLOYB_ACT_SILU;
        g.gw = gw;
        g.sbs = sbs;
        g.stage_x = stage_x ? 1 : 0;
        g.K = K;
        if (tp) {
            g.tp.world = tp->world;
            g.tp.rank = tp->rank;
            g.tp.max_n = tp->max_n;
            g.tp.spin = tp->spin_limit > 0 ? static_cast<uint32_t>(tp->spin_limit) : SPIN_LIMIT;
            for (int r = 0; r < tp->world; ++r) g.tp.peer[r] = static_cast<uint8_t*>(tp->peer[r]);
        }
        const EncodeFn encode = encoder();
        if (!encode) { set_cuda_error(cudaErrorNotSupported); rc = ALLOYB_E_CUDA; return; }
        int64_t base = 0;
        int slot_bytes = 0;
        for (int i = 0; i < n_m; ++i) {
            const alloyb_matrix& a = *m[i];
            const int kind = a.format == ALLOYB_Q6_K ? Q6 : (sbs == 2 ? Q4x2 : Q4x1);
            const int blk = kind == Q6 ? Q6K_BYTES : Q4K_BYTES;
            const int pitch = kind == Q6 ? Geom<Q6>::PITCH : (kind == Q4x2 ? Geom<Q4x2>::PITCH : Geom<Q4x1>::PITCH);
            const int64_t rb = a.row_bytes ? a.row_bytes : static_cast<int64_t>(nsb) * blk;
            if (a.N <= 0 || !a.data || rb < static_cast<int64_t>(nsb) * blk) { rc = ALLOYB_E_SHAPE; return; }
            if (reinterpret_cast<uintptr_t>(a.data) % 16 || rb % 16) { rc = ALLOYB_E_ALIGN; return; }
            GSeg& sg = g.seg[i];
            sg.data = static_cast<const uint8_t*>(a.data);
            sg.row_bytes = rb;
            sg.y = y[gated ? 0 : i];
            sg.n_rows = a.N;
            sg.row_base = gated ? 0 : static_cast<int>(base);
            sg.kind = kind;
            sg.map = static_cast<int>(maps.size());
            if (16 * pitch > slot_bytes) slot_bytes = 16 * pitch;
            if (!gated || i == 0) base += a.N;
            CUtensorMap tm;
            const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(rb) / 4, static_cast<cuuint64_t>(a.N)};
            const cuuint64_t gstr[1] = {static_cast<cuuint64_t>(rb)};
            const cuuint32_t box[2] = {static_cast<cuuint32_t>(pitch / 4), 16};
            const cuuint32_t estr[2] = {1, 1};
            if (encode(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(a.data), gdim, gstr, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
                set_cuda_error(cudaErrorInvalidValue);
                rc = ALLOYB_E_CUDA;
                return;
            }
            maps.push_back(tm);
        }
        g.slot_bytes = slot_bytes;
        g.depth = RING_WARP / slot_bytes > 3 ? 3 : RING_WARP / slot_bytes;
        g.total_rows = static_cast<int>(base);
        phases.push_back(pd);
    }
};

}  // namespace dl
}  // namespace alloyb

using namespace alloyb;

extern "C" int alloyb_decoder_create(const alloyb_decoder_desc* d, void** handle) {
    using namespace dl;
    if (!d || !handle || !d->layers || !d->norm_final || !d->inv_freq || !d->pos || !d->hidden_io || !d->logits)
        return ALLOYB_E_NULL;
    if (d->n_layers <= 0 || d->hidden <= 0 || d->ffn <= 0 || d->heads <= 0 || d->kv_heads <= 0 || d->heads % d->kv_heads)
        return ALLOYB_E_SHAPE;
    const int G = d->heads / d->kv_heads;
    if (d->head_dim != AD || G > 8) return ALLOYB_E_SHAPE;
    if (d->kv_layout != ALLOYB_KV_F16 && d->kv_layout != ALLOYB_KV_Q8_PAGED) return ALLOYB_E_SHAPE;
    if (d->S_max <= 0 || (d->kv_layout == ALLOYB_KV_Q8_PAGED && (d->S_max % PAGE_TOKENS || d->num_pages <= 0)))
        return ALLOYB_E_SHAPE;
    if (d->tp && (d->tp->world < 1 || d->tp->world > 8 || d->tp->rank < 0 || d->tp->rank >= d->tp->world ||
                  d->hidden > d->tp->max_n))
        return ALLOYB_E_SHAPE;
    Decoder* dec = new (std::nothrow) Decoder();
    if (!dec) return ALLOYB_E_CUDA;
    cudaError_t e = cudaGetDevice(&dec->device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&dec->sms, cudaDevAttrMultiProcessorCount, dec->device);
    if (e != cudaSuccess || dec->sms <= 0) { delete dec; set_cuda_error(e); return ALLOYB_E_CUDA; }

    // scratch: q | k | v | attention out | gated activations | split partials | counters, status, barrier
    const int qd = d->heads * AD, kvd = d->kv_heads * AD;
    int splits = dec->sms / d->kv_heads;
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;
    if (splits < 1) splits = 1;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    const size_t o_q = 0, o_k = o_q + up(qd * 2), o_v = o_k + up(kvd * 2), o_a = o_v + up(kvd * 2), o_act = o_a + up(qd * 2),
                 o_po = o_act + up(static_cast<size_t>(d->ffn) * 2),
                 o_pl = o_po + up(static_cast<size_t>(d->heads) * splits * AD * 4),
                 o_ctr = o_pl + up(static_cast<size_t>(d->heads) * splits * 4),
                 o_trace = o_ctr + 1024,
                 scratch_bytes = o_trace + up(static_cast<size_t>(d->n_layers * 5 + 2) * dec->sms * 4 * 8);

    Builder b;
    b.sms = dec->sms;
    const __half* h = static_cast<const __half*>(d->hidden_io);
    // placeholders for scratch addresses until the block is allocated: offsets from a null base
    uint8_t* const S0 = nullptr;
    const alloyb_tp* tp = (d->tp && d->tp->world > 1) ? d->tp : nullptr;
    for (int li = 0; li < d->n_layers; ++li) {
        const alloyb_decoder_layer& L = d->layers[li];
        if (!L.norm_in || !L.norm_post || !L.k0) { b.rc = ALLOYB_E_NULL; break; }
        // q, k, v: one phase (formats may differ; the token is staged and normalised once)
        const alloyb_matrix* qkv[3] = {&L.wq, &L.wk, &L.wv};
        void* qkv_y[3] = {S0 + o_q, S0 + o_k, S0 + o_v};
        b.gemv(h, d->hidden, static_cast<const __half*>(L.norm_in), d->eps, qkv, qkv_y, 3, false, nullptr, nullptr, true, true);
        if (L.wq.N != qd || L.wk.N != kvd || L.wv.N != kvd) b.rc = ALLOYB_E_SHAPE;
        if (b.rc != ALLOYB_OK) break;
        // attention
        {
            PhaseDesc pd = {};
            pd.type = PH_ATTN;
            pd.barrier_after = 1;
            AttnDesc& A = pd.a;
            A.q = reinterpret_cast<const __half*>(S0 + o_q);
            A.k = reinterpret_cast<const __half*>(S0 + o_k);
            A.v = reinterpret_cast<const __half*>(S0 + o_v);
            A.out = reinterpret_cast<__half*>(S0 + o_a);
            A.layout = d->kv_layout;
            A.kv.k0 = L.k0; A.kv.k1 = L.k1; A.kv.v0 = L.v0; A.kv.v1 = L.v1;
            A.kv.S_max = d->S_max;
            A.kv.max_pages = d->S_max / PAGE_TOKENS;
            A.kv.num_pages = d->num_pages;
            if (d->kv_layout == ALLOYB_KV_F16 ? !L.v0 : !L.k1) { b.rc = ALLOYB_E_NULL; break; }
            A.pos = d->pos;
            A.inv_freq = d->inv_freq;
            A.H = d->heads; A.KV_H = d->kv_heads; A.G = G; A.splits = splits;
            A.scale_log2 = (1.0f / sqrtf(static_cast<float>(AD))) * 1.4426950408889634f;
            A.part_o = reinterpret_cast<float*>(S0 + o_po);
            A.part_lse = reinterpret_cast<float*>(S0 + o_pl);
            A.counters = reinterpret_cast<unsigned int*>(S0 + o_ctr);
            A.status = reinterpret_cast<int*>(S0 + o_ctr + 512);
            b.phases.push_back(pd);
        }
        // o_proj (+ residual, + exchange), gate/up (norm, SiLU), down (+ residual, + exchange)
        const alloyb_matrix* mo[1] = {&L.wo};
        void* yo[1] = {d->hidden_io};
        b.gemv(reinterpret_cast<const __half*>(S0 + o_a), qd, nullptr, 0.f, mo, yo, 1, false, h, tp, true, true);
        const alloyb_matrix* mg[2] = {&L.wg, &L.wu};
        void* yg[2] = {S0 + o_act, S0 + o_act};
        b.gemv(h, d->hidden, static_cast<const __half*>(L.norm_post), d->eps, mg, yg, 2, true, nullptr, nullptr, true, true);
        const alloyb_matrix* md[1] = {&L.wd};
        b.gemv(reinterpret_cast<const __half*>(S0 + o_act), d->ffn, nullptr, 0.f, md, yo, 1, false, h, tp, true, true);
        if (L.wo.N != d->hidden || L.wd.N != d->hidden || L.wg.N != d->ffn) b.rc = ALLOYB_E_SHAPE;
        if (b.rc != ALLOYB_OK) break;
    }
    if (b.rc == ALLOYB_OK) {
        const alloyb_matrix* mh[1] = {&d->head};
        void* yh[1] = {d->logits};
        b.gemv(h, d->hidden, static_cast<const __half*>(d->norm_final), d->eps, mh, yh, 1, false, nullptr, nullptr, true, false);
    }
    if (b.rc != ALLOYB_OK) { const int rc = b.rc; delete dec; return rc; }

    const size_t ph_bytes = up(b.phases.size() * sizeof(PhaseDesc)), map_bytes = up(b.maps.size() * sizeof(CUtensorMap));
    e = cudaMalloc(&dec->dev_block, ph_bytes + map_bytes + scratch_bytes);
    if (e != cudaSuccess) { delete dec; set_cuda_error(e); return ALLOYB_E_CUDA; }
    uint8_t* base = static_cast<uint8_t*>(dec->dev_block);
    uint8_t* scratch = base + ph_bytes + map_bytes;
    // scratch pointers were recorded as offsets from a null base: rebase them
    auto fix = [&](const void* p) -> void* {
        const uintptr_t v = reinterpret_cast<uintptr_t>(p);
        return v < scratch_bytes ? static_cast<void*>(scratch + v) : const_cast<void*>(p);
    };
    for (PhaseDesc& pd : b.phases) {
        if (pd.type == PH_GEMV) {
            GemvDesc& g = pd.g;
            g.x = static_cast<const __half*>(fix(g.x));
            for (int i = 0; i < MAX_SEG; ++i)
                if (g.seg[i].data) g.seg[i].y = fix(g.seg[i].y);
        } else {
            AttnDesc& A = pd.a;
            A.q = static_cast<const __half*>(fix(A.q));
            A.k = static_cast<const __half*>(fix(A.k));
            A.v = static_cast<const __half*>(fix(A.v));
            A.out = static_cast<__half*>(fix(A.out));
            A.part_o = static_cast<float*>(fix(A.part_o));
            A.part_lse = static_cast<float*>(fix(A.part_lse));
            A.counters = static_cast<unsigned int*>(fix(A.counters));
            A.status = static_cast<int*>(fix(A.status));
        }
    }
    e = cudaMemcpy(base, b.phases.data(), b.phases.size() * sizeof(PhaseDesc), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(base + ph_bytes, b.maps.data(), b.maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(scratch, 0, scratch_bytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(decode_layers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { cudaFree(dec->dev_block); delete dec; set_cuda_error(e); return ALLOYB_E_CUDA; }
    dec->step.phases = reinterpret_cast<const PhaseDesc*>(base);
    dec->step.n_phases = static_cast<int>(b.phases.size());
    dec->step.maps = reinterpret_cast<const CUtensorMap*>(base + ph_bytes);
    dec->step.barrier = reinterpret_cast<unsigned int*>(scratch + o_ctr + 768);
    dec->status = reinterpret_cast<int32_t*>(scratch + o_ctr + 512);
    dec->n_phases = dec->step.n_phases;
    dec->trace = reinterpret_cast<unsigned long long*>(scratch + o_trace);
    dec->step.trace = nullptr;
    *handle = dec;
    return ALLOYB_OK;
}

extern "C" int alloyb_decoder_step(void* handle, void* stream) {
    using namespace dl;
    if (!handle) return ALLOYB_E_NULL;
    Decoder* dec = static_cast<Decoder*>(handle);
    cudaStream_t st = as_stream(stream);
    cudaError_t e = cudaMemsetAsync(dec->step.barrier, 0, sizeof(unsigned int), st);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(dec->sms);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;       // every CTA must be resident: they meet at barriers
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, decode_layers_kernel, dec->step);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

// Diagnostic: with tracing on, every CTA records four nanosecond clocks per phase (token staged, phase
// done, next phase's copies issued, barrier passed); alloyb_decoder_trace_read copies the
// phases x CTAs x 4 values of the last step.
extern "C" int alloyb_decoder_trace(void* handle, int on) {
    if (!handle) return ALLOYB_E_NULL;
    dl::Decoder* dec = static_cast<dl::Decoder*>(handle);
    dec->step.trace = on ? dec->trace : nullptr;
    return ALLOYB_OK;
}
extern "C" int alloyb_decoder_trace_read(void* handle, uint64_t* out, int n_values) {
    if (!handle || !out) return ALLOYB_E_NULL;
    dl::Decoder* dec = static_cast<dl::Decoder*>(handle);
    if (n_values < 0 || n_values > 4 * dec->n_phases * dec->sms) return ALLOYB_E_SHAPE;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(out, dec->trace, static_cast<size_t>(n_values) * 8, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

extern "C" int alloyb_decoder_phases(void* handle) {
    return handle ? static_cast<dl::Decoder*>(handle)->n_phases : ALLOYB_E_NULL;
}

extern "C" int alloyb_decoder_status(void* handle, int32_t* status_out, void* stream) {
    if (!handle || !status_out) return ALLOYB_E_NULL;
    dl::Decoder* dec = static_cast<dl::Decoder*>(handle);
    cudaError_t e = cudaMemcpyAsync(status_out, dec->status, sizeof(int32_t), cudaMemcpyDeviceToHost, as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

extern "C" int alloyb_decoder_destroy(void* handle) {
    if (!handle) return ALLOYB_OK;
    dl::Decoder* dec = static_cast<dl::Decoder*>(handle);
    const cudaError_t e = cudaFree(dec->dev_block);
    delete dec;
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

namespace alloyb {
int decode_layer_device_error(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, st::g_error, sizeof(int)) != cudaSuccess) return 0;
    if (clear && v) {
        const int z = 0;
        cudaMemcpyToSymbol(st::g_error, &z, sizeof(int));
    }
    return v;
}
}  // namespace alloyb

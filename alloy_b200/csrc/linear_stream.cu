// One-token dequant-GEMV as a persistent streaming kernel (fp16 activations, Q4_K / Q6_K weights).
//
// The decode step multiplies ONE token by every weight matrix, so the kernel's only job is to
// pull packed rows out of HBM at full speed and to spend as few instructions per byte as it can.
//
// Work split.  One CTA per SM.  The output rows of a launch (all row-stacked matrices together)
// are cut into one contiguous range per CTA, equal to within one row, so every SM streams the same
// number of bytes; a CTA walks its range in 16-row tiles (the last tile of a range or of a matrix
// is partial) and deals the tiles round-robin to its GROUPS of eight warps.  Inside a tile the K
// dimension is cut into eight slices of whole super-blocks, one per warp of the group, the same
// slice for every tile: a warp's activations (as MMA B fragments) and their per-sub-block sums
// are loop invariants and live in registers when the slice is one stage long.
//
// Data movement.  Every warp has a PRIVATE ring of slots (16 rows x one or two 144-byte
// super-blocks) with one mbarrier per slot.  A full tile's slot is filled by ONE 2-D TMA copy out
// of the row-major packed matrix; a partial tile by one plain bulk copy per valid row.  The warp
// refills a slot as soon as it has drained it, across tile boundaries, with no producer warp and
// no CTA-wide barrier on the load path.  The ring is kept SHALLOW (one or two slots in flight per
// warp): HBM delivers its peak with ~75 KB in flight per SM, and deeper queues of small strided
// boxes measurably lose row-buffer locality.  Weight copies do not depend on the previous kernel
// and start before griddepcontrol.wait.
//
// Arithmetic.  mma.sync.m16n8k16 with the 16 rows as M and the eight MMA columns used for the
// eight SUB-BLOCKS of a super-block (the B operand carries the token's activations of sub-block n
// in column n, zero elsewhere).  The A operand is the raw nibbles as fp16 subnormals (n * 2^-24,
// high nibbles as 16n * 2^-24; one shift and four ANDs per 32-bit word give four A registers), so
// after sixteen MMAs the accumulator tile holds  sum nib*x  per (row, sub-block) and the 6-bit
// scales and mins are applied to eight numbers per lane.  Exact products, fp32 accumulation: the
// factored form  sum_g d*sc_g*(sum nib*x) - dmin*m_g*(sum x)  of the reference's GEMV
// (metal/std/quant.py:1312-1347).
//
// One group-wide named barrier per tile folds the eight K slices (double-buffered partials in
// shared memory); 16 threads apply the activation / residual and store.
#include "linear_stream.cuh"

namespace alloyb {
namespace st {

// KIND: slot geometry / weight format.  RT: matrices per tile (2 = gate/up pair).  CACHE: the warp's
// slice is exactly one slot long and its B fragments stay in registers for the whole launch.
// GU: gate/up pair with the two matrices dealt to the two groups (group 0 streams gate rows, group 1
// the up rows of the SAME tiles, RT = 1 each), so both groups do the same work whatever the tile count.
template <int KIND, int RT, bool CACHE, int GW, bool GU = false>
__global__ void __launch_bounds__(WARPS * 32, 1)
gemv_stream_kernel(const __grid_constant__ Maps maps, const Params P) {
    constexpr int SBS = Geom<KIND>::SBS, PITCH = Geom<KIND>::PITCH, SLOT = 16 * PITCH, BLK = Geom<KIND>::BLK;
    constexpr bool MIX = KIND == QMIX;             // Q4_K tiles (two super-blocks per slot) first, Q6_K tiles after them
    static_assert(!MIX || (RT == 1 && !GU && GW > 1), "mixed formats: plain linears with a K split");
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int grp = warp / GW, wg = warp % GW;
    constexpr int n_warps = WARPS, n_groups = WARPS / GW;
    static_assert(!GU || (RT == 1 && GW == 8), "gate/up split: two groups of eight warps");
    constexpr int tstep = GU ? 1 : n_groups;                        // tiles between two of this group's tiles
    const int D = P.depth;
    // [warps][D] slots | [groups][2][GW][RT][16] partials | [warps][MAX_D] barriers
    float* red_all = reinterpret_cast<float*>(smem + n_warps * D * SLOT);
    float* red = red_all + grp * (2 * GW * RT * 16);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + n_warps * D * SLOT + n_groups * 2 * GW * RT * 16 * 4);
    const uint32_t ring = smem_u32(smem + warp * D * SLOT);
    const uint32_t bar0 = smem_u32(bars + warp * MAX_D);
    const int xs_off = n_warps * D * SLOT + n_groups * 2 * GW * RT * 16 * 4 + n_warps * MAX_D * 8;      // 16-byte aligned

    if (threadIdx.x < (P.gated ? 2 : P.n_seg))        // the TMA unit fetches the descriptors ahead of the first copy
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.m[threadIdx.x])) : "memory");
    if (lane == 0) {
        for (int s = 0; s < D; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    pdl_launch_dependents();

    // this CTA's rows (whole 16-row tiles of the stacked row space: a tile split between two CTAs would cost
    // both of them a full tile's work), this group's tiles (every n_groups-th), this warp's K slice
    constexpr int GRAIN = MIX ? 16 * Q6_ROW_COST : 16;
    const int grains = (P.total_rows + GRAIN - 1) / GRAIN;
    const int lo = static_cast<int>(static_cast<int64_t>(grains) * blockIdx.x / gridDim.x) * GRAIN;
    const int hi_g = static_cast<int>(static_cast<int64_t>(grains) * (blockIdx.x + 1) / gridDim.x) * GRAIN;
    const int hi = hi_g < P.total_rows ? hi_g : P.total_rows;
    // super-blocks [sb_lo, sb_lo + slice) of every tile; slices differ by at most one super-block
    // when GW does not divide the count (one-super-block slots only)
    const int sb_lo = (wg * P.nsb) / GW;
    const int slice = ((wg + 1) * P.nsb) / GW - sb_lo;
    // stages per tile (a Q6_K tile of a mixed launch has one super-block per slot)
    auto spt_of = [&](int seg) { return (MIX && P.seg[seg].q6) ? slice : (slice / SBS) * RT; };
    int my_tiles = 0, n_stage = 0;
    {
        Cursor c = {0, 0, 0};
        cursor_enter<MIX>(c, P, lo, hi);
        cursor_next<MIX>(c, P, lo, hi, GU ? 0 : grp);
        while (c.seg < P.n_seg) {
            ++my_tiles;
            n_stage += spt_of(c.seg);
            cursor_next<MIX>(c, P, lo, hi, tstep);
        }
    }

    // producer side: stage sequence = for tile, for slot-sized step of the slice, for matrix
    Cursor pc = {0, 0, 0};
    cursor_enter<MIX>(pc, P, lo, hi);
    cursor_next<MIX>(pc, P, lo, hi, GU ? 0 : grp);
    int issued = 0, p_r = 0, p_slot = 0;
    auto issue = [&]() {
        // the geometry of this stage's tile (fixed by KIND unless the launch mixes formats)
        const bool six = KIND == Q6 || (MIX && P.seg[pc.seg].q6);
        const int sbs = MIX ? (six ? 1 : 2) : SBS, blk = MIX ? (six ? Q6K_BYTES : Q4K_BYTES) : BLK;
        const int pitch = MIX ? (six ? Geom<Q6>::PITCH : Geom<Q4x2>::PITCH) : PITCH;
        const int sb = sb_lo + (p_r / RT) * sbs, mt = p_r % RT;
        const int si = GU ? grp : (P.gated ? mt : pc.seg);
        const uint32_t bar = bar0 + 8 * p_slot, dst = ring + p_slot * SLOT;
        const int win = (sb * blk) & ~15;                            // 16-byte-aligned start of the stage in a row
        // one box of sixteen rows, also for the last tile of a matrix whose row count is no multiple of 16 (rows
        // past the end come in as zeros) and for a tile cut short by the next CTA's range (its rows are read twice)
        if (lane == 0) {
            mbar_expect_tx(bar, 16 * pitch);
            tma_2d(dst, &maps.m[si], win / 4, pc.row, bar);
        }
        ++issued;
        if (++p_slot == D) p_slot = 0;
        if (++p_r == spt_of(pc.seg)) {
            p_r = 0;
            cursor_next<MIX>(pc, P, lo, hi, tstep);
        }
    };
    while (issued < n_stage && issued < D) issue();

    pdl_wait();          // activations, residual and outputs belong to the previous kernel until here

    // Fused RMSNorm: the CTA normalises the token once into shared memory (same arithmetic as the
    // stand-alone kernel: fp32 sum of squares, x * r narrowed to fp16, then times the fp16 weight)
    // and every warp builds its B fragments from there.
    const __half* xsrc = P.x;
    if (P.norm_w) {
        const int K = P.nsb * QK_K;
        __half* xs = reinterpret_cast<__half*>(smem + xs_off);
        float* nred = reinterpret_cast<float*>(smem + xs_off + K * 2);
        float ssq = 0.f;
        for (int i = threadIdx.x * 8; i < K; i += WARPS * 32 * 8) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(P.x + i));
            const __half2* h2 = reinterpret_cast<const __half2*>(&v);
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
        const float r = rsqrtf(tot / static_cast<float>(K) + P.eps);
        for (int i = threadIdx.x * 8; i < K; i += WARPS * 32 * 8) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(P.x + i));
            const uint4 w = __ldg(reinterpret_cast<const uint4*>(P.norm_w + i));
            const __half* hv = reinterpret_cast<const __half*>(&v);
            const __half* hw = reinterpret_cast<const __half*>(&w);
            uint4 o;
            __half* ho = reinterpret_cast<__half*>(&o);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const __half normed = __float2half_rn(__half2float(hv[j]) * r);
                ho[j] = __float2half_rn(__half2float(hw[j]) * __half2float(normed));
            }
            *reinterpret_cast<uint4*>(xs + i) = o;
        }
        __syncthreads();
        xsrc = xs;
    }

    // tensor-parallel exchange: this call's epoch and slot set
    uint32_t tp_next = 0;
    if (RT == 1 && !GU && P.tp.world) {
        tp_next = *reinterpret_cast<volatile uint32_t*>(P.tp.peer[P.tp.rank]) + 1u;
    }

    const ScaleSel ss = make_scale_sel(t);
    // the token's fragments of this warp's slice, kept in registers where the slice is a single slot
    XFrag xc[(CACHE && KIND != Q6) ? SBS : 1];
    XFrag6 xc6;
    if (CACHE) {
        if constexpr (KIND == Q6) {
            load_xfrag6(xc6, xsrc, sb_lo, g, t);
        } else {
#pragma unroll
            for (int i = 0; i < SBS; ++i) load_xfrag(xc[i], xsrc, sb_lo + i, g, t);
        }
    }

    // Q6_K without the cached fragments: the next super-block's activations are requested while this one is
    // worked on (the sequence of super-blocks is the warp's slice, again for every tile)
    uint2 xahead[2] = {};
    if (KIND == Q6 && !CACHE && my_tiles > 0) load_xraw6(xahead, xsrc, sb_lo, g, t);

    bool ok = true;
    int c_slot = 0;
    uint32_t c_ph = 0;
    Cursor cc = {0, 0, 0};
    cursor_enter<MIX>(cc, P, lo, hi);
    cursor_next<MIX>(cc, P, lo, hi, GU ? 0 : grp);
    int it = 0;
    // One tile of kind TK (the launch's own kind; a mixed launch runs its Q4_K tiles, then its Q6_K tiles).
    auto run_tile = [&](auto kind_c) {
        constexpr int TK = decltype(kind_c)::value;
        constexpr int T_SBS = Geom<TK>::SBS, T_PITCH = Geom<TK>::PITCH, T_BLK = Geom<TK>::BLK;
        float acc[RT][2];
#pragma unroll
        for (int m = 0; m < RT; ++m) acc[m][0] = acc[m][1] = 0.f;
        for (int sb = sb_lo; sb < sb_lo + slice; sb += T_SBS) {
            uint32_t slot[RT];
#pragma unroll
            for (int mt = 0; mt < RT; ++mt) {
                slot[mt] = ring + c_slot * SLOT;
                if (ok) ok = mbar_wait(bar0 + 8 * c_slot, c_ph);
                if (++c_slot == D) {
                    c_slot = 0;
                    c_ph ^= 1u;
                }
            }
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
#pragma unroll
                for (int i = 0; i < T_SBS; ++i) {
                    if constexpr (TK == Q6) {
                        XFrag6 x6;
                        if constexpr (KIND == Q6 && CACHE) {
                            x6 = xc6;
                        } else {
                            build_xfrag6(x6, xahead);
                            load_xraw6(xahead, xsrc, sb + 1 < sb_lo + slice ? sb + 1 : sb_lo, g, t);
                        }
                        const uint32_t off = static_cast<uint32_t>(sb * T_BLK) & 15u;
                        if (off & 2u) unit_q6k<false>(slot[0] + off, x6, g, t, acc[0][0], acc[0][1]);
                        else unit_q6k<true>(slot[0] + off, x6, g, t, acc[0][0], acc[0][1]);
                    } else {
                        if (!CACHE) load_xfrag(xc[0], xsrc, sb + i, g, t);
#pragma unroll
                        for (int mt = 0; mt < RT; ++mt)
                            unit_q4k<T_PITCH>(slot[mt] + i * T_BLK, xc[CACHE ? i : 0], ss, g, t, acc[mt][0], acc[mt][1]);
                    }
                }
            }
            __syncwarp();
#pragma unroll
            for (int mt = 0; mt < RT; ++mt)
                if (issued < n_stage) issue();                       // refills the slots just drained
        }
        // fold the four t lanes ...
#pragma unroll
        for (int m = 0; m < RT; ++m)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float v = acc[m][i];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                acc[m][i] = v;
            }
        auto store = [&](int tl, float v, float u) {
            if (cc.row + tl >= cc.lim) return;
            const Seg& sg = P.seg[cc.seg];
            const int row = cc.row + tl;
            __half* y = static_cast<__half*>(sg.y);
            if (RT == 2 || GU) {
                const float a = (P.act == ALLOYB_ACT_SILU) ? act_silu(v) : act_gelu_tanh(v);
                y[row] = __float2half_rn(a * u);
            } else if (P.tp.world) {
                // this rank's partial of output `row`, delivered to every rank's slot for this rank
                const size_t off = TP_SLOTS_OFF + (static_cast<size_t>((tp_next & 1u) * 8 + P.tp.rank) * P.tp.max_n + row) * 4;
                for (int p = 0; p < P.tp.world; ++p) *reinterpret_cast<float*>(P.tp.peer[p] + off) = v;
            } else {
                __half r = __float2half_rn(v);
                if (P.residual) r = __float2half_rn(__half2float(P.residual[row]) + __half2float(r));
                y[row] = r;
            }
        };
        if constexpr (GW == 1) {
            // ... and the tile is done: lanes t == 0 hold rows g and g + 8
            if (t == 0) {
                store(g, acc[0][0], RT == 2 ? acc[RT - 1][0] : 0.f);
                store(g + 8, acc[0][1], RT == 2 ? acc[RT - 1][1] : 0.f);
            }
        } else if constexpr (GU) {
            // ... then gate (warps 0-7) and up (warps 8-15) meet: double-buffered partials, one CTA barrier
            float* rbuf = red_all + (it & 1) * (WARPS * 16);
            if (t == 0) {
                rbuf[warp * 16 + g] = acc[0][0];
                rbuf[warp * 16 + g + 8] = acc[0][1];
            }
            __syncthreads();
            if (threadIdx.x < 16) {
                float v = 0.f, u = 0.f;
#pragma unroll
                for (int w = 0; w < GW; ++w) {
                    v += rbuf[w * 16 + threadIdx.x];
                    u += rbuf[(GW + w) * 16 + threadIdx.x];
                }
                store(threadIdx.x, v, u);
            }
        } else {
            // ... then the K slices of the group (double-buffered partials, one named barrier)
            float* rbuf = red + (it & 1) * (GW * RT * 16);
            if (t == 0) {
#pragma unroll
                for (int m = 0; m < RT; ++m) {
                    rbuf[(wg * RT + m) * 16 + g] = acc[m][0];
                    rbuf[(wg * RT + m) * 16 + g + 8] = acc[m][1];
                }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "n"(GW * 32) : "memory");
            const int tl = threadIdx.x - grp * GW * 32;
            if (tl < 16) {
                float v = 0.f, u = 0.f;
#pragma unroll
                for (int w = 0; w < GW; ++w) {
                    v += rbuf[(w * RT) * 16 + tl];
                    if (RT == 2) u += rbuf[(w * RT + 1) * 16 + tl];
                }
                store(tl, v, u);
            }
        }
        cursor_next<MIX>(cc, P, lo, hi, tstep);
        ++it;
    };
    if constexpr (MIX) {
        while (it < my_tiles && !P.seg[cc.seg].q6) run_tile(std::integral_constant<int, Q4x2>{});
        if (it < my_tiles) load_xraw6(xahead, xsrc, sb_lo, g, t);
        while (it < my_tiles) run_tile(std::integral_constant<int, Q6>{});
    } else {
        while (it < my_tiles) run_tile(std::integral_constant<int, KIND>{});
    }
    if (RT == 1 && !GU && P.tp.world) {
        // ---- all-reduce of this CTA's rows: publish, wait for the same CTA of every rank, sum in
        // rank order (identical on all ranks), add the residual, store.
        __syncthreads();
        uint8_t* mine = P.tp.peer[P.tp.rank];
        // one lane per peer (second warp): each release waits for the CTA's stores to that side of
        // the switch on its own, so the eight round trips overlap instead of queueing behind one lane
        if (threadIdx.x >= 32 && threadIdx.x < 32 + P.tp.world) {
            const int p = threadIdx.x - 32;
            uint32_t* f = reinterpret_cast<uint32_t*>(P.tp.peer[p] + TP_FLAGS_OFF) + P.tp.rank * 256 + blockIdx.x;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(tp_next) : "memory");
        }
        if (threadIdx.x < P.tp.world) {
            const uint32_t* f = reinterpret_cast<const uint32_t*>(mine + TP_FLAGS_OFF) + threadIdx.x * 256 + blockIdx.x;
            uint32_t v = 0, i = 0;
            for (; i < P.tp.spin; ++i) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                if (static_cast<int32_t>(v - tp_next) >= 0) break;
                if (i > 64) __nanosleep(64);
            }
            if (i == P.tp.spin) atomicExch(&g_error, 1);
        }
        __syncthreads();
        const float* slots = reinterpret_cast<const float*>(mine + TP_SLOTS_OFF) +
                             static_cast<size_t>(tp_next & 1u) * 8 * P.tp.max_n;
        __half* y = static_cast<__half*>(P.seg[0].y);
        for (int row = lo + threadIdx.x; row < hi; row += blockDim.x) {
            float v = 0.f;
            for (int r = 0; r < P.tp.world; ++r) v += __ldcg(slots + static_cast<size_t>(r) * P.tp.max_n + row);
            __half o = __float2half_rn(v);
            if (P.residual) o = __float2half_rn(__half2float(P.residual[row]) + __half2float(o));
            y[row] = o;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t* ctr = reinterpret_cast<uint32_t*>(mine + 4);
            __threadfence();
            if (atomicAdd(ctr, 1u) == gridDim.x - 1) {
                *ctr = 0u;
                __threadfence();
                *reinterpret_cast<volatile uint32_t*>(mine) = tp_next;      // the next call's epoch
            }
        }
    }
    if (!ok) {
        // a wait ran out (sticky error word set; this CTA's results are garbage): let copies in
        // flight land before the shared memory is released
        for (uint32_t i = 0; i < 2048; ++i) __nanosleep(512);
    }
}

template <int KIND, int RT, bool CACHE, int GW, bool GU = false>
static int launch(const Maps& maps, const Params& P, cudaStream_t stream) {
    // the opt-in to large dynamic shared memory and the SM count belong to a device, not to the process
    static bool configured[MAX_DEVICES] = {};
    static int sm_count[MAX_DEVICES] = {};
    auto kern = gemv_stream_kernel<KIND, RT, CACHE, GW, GU>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) dev = 0;
    if (!configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
        configured[dev] = true;
    }
    if (!sm_count[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sm_count[dev] = n;
    }
    const int sms = sm_count[dev];
    constexpr int n_warps = WARPS, n_groups = WARPS / GW;
    const int smem = n_warps * P.depth * 16 * Geom<KIND>::PITCH + n_groups * 2 * GW * RT * 16 * 4 + n_warps * MAX_D * 8 +
                     (P.norm_w ? P.nsb * QK_K * 2 + WARPS * 4 : 0);
    int grid = sms;
    const int tiles = (P.total_rows + 15) / 16;
    if (grid > tiles) grid = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(n_warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, maps, P);
    if (e != cudaSuccess) { set_cuda_error(e); return ALLOYB_E_CUDA; }
    return ALLOYB_OK;
}

// The driver's tensor-map encoder, looked up through the runtime (no link-time dependency on the driver).
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

}  // namespace st

// One fp16 token against Q4_K or Q6_K matrices of one format (plain: up to MAX_SEGS row-stacked
// outputs; gated: Q4_K gate/up pair with the activation fused).  NOT_TAKEN for anything else.
int try_gemv_stream(const void* x, int M, int K, int dtype, const WeightSeg* seg, int n_seg, bool gated, int act,
                    const void* residual, const void* norm_w, float eps, cudaStream_t stream, const alloyb_tp* tp) {
    using namespace st;
    if (tp && (gated || n_seg != 1 || tp->world < 1 || tp->world > 8 || tp->rank < 0 || tp->rank >= tp->world ||
               seg[0].N > tp->max_n))
        return ALLOYB_NOT_TAKEN;
    if (M != 1 || dtype != ALLOYB_F16 || K % QK_K || n_seg < 1 || n_seg > MAX_SEG) return ALLOYB_NOT_TAKEN;
    // With an exchange attached every rank must take the same path: "not taken" is kept for what all
    // ranks see alike (shape, format); a pointer or pitch only this rank has wrong is a hard error,
    // so that no rank falls back to another all-reduce on its own while its peers wait here.
    const int misaligned = tp ? ALLOYB_E_ALIGN : ALLOYB_NOT_TAKEN;
    if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(norm_w) % 16) return misaligned;
    if (norm_w && K > 16384) return ALLOYB_NOT_TAKEN;             // the normalised token lives in shared memory
    const int nsb = K / QK_K;
    if (gated && (n_seg != 2 || seg[0].N != seg[1].N)) return ALLOYB_NOT_TAKEN;
    const int fmt = seg[0].format;
    if (fmt != ALLOYB_Q4_K && !(fmt == ALLOYB_Q6_K && !gated)) return ALLOYB_NOT_TAKEN;
    int64_t all_rows = 0;
    for (int i = 0; i < (gated ? 1 : n_seg); ++i) all_rows += seg[i].N;
    // whole tiles per warp once every SM owns at least two tiles per warp, else the K dimension of
    // a tile is split over 8 warps (4 when a row has only 4-7 super-blocks)
    int gw = (all_rows / 16 >= static_cast<int64_t>(2) * WARPS * 148) ? 1 : (nsb >= 8 ? 8 : (nsb >= 4 ? 4 : 0));
    // an odd, small number of tiles per SM would leave one of the two groups a tile short: all
    // sixteen warps then share every tile (one super-block wide slices)
    const int tiles_per_cta = static_cast<int>((all_rows + 16 * 148 - 1) / (16 * 148));
    if (gw == 8 && !gated && nsb >= 16 && nsb % 16 == 0 && (tiles_per_cta == 1 || tiles_per_cta == 3)) gw = 16;
    if (gw == 0) return ALLOYB_NOT_TAKEN;
    // two super-blocks per slot only when every warp's slice is a whole number of pairs
    const int kind = fmt == ALLOYB_Q6_K ? Q6 : ((nsb % (2 * gw) == 0) ? Q4x2 : Q4x1);
    const int sbs = kind == Q4x2 ? 2 : 1;
    const int blk = fmt == ALLOYB_Q6_K ? Q6K_BYTES : Q4K_BYTES;
    const int pitch = kind == Q6 ? Geom<Q6>::PITCH : (kind == Q4x2 ? Geom<Q4x2>::PITCH : Geom<Q4x1>::PITCH);
    Params P = {};
    Maps maps;
    P.x = static_cast<const __half*>(x);
    P.residual = static_cast<const __half*>(residual);
    P.norm_w = static_cast<const __half*>(norm_w);
    P.eps = eps;
    if (tp) {
        P.tp.world = tp->world;
        P.tp.rank = tp->rank;
        P.tp.max_n = tp->max_n;
        P.tp.spin = tp->spin_limit > 0 ? static_cast<uint32_t>(tp->spin_limit) : SPIN_LIMIT;
        for (int r = 0; r < tp->world; ++r) P.tp.peer[r] = static_cast<uint8_t*>(tp->peer[r]);
    }
    P.n_seg = gated ? 1 : n_seg;
    P.nsb = nsb;
    P.gated = gated ? 1 : 0;
    P.act = act;
    P.depth = kind == Q4x1 ? 3 : 2;                               // ring slots per warp (measured best)
    int64_t rows = 0;
    for (int i = 0; i < n_seg; ++i) {
        if (seg[i].format != fmt || seg[i].N <= 0) return ALLOYB_NOT_TAKEN;
        if (reinterpret_cast<uintptr_t>(seg[i].data) % 16 || seg[i].row_bytes % 16) return misaligned;
        if (seg[i].row_bytes < static_cast<int64_t>(nsb) * blk) return ALLOYB_NOT_TAKEN;
        P.seg[i].data = static_cast<const uint8_t*>(seg[i].data);
        P.seg[i].row_bytes = seg[i].row_bytes;
        P.seg[i].y = seg[i].y;
        P.seg[i].n_rows = seg[i].N;
        P.seg[i].row_base = gated ? 0 : static_cast<int>(rows);
        if (!gated || i == 0) rows += seg[i].N;
    }
    if (rows > (1 << 30)) return ALLOYB_NOT_TAKEN;
    P.total_rows = static_cast<int>(rows);
    const EncodeFn encode = encoder();
    if (!encode) { set_cuda_error(cudaErrorNotSupported); return ALLOYB_E_CUDA; }
    for (int i = 0; i < n_seg; ++i) {
        // the packed matrix as rows of 32-bit words; a box is one slot: pitch/4 words x 16 rows
        const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(seg[i].row_bytes) / 4, static_cast<cuuint64_t>(seg[i].N)};
        const cuuint64_t gstr[1] = {static_cast<cuuint64_t>(seg[i].row_bytes)};
        const cuuint32_t box[2] = {static_cast<cuuint32_t>(pitch / 4), 16};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult cr = encode(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(seg[i].data), gdim, gstr,
                                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) { set_cuda_error(cudaErrorInvalidValue); return ALLOYB_E_CUDA; }
    }
    for (int i = n_seg; i < MAX_SEG; ++i) maps.m[i] = maps.m[0];
    const bool cache = gw > 1 && nsb == sbs * gw;        // every warp's slice is exactly one slot
    if (gw == 16) {
        if (kind == Q6) return cache ? launch<Q6, 1, true, 16>(maps, P, stream) : launch<Q6, 1, false, 16>(maps, P, stream);
        if (kind == Q4x2) return cache ? launch<Q4x2, 1, true, 16>(maps, P, stream) : launch<Q4x2, 1, false, 16>(maps, P, stream);
        return cache ? launch<Q4x1, 1, true, 16>(maps, P, stream) : launch<Q4x1, 1, false, 16>(maps, P, stream);
    }
#define ALLOYB_ST_LAUNCH(KIND, RT)                                                                              \
    (gw == 1 ? launch<KIND, RT, false, 1>(maps, P, stream)                                                     \
     : gw == 4 ? (cache ? launch<KIND, RT, true, 4>(maps, P, stream) : launch<KIND, RT, false, 4>(maps, P, stream)) \
               : (cache ? launch<KIND, RT, true, 8>(maps, P, stream) : launch<KIND, RT, false, 8>(maps, P, stream)))
    if (kind == Q6) return ALLOYB_ST_LAUNCH(Q6, 1);
    if (gated && gw == 8) {
        // the two matrices go to the two groups of eight warps
        if (kind == Q4x2)
            return cache ? launch<Q4x2, 1, true, 8, true>(maps, P, stream) : launch<Q4x2, 1, false, 8, true>(maps, P, stream);
        return cache ? launch<Q4x1, 1, true, 8, true>(maps, P, stream) : launch<Q4x1, 1, false, 8, true>(maps, P, stream);
    }
    if (gated) return kind == Q4x2 ? ALLOYB_ST_LAUNCH(Q4x2, 2) : ALLOYB_ST_LAUNCH(Q4x1, 2);
    return kind == Q4x2 ? ALLOYB_ST_LAUNCH(Q4x2, 1) : ALLOYB_ST_LAUNCH(Q4x1, 1);
#undef ALLOYB_ST_LAUNCH
}

// Q4_K matrices and Q6_K matrices of one token in ONE launch (q/k and v of a decode step): the Q4_K rows
// first, a Q6_K row counted Q6_ROW_COST times when the rows are shared out over the CTAs.  The caller has
// checked formats, alignment and row lengths; K is a multiple of 16 super-blocks (eight K slices of whole
// two-super-block slots).
static int launch_mixed(const void* x, int K, const WeightSeg (*grp)[MAX_SEGS], const int* cnt, const void* norm_w,
                        float eps, cudaStream_t stream) {
    using namespace st;
    const int nsb = K / QK_K;
    Params P = {};
    Maps maps;
    P.x = static_cast<const __half*>(x);
    P.norm_w = static_cast<const __half*>(norm_w);
    P.eps = eps;
    P.nsb = nsb;
    P.depth = 2;
    const EncodeFn encode = encoder();
    if (!encode) { set_cuda_error(cudaErrorNotSupported); return ALLOYB_E_CUDA; }
    int64_t units = 0;
    int n = 0;
    for (int f = 0; f < 2; ++f)
        for (int i = 0; i < cnt[f]; ++i, ++n) {
            const WeightSeg& w = grp[f][i];
            P.seg[n].data = static_cast<const uint8_t*>(w.data);
            P.seg[n].row_bytes = w.row_bytes;
            P.seg[n].y = w.y;
            P.seg[n].n_rows = w.N;
            P.seg[n].row_base = static_cast<int>(units);
            P.seg[n].q6 = f;
            units += static_cast<int64_t>(w.N) * (f ? Q6_ROW_COST : 1);
            if (units > (1 << 30)) return ALLOYB_NOT_TAKEN;
            const int pitch = f ? Geom<Q6>::PITCH : Geom<Q4x2>::PITCH;
            const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(w.row_bytes) / 4, static_cast<cuuint64_t>(w.N)};
            const cuuint64_t gstr[1] = {static_cast<cuuint64_t>(w.row_bytes)};
            const cuuint32_t box[2] = {static_cast<cuuint32_t>(pitch / 4), 16};
            const cuuint32_t estr[2] = {1, 1};
            const CUresult cr = encode(&maps.m[n], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(w.data), gdim, gstr, box,
                                       estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (cr != CUDA_SUCCESS) { set_cuda_error(cudaErrorInvalidValue); return ALLOYB_E_CUDA; }
        }
    for (int i = n; i < MAX_SEG; ++i) maps.m[i] = maps.m[0];
    P.n_seg = n;
    P.total_rows = static_cast<int>(units);
    return nsb == 16 ? launch<QMIX, 1, true, 8>(maps, P, stream) : launch<QMIX, 1, false, 8>(maps, P, stream);
}

int try_gemv_stream_mixed(const void* x, int M, int K, int dtype, const WeightSeg* seg, int n_seg, const void* residual,
                          const void* norm_w, float eps, cudaStream_t stream) {
    if (M != 1 || n_seg < 1 || n_seg > MAX_SEGS) return ALLOYB_NOT_TAKEN;
    WeightSeg grp[2][MAX_SEGS];
    int cnt[2] = {0, 0};
    for (int i = 0; i < n_seg; ++i) {
        const int f = seg[i].format == ALLOYB_Q4_K ? 0 : (seg[i].format == ALLOYB_Q6_K ? 1 : -1);
        if (f < 0) return ALLOYB_NOT_TAKEN;
        grp[f][cnt[f]++] = seg[i];
    }
    if (cnt[0] == 0 || cnt[1] == 0)
        return try_gemv_stream(x, M, K, dtype, seg, n_seg, false, 0, residual, norm_w, eps, stream, nullptr);
    if (residual) return ALLOYB_NOT_TAKEN;
    // both launches must be possible before the first one is made: probe with the cheap checks
    if (dtype != ALLOYB_F16 || K % QK_K || (K / QK_K) % 8) return ALLOYB_NOT_TAKEN;
    for (int i = 0; i < n_seg; ++i)
        if (reinterpret_cast<uintptr_t>(seg[i].data) % 16 || seg[i].row_bytes % 16 || seg[i].N <= 0 ||
            seg[i].row_bytes < static_cast<int64_t>(K / QK_K) * (seg[i].format == ALLOYB_Q4_K ? Q4K_BYTES : Q6K_BYTES))
            return ALLOYB_NOT_TAKEN;
    // one launch for both formats where the K split is whole slots (else one launch per format)
    if ((K / QK_K) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(norm_w) % 16 == 0 &&
        !(norm_w && K > 16384))
        return launch_mixed(x, K, grp, cnt, norm_w, eps, stream);
    for (int f = 0; f < 2; ++f) {
        const int rc = try_gemv_stream(x, M, K, dtype, grp[f], cnt[f], false, 0, nullptr, norm_w, eps, stream, nullptr);
        if (rc != ALLOYB_OK) return rc == ALLOYB_NOT_TAKEN ? ALLOYB_E_SHAPE : rc;
    }
    return ALLOYB_OK;
}

int gemv_stream_device_error(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, st::g_error, sizeof(int)) != cudaSuccess) return 0;
    if (clear && v) {
        const int z = 0;
        cudaMemcpyToSymbol(st::g_error, &z, sizeof(int));
    }
    return v;
}

}  // namespace alloyb

// Quantised linear: host-side routing and the CUDA-core row kernels.
#include "linear.cuh"
#include "linear_rows.cuh"

namespace alloyb {

constexpr int ROWS_WARPS = 8;     // warps (= weight rows) per CTA in the row kernels
constexpr int ROWS_MT = 4;        // activation rows handled per pass

struct RowSegs {
    WeightSeg seg[MAX_SEGS];
    int n_seg;
    int total_rows;
};

template <typename XT>
__global__ void __launch_bounds__(ROWS_WARPS * 32)
linear_rows_kernel(const XT* __restrict__ x, int M, int K, RowSegs segs,
                   const XT* __restrict__ residual) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int row = blockIdx.x * ROWS_WARPS + warp;
    if (row >= segs.total_rows) return;
    int si = 0;
    while (si + 1 < segs.n_seg && row >= segs.seg[si].N) {
        row -= segs.seg[si].N;
        ++si;
    }
    const WeightSeg& sg = segs.seg[si];
    const uint8_t* wrow = static_cast<const uint8_t*>(sg.data) + static_cast<int64_t>(row) * sg.row_bytes;
    const __half* srow = sg.scales ? static_cast<const __half*>(sg.scales) +
                                         static_cast<int64_t>(row) * (K / Q8_BLOCK)
                                   : nullptr;
    pdl_wait();
    for (int m0 = 0; m0 < M; m0 += ROWS_MT) {
        float acc[ROWS_MT];
#pragma unroll
        for (int t = 0; t < ROWS_MT; ++t) acc[t] = 0.f;
        const XT* xm = x + static_cast<int64_t>(m0) * K;
        const int m_left = M - m0;
        if (sg.format == ALLOYB_Q4_K)
            row_dot_q4k<XT, ROWS_MT>(wrow, xm, K, K, m_left, acc);
        else if (sg.format == ALLOYB_Q6_K)
            row_dot_q6k<XT, ROWS_MT>(wrow, xm, K, K, m_left, acc);
        else
            row_dot_q8_0<XT, ROWS_MT>(reinterpret_cast<const int8_t*>(wrow), srow, xm, K, K, m_left,
                                      acc);
#pragma unroll
        for (int t = 0; t < ROWS_MT; ++t) {
            const float v = warp_sum(acc[t]);
            if (lane == 0 && t < m_left) {
                const int64_t o = static_cast<int64_t>(m0 + t) * sg.ldy + row;
                XT y = from_f32<XT>(v);
                if (residual) y = from_f32<XT>(to_f32<XT>(residual[o]) + to_f32<XT>(y));
                static_cast<XT*>(sg.y)[o] = y;
            }
        }
    }
}

template <typename XT>
__global__ void __launch_bounds__(ROWS_WARPS * 32)
gated_rows_kernel(const XT* __restrict__ x, int M, int K, int N, int format,
                  const uint8_t* __restrict__ gate, const __half* __restrict__ gate_scales,
                  const uint8_t* __restrict__ up, const __half* __restrict__ up_scales,
                  int64_t row_bytes, XT* __restrict__ y, int act) {
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * ROWS_WARPS + warp;
    if (row >= N) return;
    const uint8_t* grow = gate + static_cast<int64_t>(row) * row_bytes;
    const uint8_t* urow = up + static_cast<int64_t>(row) * row_bytes;
    pdl_wait();
    for (int m0 = 0; m0 < M; m0 += ROWS_MT) {
        float ag[ROWS_MT], au[ROWS_MT];
#pragma unroll
        for (int t = 0; t < ROWS_MT; ++t) ag[t] = au[t] = 0.f;
        const XT* xm = x + static_cast<int64_t>(m0) * K;
        const int m_left = M - m0;
        if (format == ALLOYB_Q4_K) {
            row_dot_q4k<XT, ROWS_MT>(grow, xm, K, K, m_left, ag);
            row_dot_q4k<XT, ROWS_MT>(urow, xm, K, K, m_left, au);
        } else {
            const int64_t so = static_cast<int64_t>(row) * (K / Q8_BLOCK);
            row_dot_q8_0<XT, ROWS_MT>(reinterpret_cast<const int8_t*>(grow), gate_scales + so, xm, K,
                                      K, m_left, ag);
            row_dot_q8_0<XT, ROWS_MT>(reinterpret_cast<const int8_t*>(urow), up_scales + so, xm, K,
                                      K, m_left, au);
        }
#pragma unroll
        for (int t = 0; t < ROWS_MT; ++t) {
            const float g = warp_sum(ag[t]);
            const float u = warp_sum(au[t]);
            if (lane == 0 && t < m_left) {
                const float a = (act == ALLOYB_ACT_SILU) ? act_silu(g) : act_gelu_tanh(g);
                y[static_cast<int64_t>(m0 + t) * N + row] = from_f32<XT>(a * u);
            }
        }
    }
}

static int validate_segs(const alloyb_weight* w, int n_w, int K, RowSegs& out) {
    if (!w) return ALLOYB_E_NULL;
    if (n_w < 1 || n_w > MAX_SEGS) return ALLOYB_E_SHAPE;
    out.n_seg = n_w;
    out.total_rows = 0;
    for (int i = 0; i < n_w; ++i) {
        const alloyb_weight& a = w[i];
        if (!a.data || !a.y) return ALLOYB_E_NULL;
        if (a.N <= 0) return ALLOYB_E_SHAPE;
        int64_t dense;
        switch (a.format) {
            case ALLOYB_Q4_K:
                if (K % QK_K) return ALLOYB_E_SHAPE;
                dense = static_cast<int64_t>(K / QK_K) * Q4K_BYTES;
                break;
            case ALLOYB_Q6_K:
                if (K % QK_K) return ALLOYB_E_SHAPE;
                dense = static_cast<int64_t>(K / QK_K) * Q6K_BYTES;
                break;
            case ALLOYB_Q8_0:
                if (K % Q8_BLOCK) return ALLOYB_E_SHAPE;
                if (!a.scales) return ALLOYB_E_NULL;
                dense = K;
                break;
            default:
                return ALLOYB_E_SHAPE;
        }
        WeightSeg& s = out.seg[i];
        s.format = a.format;
        s.N = a.N;
        s.data = a.data;
        s.scales = a.scales;
        s.row_bytes = a.row_bytes ? a.row_bytes : dense;
        if (s.row_bytes < dense) return ALLOYB_E_SHAPE;
        const int need = (a.format == ALLOYB_Q6_K) ? 2 : 4;
        if ((reinterpret_cast<uintptr_t>(a.data) % need) || (s.row_bytes % need)) return ALLOYB_E_ALIGN;
        s.y = a.y;
        s.ldy = a.ldy ? a.ldy : a.N;
        if (s.ldy < a.N) return ALLOYB_E_SHAPE;
        out.total_rows += a.N;
    }
    return ALLOYB_OK;
}

template <typename XT>
static int launch_rows(const void* x, int M, int K, const RowSegs& segs, const void* residual,
                       cudaStream_t st) {
    const int blocks = (segs.total_rows + ROWS_WARPS - 1) / ROWS_WARPS;
    launch_pdl(linear_rows_kernel<XT>, dim3(blocks), dim3(ROWS_WARPS * 32), 0, st, 
        static_cast<const XT*>(x), M, K, segs, static_cast<const XT*>(residual));
    return check_launch();
}

}  // namespace alloyb

using namespace alloyb;

// The GEMV family and, last, the exact-weight row kernels: any M, any alignment.
static int linear_few_tokens(const void* x, int M, int K, int dtype, const RowSegs& segs, const void* residual,
                             cudaStream_t st) {
    int rc;
    rc = try_linear_fast(x, M, K, dtype, segs.seg, segs.n_seg, residual, st);
    if (rc != ALLOYB_NOT_TAKEN) return rc;
    {
        // Q8_0 matrices: the streaming GEMV of linear_q8.cu, one launch per matrix and four tokens
        bool all_q8 = true;
        for (int i = 0; i < segs.n_seg; ++i) all_q8 &= segs.seg[i].format == ALLOYB_Q8_0 && segs.seg[i].row_bytes == K;
        if (all_q8 && M < 64) {
            bool taken = true;
            for (int i = 0; i < segs.n_seg && taken; ++i) {
                const WeightSeg& sg = segs.seg[i];
                rc = try_q8_gemv(x, M, K, dtype, sg.data, sg.scales, nullptr, nullptr, sg.y, sg.N, sg.ldy, residual, false, 0, st);
                if (rc == ALLOYB_NOT_TAKEN) taken = false;          // only possible for the first matrix (shape-wide reasons)
                else if (rc != ALLOYB_OK) return rc;
            }
            if (taken) return ALLOYB_OK;
        }
    }

    switch (dtype) {
        case ALLOYB_F16: return launch_rows<__half>(x, M, K, segs, residual, st);
        case ALLOYB_BF16: return launch_rows<__nv_bfloat16>(x, M, K, segs, residual, st);
        case ALLOYB_F32: return launch_rows<float>(x, M, K, segs, residual, st);
        default: return ALLOYB_E_DTYPE;
    }
}

extern "C" int alloyb_linear(const void* x, int M, int K, int dtype, const alloyb_weight* w, int n_w,
                             const void* residual, void* stream) {
    if (!x) return ALLOYB_E_NULL;
    if (M < 0 || K <= 0) return ALLOYB_E_SHAPE;
    RowSegs segs;
    int rc = validate_segs(w, n_w, K, segs);
    if (rc != ALLOYB_OK) return rc;
    if (residual && n_w != 1) return ALLOYB_E_SHAPE;
    if (M == 0) return ALLOYB_OK;
    cudaStream_t st = as_stream(stream);

    if (M >= GEMM_TC_MIN_M) {
        // more than a handful of tokens: one tcgen05 GEMM per matrix; a matrix it does not take (type,
        // alignment) goes through the kernels below on its own
        for (int i = 0; i < segs.n_seg; ++i) {
            // two matrices of one format that lie back to back in one buffer (q and k of a layer) run as ONE
            // GEMM; its epilogue sends the second matrix's rows to their own output
            const WeightSeg& a = segs.seg[i];
            if (i + 1 < segs.n_seg && !residual && a.format != ALLOYB_Q8_0 && a.N % 128 == 0) {
                const WeightSeg& b = segs.seg[i + 1];
                if (b.format == a.format && b.row_bytes == a.row_bytes &&
                    static_cast<const uint8_t*>(b.data) == static_cast<const uint8_t*>(a.data) + static_cast<int64_t>(a.N) * a.row_bytes) {
                    rc = try_gemm_tc(x, M, K, dtype, a, nullptr, nullptr, nullptr, 0, st, &b);
                    if (rc == ALLOYB_OK) {
                        ++i;
                        continue;
                    }
                    if (rc != ALLOYB_NOT_TAKEN) return rc;
                }
            }
            rc = try_gemm_tc(x, M, K, dtype, segs.seg[i], residual, nullptr, nullptr, 0, st);
            if (rc == ALLOYB_NOT_TAKEN) {
                RowSegs one;
                one.n_seg = 1;
                one.seg[0] = segs.seg[i];
                one.total_rows = segs.seg[i].N;
                rc = linear_few_tokens(x, M, K, dtype, one, residual, st);
            }
            if (rc != ALLOYB_OK) return rc;
        }
        return ALLOYB_OK;
    }
    return linear_few_tokens(x, M, K, dtype, segs, residual, st);
}

static int single(const void* x, int fmt, const void* data, const void* scales, void* y, int M,
                  int N, int K, int dtype, void* stream) {
    alloyb_weight w;
    w.format = fmt;
    w.N = N;
    w.data = data;
    w.scales = scales;
    w.row_bytes = 0;
    w.y = y;
    w.ldy = 0;
    return alloyb_linear(x, M, K, dtype, &w, 1, nullptr, stream);
}

extern "C" int alloyb_q4k_mm(const void* x, const void* blocks, void* y, int M, int N, int K,
                             int dtype, void* stream) {
    return single(x, ALLOYB_Q4_K, blocks, nullptr, y, M, N, K, dtype, stream);
}
extern "C" int alloyb_q6k_mm(const void* x, const void* blocks, void* y, int M, int N, int K,
                             int dtype, void* stream) {
    return single(x, ALLOYB_Q6_K, blocks, nullptr, y, M, N, K, dtype, stream);
}
extern "C" int alloyb_q8_0_mm(const void* x, const void* qweight, const void* scales, void* y, int M,
                              int N, int K, int dtype, void* stream) {
    return single(x, ALLOYB_Q8_0, qweight, scales, y, M, N, K, dtype, stream);
}

extern "C" int alloyb_gated_linear(const void* x, const void* gate, const void* gate_scales,
                                   const void* up, const void* up_scales, void* y, int M, int N,
                                   int K, int format, int act, int dtype, void* stream) {
    if (!x || !gate || !up || !y) return ALLOYB_E_NULL;
    if (M < 0 || N <= 0 || K <= 0) return ALLOYB_E_SHAPE;
    if (act != ALLOYB_ACT_SILU && act != ALLOYB_ACT_GELU_TANH) return ALLOYB_E_SHAPE;
    int64_t row_bytes;
    if (format == ALLOYB_Q4_K) {
        if (K % QK_K) return ALLOYB_E_SHAPE;
        row_bytes = static_cast<int64_t>(K / QK_K) * Q4K_BYTES;
    } else if (format == ALLOYB_Q8_0) {
        if (K % Q8_BLOCK) return ALLOYB_E_SHAPE;
        if (!gate_scales || !up_scales) return ALLOYB_E_NULL;
        row_bytes = K;
    } else {
        return ALLOYB_E_SHAPE;   // the reference fuses gate/up only for Q4_K and Q8_0
    }
    if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up)) % 4) return ALLOYB_E_ALIGN;
    if (M == 0) return ALLOYB_OK;
    cudaStream_t st = as_stream(stream);

    int rc = ALLOYB_NOT_TAKEN;
    if (M >= GEMM_TC_MIN_M) {
        const WeightSeg g = {format, N, gate, gate_scales, row_bytes, y, N};
        rc = try_gemm_tc(x, M, K, dtype, g, nullptr, up, up_scales, act, st);
        if (rc != ALLOYB_NOT_TAKEN) return rc;
    }
    rc = try_gated_fast(x, gate, gate_scales, up, up_scales, y, M, N, K, format, act, dtype, st);
    if (rc != ALLOYB_NOT_TAKEN) return rc;
    if (format == ALLOYB_Q8_0) {
        rc = try_q8_gemv(x, M, K, dtype, gate, gate_scales, up, up_scales, y, N, N, nullptr, true, act, st);
        if (rc != ALLOYB_NOT_TAKEN) return rc;
    }

    const int blocks = (N + ROWS_WARPS - 1) / ROWS_WARPS;
    const uint8_t* g8 = static_cast<const uint8_t*>(gate);
    const uint8_t* u8 = static_cast<const uint8_t*>(up);
    const __half* gs = static_cast<const __half*>(gate_scales);
    const __half* us = static_cast<const __half*>(up_scales);
    switch (dtype) {
        case ALLOYB_F16:
            launch_pdl(gated_rows_kernel<__half>, dim3(blocks), dim3(ROWS_WARPS * 32), 0, st, 
                static_cast<const __half*>(x), M, K, N, format, g8, gs, u8, us, row_bytes,
                static_cast<__half*>(y), act);
            break;
        case ALLOYB_BF16:
            launch_pdl(gated_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(ROWS_WARPS * 32), 0, st, 
                static_cast<const __nv_bfloat16*>(x), M, K, N, format, g8, gs, u8, us, row_bytes,
                static_cast<__nv_bfloat16*>(y), act);
            break;
        case ALLOYB_F32:
            launch_pdl(gated_rows_kernel<float>, dim3(blocks), dim3(ROWS_WARPS * 32), 0, st, 
                static_cast<const float*>(x), M, K, N, format, g8, gs, u8, us, row_bytes,
                static_cast<float*>(y), act);
            break;
        default:
            return ALLOYB_E_DTYPE;
    }
    return check_launch();
}

// ---- RMSNorm fused into the activation load (one token), two launches otherwise

extern "C" int alloyb_linear_normed(const void* x, const void* norm_weight, float eps, void* xn_scratch, int M, int K,
                                    int dtype, const alloyb_weight* w, int n_w, void* stream) {
    if (!x || !norm_weight || !xn_scratch) return ALLOYB_E_NULL;
    if (M < 0 || K <= 0) return ALLOYB_E_SHAPE;
    RowSegs segs;
    int rc = validate_segs(w, n_w, K, segs);
    if (rc != ALLOYB_OK) return rc;
    if (M == 0) return ALLOYB_OK;
    rc = try_gemv_stream_mixed(x, M, K, dtype, segs.seg, segs.n_seg, nullptr, norm_weight, eps, as_stream(stream));
    if (rc != ALLOYB_NOT_TAKEN) return rc;
    rc = alloyb_rms_norm(x, norm_weight, xn_scratch, M, K, eps, dtype, stream);
    if (rc != ALLOYB_OK) return rc;
    return alloyb_linear(xn_scratch, M, K, dtype, w, n_w, nullptr, stream);
}

extern "C" int alloyb_gated_linear_normed(const void* x, const void* norm_weight, float eps, void* xn_scratch,
                                          const void* gate, const void* gate_scales, const void* up,
                                          const void* up_scales, void* y, int M, int N, int K, int format, int act,
                                          int dtype, void* stream) {
    if (!x || !norm_weight || !xn_scratch || !gate || !up || !y) return ALLOYB_E_NULL;
    if (M < 0 || N <= 0 || K <= 0) return ALLOYB_E_SHAPE;
    if (act != ALLOYB_ACT_SILU && act != ALLOYB_ACT_GELU_TANH) return ALLOYB_E_SHAPE;
    if (M == 0) return ALLOYB_OK;
    if (format == ALLOYB_Q4_K && K % QK_K == 0 && M == 1) {
        const int64_t rb = static_cast<int64_t>(K / QK_K) * Q4K_BYTES;
        const WeightSeg pair[2] = {{ALLOYB_Q4_K, N, gate, nullptr, rb, y, N}, {ALLOYB_Q4_K, N, up, nullptr, rb, y, N}};
        const int rc = try_gemv_stream(x, M, K, dtype, pair, 2, true, act, nullptr, norm_weight, eps, as_stream(stream), nullptr);
        if (rc != ALLOYB_NOT_TAKEN) return rc;
    }
    const int rc = alloyb_rms_norm(x, norm_weight, xn_scratch, M, K, eps, dtype, stream);
    if (rc != ALLOYB_OK) return rc;
    return alloyb_gated_linear(xn_scratch, gate, gate_scales, up, up_scales, y, M, N, K, format, act, dtype, stream);
}

// ---- row-parallel linear with the all-reduce over peer memory inside the launch

extern "C" int alloyb_linear_allreduce(const void* x, int M, int K, int dtype, const alloyb_weight* w,
                                       const void* residual, const alloyb_tp* tp, void* stream) {
    if (!x || !w || !tp) return ALLOYB_E_NULL;
    if (M < 0 || K <= 0) return ALLOYB_E_SHAPE;
    if (tp->world < 1 || tp->world > 8 || tp->rank < 0 || tp->rank >= tp->world) return ALLOYB_E_SHAPE;
    for (int r = 0; r < tp->world; ++r)
        if (!tp->peer[r]) return ALLOYB_E_NULL;
    RowSegs segs;
    const int rc = validate_segs(w, 1, K, segs);
    if (rc != ALLOYB_OK) return rc;
    if (segs.seg[0].N > tp->max_n) return ALLOYB_E_LIMIT;
    if (M == 0) return ALLOYB_OK;
    return try_gemv_stream(x, M, K, dtype, segs.seg, 1, false, 0, residual, nullptr, 0.f, as_stream(stream), tp);
}

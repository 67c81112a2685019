// Internal interfaces of the quantised-linear family.
#pragma once
#include "common.cuh"

namespace alloyb {

constexpr int MAX_SEGS = 4;            // weight matrices per launch (q/k/v + one spare)

struct WeightSeg {
    int format;
    int N;
    const void* data;
    const void* scales;
    int64_t row_bytes;
    void* y;
    int64_t ldy;
};

// Tensor-core GEMV family / tcgen05 GEMM.  Return ALLOYB_NOT_TAKEN when the
// shape, type or alignment is outside what they are built for.
int try_linear_fast(const void* x, int M, int K, int dtype, const WeightSeg* seg, int n_seg,
                    const void* residual, cudaStream_t st);
int try_gated_fast(const void* x, const void* gate, const void* gate_scales, const void* up,
                   const void* up_scales, void* y, int M, int N, int K, int format, int act,
                   int dtype, cudaStream_t st);

// Persistent streaming GEMV for one fp16 token against Q4_K matrices.
// norm_w != nullptr fuses RMSNorm(x; norm_w, eps) into the activation load; tp != nullptr sums the
// (single) output over the ranks through peer memory inside the launch.
int try_gemv_stream(const void* x, int M, int K, int dtype, const WeightSeg* seg, int n_seg, bool gated, int act,
                    const void* residual, const void* norm_w, float eps, cudaStream_t stream,
                    const alloyb_tp* tp = nullptr);
// One token, any mix of Q4_K / Q6_K matrices: one streaming launch per format present.
int try_gemv_stream_mixed(const void* x, int M, int K, int dtype, const WeightSeg* seg, int n_seg, const void* residual,
                          const void* norm_w, float eps, cudaStream_t stream);
int gemv_stream_device_error(int clear);
int decode_layer_device_error(int clear);

// Q8_0 streaming GEMV (1..63 tokens, four per pass), plain (w1 == nullptr) or gate/up fused.
int try_q8_gemv(const void* x, int M, int K, int dtype, const void* w0, const void* s0, const void* w1, const void* s1,
                void* y, int N, int64_t ldy, const void* residual, bool gated, int act, cudaStream_t st);

// tcgen05 dequant-GEMM for prefill-sized M (one matrix).
// Fewer tokens go to the GEMV family: the tcgen05 kernel decodes every weight on the CUDA cores at about
// 2.4e12 weights/s whatever the token count (35 us for 14336 x 4096), and below this the tokens-as-columns
// GEMV, whose cost grows with the token count, is still ahead.
constexpr int GEMM_TC_MIN_M = 28;
// `tail`: a second matrix whose packed rows follow seg's in memory, run in the same launch (its rows go to its
// own output).
int try_gemm_tc(const void* x, int M, int K, int dtype, const WeightSeg& seg, const void* residual, const void* up,
                const void* up_scales, int act, cudaStream_t st, const WeightSeg* tail = nullptr);
int gemm_tc_device_error(int clear);

}  // namespace alloyb

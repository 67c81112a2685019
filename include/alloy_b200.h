/*
 * alloy_b200 — C ABI of the B200 (sm_100a) quantised-LLM hot path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the
 * stream the caller passes (a cudaStream_t cast to void*; NULL = the legacy
 * default stream), allocates nothing unless its comment says otherwise, never
 * exits or aborts, and returns ALLOYB_OK (0) or a negative ALLOYB_E_* code
 * (text via alloyb_error_string).  Shape and alignment problems are reported
 * before anything is launched.
 *
 * Each declaration names the reference interface it stands in for; paths are
 * relative to the rayanht/alloy checkout:
 *   torch/  = packages/alloy-torch/src/alloy_torch/
 *   metal/  = packages/alloy-metal/src/alloy/
 *   server/ = packages/alloy-server/src/alloy_server/
 */
#ifndef ALLOY_B200_H
#define ALLOY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activations / outputs */
enum { ALLOYB_F16 = 0, ALLOYB_BF16 = 1, ALLOYB_F32 = 2 };
/* weight formats */
enum { ALLOYB_Q4_K = 0, ALLOYB_Q6_K = 1, ALLOYB_Q8_0 = 2 };
/* gate activation of the fused gate/up op */
enum { ALLOYB_ACT_SILU = 0, ALLOYB_ACT_GELU_TANH = 1 };
/* KV cache layouts */
enum { ALLOYB_KV_F16 = 0, ALLOYB_KV_Q8_SPLIT = 1, ALLOYB_KV_Q8_PAGED = 2 };

enum {
    ALLOYB_OK = 0,
    ALLOYB_E_SHAPE = -1,      /* a dimension is not supported (message names it) */
    ALLOYB_E_ALIGN = -2,      /* a pointer or row pitch misses the alignment the kernel needs */
    ALLOYB_E_DTYPE = -3,
    ALLOYB_E_NULL = -4,
    ALLOYB_E_CUDA = -5,       /* a CUDA runtime call failed; see alloyb_last_cuda_error */
    ALLOYB_E_WORKSPACE = -6,  /* caller-provided workspace too small */
    ALLOYB_E_DEVICE = -7,     /* a bounded device-side wait ran out (status word set) */
    ALLOYB_E_LIMIT = -8       /* a size exceeds a stated fixed maximum */
};

int alloyb_version(void);
const char* alloyb_error_string(int code);
/* cudaError_t of the most recent failed runtime call on this thread (0 if none). */
int alloyb_last_cuda_error(void);
/* 1 when the library was built for sm_100a and the current device is CC 10.x. */
int alloyb_device_supported(void);
/* Sticky device-side error word of the current device: non-zero after a kernel's bounded
 * wait (mbarrier) ran out; the kernel then finished with undefined results instead of
 * hanging.  clear != 0 resets it.  Synchronises the device.  Negative = ALLOYB_E_*. */
int alloyb_device_error(int clear);

/* ------------------------------------------------------------------ dequantisers / embeddings
 * Bit-exact fp32 decode of packed rows.  ids == NULL decodes rows [0, n_rows);
 * otherwise out row i = decode(row ids[i]) (ids int64).  Stand in for the
 * embedding kernels metal/std/quant.py:836-884 (embedding_q4_k), :1201-1270
 * (embedding_q6_k), :812-832 (embedding_q8_0) behind torch/custom_ops.py:67-69,
 * :97-99, :103; also the test hook for the weight decode.
 *   blocks: Q4_K (rows, K/256*144) u8; Q6_K (rows, K/256*210) u8.
 *   Q8_0 takes the normalised pair: int8 (rows,K) + fp16 (rows,K/32).
 *   out: (n_rows, K) fp32 (out_dtype F32) or fp16/bf16 (rounded once from fp32). */
int alloyb_dequant_q4k(const void* blocks, const int64_t* ids, void* out, int64_t n_rows,
                       int64_t table_rows, int K, int out_dtype, void* stream);
int alloyb_dequant_q6k(const void* blocks, const int64_t* ids, void* out, int64_t n_rows,
                       int64_t table_rows, int K, int out_dtype, void* stream);
int alloyb_dequant_q8_0(const void* qweight, const void* scales, const int64_t* ids, void* out,
                        int64_t n_rows, int64_t table_rows, int K, int out_dtype, void* stream);

/* Q5_0 in the reference's normalised three-buffer form (server/gguf/quant.py:414-490
 * split_q5_0_weight): qweight (rows, K/2) u8 packs element k in the low and k+1 in the high nibble
 * of byte k/2, qhigh (rows, K/2) u8 holds their fifth bits in bit 0 / bit 4 of the same byte,
 * scales (rows, K/32) fp16; w = scale * ((nibble | fifth << 4) - 16).  Stands in for
 * embedding_q5_0 (metal/std/quant.py:887-940) behind torch/custom_ops.py:89-91. */
int alloyb_dequant_q5_0(const void* qweight, const void* qhigh, const void* scales, const int64_t* ids,
                        void* out, int64_t n_rows, int64_t table_rows, int K, int out_dtype, void* stream);

/* ------------------------------------------------------------------ quantised linear
 * y[m,n] = sum_k x[m,k] * deq(W)[n,k], fp32 accumulate, y in the activation
 * dtype.  One descriptor per weight matrix lets several sibling projections
 * (q/k/v; mixed formats allowed) run as ONE launch, which is what the
 * reference's batched ops do by concatenating rows
 * (torch/ops/linalg.py:555-669, torch/custom_ops.py:50-52, :100-102, :106-108).
 *
 * M routing inside the library replaces torch/ops/linalg.py:462-497 (Q4_K),
 * :726-739 (Q6_K), :346-401 (Q8_0): small M runs the bandwidth-bound
 * dequant-GEMV family (metal/std/quant.py:1356-1453 dot_q4_k_v2, :2201-2277
 * _rows, :1995-2126 dot_q6_k_v2, :61-273 dot_q8_0_v2); large M with bf16/fp16
 * activations runs the tcgen05 dequant-GEMM (metal/std/quant.py:768-808
 * dot_q4_k, :1949-1990 dot_q6_k and the load stage
 * metal/_compiler/msl/memory.py:441-879). */
typedef struct alloyb_weight {
    int format;              /* ALLOYB_Q4_K / Q6_K / Q8_0 */
    int N;                   /* output rows of this matrix */
    const void* data;        /* Q4_K/Q6_K: packed blocks (N, row_bytes); Q8_0: int8 (N,K) */
    const void* scales;      /* Q8_0: fp16 (N, K/32); else NULL */
    int64_t row_bytes;       /* pitch of `data` rows in bytes; 0 = dense */
    void* y;                 /* output (M, N) for this matrix, row pitch ldy elements */
    int64_t ldy;             /* 0 = N */
} alloyb_weight;

/* Generic entry: n_w matrices sharing activations x (M,K).
 * residual (may be NULL): same shape/pitch as y of matrix 0, added in the
 * epilogue as dtype(residual + dtype(acc)); only with n_w == 1.
 * One fp16 token against Q4_K and Q6_K matrices (q/k and v of a decode step) is one launch; from 28 tokens
 * up two consecutive descriptors of one format whose packed rows lie back to back in memory (the second's
 * data = the first's data + N * row_bytes, N a multiple of 128) run as one GEMM, each with its own output. */
int alloyb_linear(const void* x, int M, int K, int dtype, const alloyb_weight* w, int n_w,
                  const void* residual, void* stream);

/* Convenience forms with the reference ops' argument order
 * (torch/custom_ops.py:47-49 gguf_q4_k_mm, :96 gguf_q6_k_mm, :104 gguf_q8_0_mm). */
int alloyb_q4k_mm(const void* x, const void* blocks, void* y, int M, int N, int K, int dtype,
                  void* stream);
int alloyb_q6k_mm(const void* x, const void* blocks, void* y, int M, int N, int K, int dtype,
                  void* stream);
int alloyb_q8_0_mm(const void* x, const void* qweight, const void* scales, void* y, int M, int N,
                   int K, int dtype, void* stream);

/* Q5_0 linear (torch/custom_ops.py:86-88 gguf_q5_0_mm; kernels metal/std/quant.py:941-1197):
 * y (M, N) = x (M, K) * deq(W)^T, fp32 accumulate, y in the activation dtype.  A CUDA-core
 * warp-per-row kernel for every M (the format is outside the Q4_K_M mixes). */
int alloyb_q5_0_mm(const void* x, const void* qweight, const void* qhigh, const void* scales, void* y,
                   int M, int N, int K, int dtype, void* stream);

/* y = act(x*G^T) * (x*U^T), one launch sharing the activation load
 * (torch/custom_ops.py:53-58 gguf_q4_k_silu/_gelu, :109-111 gguf_q8_0_silu;
 * kernels metal/std/quant.py:1458-1723, :358-695; policy torch/ops/linalg.py:758-802).
 * format is ALLOYB_Q4_K or ALLOYB_Q8_0 (scales NULL for Q4_K). */
int alloyb_gated_linear(const void* x, const void* gate, const void* gate_scales, const void* up,
                        const void* up_scales, void* y, int M, int N, int K, int format, int act,
                        int dtype, void* stream);

/* RMSNorm folded into the linear that consumes it (no single counterpart op in the reference,
 * which runs rms_norm -- metal/std/norm.py:58-73 -- and the quantised matmul as two graph nodes;
 * the results are those of alloyb_rms_norm followed by alloyb_linear / alloyb_gated_linear).
 * For one fp16 token on Q4_K / Q6_K weights the normalisation happens inside the GEMV launch;
 * every other shape runs the two launches through xn_scratch (M*K elements of `dtype`, caller's
 * memory, contents undefined afterwards). */
int alloyb_linear_normed(const void* x, const void* norm_weight, float eps, void* xn_scratch, int M,
                         int K, int dtype, const alloyb_weight* w, int n_w, void* stream);
int alloyb_gated_linear_normed(const void* x, const void* norm_weight, float eps, void* xn_scratch,
                               const void* gate, const void* gate_scales, const void* up,
                               const void* up_scales, void* y, int M, int N, int K, int format,
                               int act, int dtype, void* stream);

/* RoPE of the decode token's q (fp16, contiguous (B, H, D), rotated in place) and k, plus the
 * append of the rotated k and of v to the cache at pos, in one launch (the reference runs
 * rope_apply -- metal/std/rope.py:28-84 -- and the fused cache write of attention_cache[_q8] as
 * separate steps; results are those of alloyb_rope_inplace followed by the append).  Cache
 * pointers as in alloyb_attn_decode for the same layout; attention then runs with write_kv = 0.
 * D must be a multiple of 64.  status (may be NULL): OR of the bits alloyb_attn_workspace_status
 * reports. */
int alloyb_rope_kv_append(int layout, void* q, const void* new_k, const void* new_v,
                          int64_t new_batch_stride, int64_t new_head_stride, void* k0, void* k1,
                          void* v0, void* v1, const int32_t* pos, int pos_count,
                          const float* inv_freq, int B, int H, int KV_H, int D, int S_max,
                          int64_t num_pages, int32_t* status, void* stream);

/* ------------------------------------------------------------------ tensor parallel (new)
 * The reference is single-GPU; these have no counterpart in it.  One process per GPU.  Every
 * rank allocates one exchange buffer (alloyb_tp_buffer_bytes(max_n) bytes, zero-filled by
 * alloyb_tp_alloc), exports its CUDA IPC handle (64 bytes), and imports the other ranks'
 * handles; `peer[r]` is rank r's buffer as mapped in this process (the own pointer for r ==
 * rank).  max_n = the largest output width that will be reduced. */
typedef struct alloyb_tp {
    int world;      /* 1..8 */
    int rank;
    int max_n;
    int spin_limit; /* polls of a peer's flag before a wait gives up; 0 = the default (about 4 million,
                       a few hundred ms).  A wait that gives up sets the sticky word alloyb_device_error
                       reports; the call still returns, its output is then undefined. */
    void* peer[8];
} alloyb_tp;
size_t alloyb_tp_buffer_bytes(int max_n);
int alloyb_tp_alloc(size_t bytes, void** out);
int alloyb_tp_free(void* p);
int alloyb_tp_ipc_export(void* p, void* handle64);
int alloyb_tp_ipc_import(const void* handle64, void** out);
int alloyb_tp_ipc_close(void* p);
/* Row-parallel linear: y = residual + sum over ranks of x_r * W_r^T, where every rank holds a K
 * slice of the weight (whole super-blocks) and the matching slice of the activations.  The
 * partial outputs cross NVLink inside the GEMV launch (stores into the peers' exchange buffers,
 * a flag per CTA, the sum taken in rank order on every rank): no separate collective.  All
 * ranks must make the same sequence of calls.  Returns 1 (nothing launched) when the shape is
 * outside the fused kernel -- it covers one fp16 token on a Q4_K / Q6_K matrix whose rows hold at
 * least four super-blocks (K >= 1024 on this rank) -- and the caller then runs alloyb_linear and
 * its own all-reduce; that answer depends on shape and format only, so every rank gets the same
 * one.  A pointer or row pitch that misses 16-byte alignment is ALLOYB_E_ALIGN here, never a
 * quiet per-rank fallback. */
int alloyb_linear_allreduce(const void* x, int M, int K, int dtype, const alloyb_weight* w,
                            const void* residual, const alloyb_tp* tp, void* stream);

/* ------------------------------------------------------------------ q8_0 KV cache
 * Quantise n_tokens rows per (batch, kv head) of fp16 `src` into the split
 * cache tensors at positions [start, start+n_tokens): codes int8 (B,KV_H,S_max,D),
 * scales fp16 (B,KV_H,S_max,D/32).  Strides of src in elements.
 * Replaces kv_quantize_q8_range (metal/std/kv_quant.py:24-70). */
int alloyb_kv_quantize_q8(const void* src, int64_t src_batch_stride, int64_t src_head_stride,
                          int64_t src_tok_stride, void* codes, void* scales, int B, int KV_H,
                          int S_max, int D, int start, int n_tokens, void* stream);
/* fp16(code*scale) for positions [0, end) into scratch (B,KV_H,S_max,D) fp16.
 * Replaces kv_dequant_q8_range (metal/std/kv_quant.py:73-108). */
int alloyb_kv_dequant_q8(const void* codes, const void* scales, void* out, int B, int KV_H,
                         int S_max, int D, int end, void* stream);

/* Paged pool: uint8 (num_pages, 2 [K,V], KV_H, 16 tokens, D/32 blocks, 34 bytes);
 * a block is fp16 scale + 32 int8 codes.  page_table int32 (B, max_pages).
 * Appends one new token per sequence at position seq_pos[b] (int32 (B,)):
 * new_k/new_v fp16 (B, KV_H, D) with the given strides (elements).
 * No reference counterpart as a kernel of its own (the reference fuses the
 * write into its attention kernel, metal/std/kv_quant.py:212-246); same
 * arithmetic as kv_quantize_q8_range.  A position or page id outside the
 * table is skipped, not written; when status (device int32, may be NULL) is
 * given, bit 0 / bit 1 is set there for a bad position / page id. */
int alloyb_kv_append_q8_paged(const void* new_k, const void* new_v, int64_t batch_stride,
                              int64_t head_stride, void* pool, const int32_t* page_table,
                              int max_pages, int64_t num_pages, const int32_t* seq_pos, int B,
                              int KV_H, int D, int32_t* status, void* stream);

/* Write n_tokens new rows per (sequence, kv head) at positions [start_b, start_b + n_tokens) of a
 * cache in any layout (k0..v1, S_max, num_pages as in alloyb_attn_decode); the q8 layouts quantise
 * each row exactly as the one-token append does.  new_k / new_v: fp16 (B, KV_H, n_tokens, D) with
 * the given strides in elements.  start: int32 device (start_count,), 1 = shared by every
 * sequence.  The chunk write of the reference's prefill branch: kv_quantize_q8_range
 * (metal/std/kv_quant.py:24-70) launched from torch/ops/kv_quant.py:101-119, and the fp16 row
 * write of attention_prefill_warm (torch/ops/attention.py:96-100).  status as in
 * alloyb_kv_append_q8_paged. */
int alloyb_kv_write(int layout, const void* new_k, const void* new_v, int64_t batch_stride,
                    int64_t head_stride, int64_t tok_stride, void* k0, void* k1, void* v0, void* v1,
                    const int32_t* start, int start_count, int B, int KV_H, int D, int S_max,
                    int64_t num_pages, int n_tokens, int32_t* status, void* stream);

/* Causal attention of a chunk of n_tokens query tokens per sequence over a cache that already
 * holds the chunk's rows: query i sits at position start_b + i and attends to [0, start_b + i].
 * Covers the seq_len > 1 branches of attention_cache / attention_cache_q8 (prefill:
 * torch/ops/kv_quant.py:121-162, where the reference dequantises history + chunk to an fp16
 * scratch, metal/std/kv_quant.py:73-108, and runs fp16 prefill attention; here the codes are read
 * directly and dequantised per tile in shared memory to the same fp16 values) and the 2..16-token
 * verify step attention_kv_update_multi (torch/ops/attention.py:1255-1275).  q: (B, H, n_tokens,
 * D) with strides in elements, f16 / bf16 / f32 (computed as fp16); out: (B, n_tokens, H, D)
 * dense in q's dtype.  D is 64, 128 or 256.  No workspace.  status (may be NULL) receives the
 * same bits as alloyb_attn_workspace_status. */
int alloyb_attn_chunk(int layout, const void* q, int64_t q_batch_stride, int64_t q_head_stride,
                      int64_t q_tok_stride, int q_dtype, void* k0, void* k1, void* v0, void* v1,
                      const int32_t* start, int start_count, void* out, int B, int H, int KV_H, int D,
                      int n_tokens, int S_max, int64_t num_pages, float scale, int32_t* status,
                      void* stream);

/* ------------------------------------------------------------------ decode attention
 * One query token per sequence, GQA (head h reads kv head h / (H/KV_H)),
 * causal over positions [0, pos_b]; split-K partials merged with log-sum-exp.
 * Replaces attention_decode_vector_split_q8 (metal/std/kv_quant.py:111-414),
 * attention_decode_vector_split (metal/std/attention.py:2126-2363) and the
 * combine kernels (metal/std/attention.py:2367-2410, :2657-2722) behind
 * attention_cache_q8 / attention_cache (torch/custom_ops.py:136-150;
 * handlers torch/ops/kv_quant.py:58-249, torch/ops/attention.py:886-1089).
 *
 * layout selects how k0..v1 are read:
 *   ALLOYB_KV_F16      k0 = K (B,KV_H,S_max,D) fp16, v0 = V, k1 = v1 = NULL
 *   ALLOYB_KV_Q8_SPLIT k0 = K codes int8 (B,KV_H,S_max,D), k1 = K scales fp16
 *                      (B,KV_H,S_max,D/32), v0/v1 likewise
 *   ALLOYB_KV_Q8_PAGED k0 = pool (see above), k1 = page_table int32 (B,max_pages),
 *                      S_max = max_pages*16, v0 = v1 = NULL
 * q: (B,H,D) with strides in elements, dtype f16/bf16/f32 (computed as fp16
 * like the reference, torch/ops/kv_quant.py:175-180).  out: (B,H,D) dense in
 * q's dtype.  pos: int32 (pos_count,) newest position per sequence; when
 * pos_count == 1 every sequence uses pos[0] (the reference's cache_pos[:1]).
 * write_kv != 0: new_k/new_v fp16 (B,KV_H,D) are first stored (quantised for
 * the q8 layouts) at position pos_b, then attended, as the reference's fused
 * WRITE_KV does.  scale <= 0 selects 1/sqrt(D).
 * workspace: at least alloyb_attn_workspace_bytes(B,H,D) bytes, 256-aligned;
 * it holds a status word, completion counters and the fp32 split partials,
 * must be cleared once with alloyb_attn_workspace_init before its first use,
 * and must not be shared by calls that may overlap on the device.  Positions
 * or page ids outside the cache are skipped on the device and recorded in the
 * status word (bit 0 position, bit 1 page id), read back with
 * alloyb_attn_workspace_status (which synchronises the stream). */
size_t alloyb_attn_workspace_bytes(int B, int H, int D);
int alloyb_attn_workspace_init(void* workspace, size_t workspace_bytes, int B, int H, void* stream);
int alloyb_attn_workspace_status(const void* workspace, int32_t* status_out, void* stream);
int alloyb_attn_decode(int layout, const void* q, int64_t q_batch_stride, int64_t q_head_stride,
                       int q_dtype, void* k0, void* k1, void* v0, void* v1, const void* new_k,
                       const void* new_v, int64_t new_batch_stride, int64_t new_head_stride,
                       const int32_t* pos, int pos_count, void* out, int B, int H, int KV_H, int D,
                       int S_max, int64_t num_pages, float scale, int write_kv, void* workspace,
                       size_t workspace_bytes, void* stream);

/* The decode token's whole attention step in ONE launch: rotate-half RoPE of q and of the new K row, the
 * append of the new K / V rows (any layout; q8 layouts quantise) and the attention.  Bit-identical to
 * alloyb_rope_kv_append followed by alloyb_attn_decode(write_kv = 0), except that q is left unrotated
 * in memory.  fp16 q with 16-byte-aligned rows, head_dim 128, at most eight query heads per KV head;
 * other shapes return ALLOYB_NOT_TAKEN (1) and nothing is launched.  No reference counterpart: the
 * reference rotates in model code and fuses only the cache write
 * (packages/alloy-metal/src/alloy/std/kv_quant.py:212-246). */
int alloyb_attn_decode_rope(int layout, const void* q, int64_t q_batch_stride, int64_t q_head_stride,
                            void* k0, void* k1, void* v0, void* v1, const void* new_k, const void* new_v,
                            int64_t new_batch_stride, int64_t new_head_stride, const int32_t* pos,
                            int pos_count, const float* inv_freq, void* out, int B, int H, int KV_H, int D,
                            int S_max, int64_t num_pages, float scale, void* workspace,
                            size_t workspace_bytes, void* stream);

/* Decode attention that allocates nothing and needs no workspace from the caller (no
 * counterpart in the reference, whose runtime owns its scratch buffers).  For hosts that may
 * not allocate device memory where the decode step runs -- a serving loop with a frozen
 * memory plan, a plugin host that forbids allocation after start-up -- the split-K partials
 * live in a fixed device array inside the library image: ALLOYB_ATTN_STATIC_BYTES on every
 * GPU that loads the library, until the process exits.  Same arguments and results as
 * alloyb_attn_decode without workspace/workspace_bytes.  Shapes whose
 * alloyb_attn_workspace_bytes(B,H,D) exceeds ALLOYB_ATTN_STATIC_BYTES return ALLOYB_E_LIMIT.
 * The first call on a device looks up the array's device address (make that call before any
 * stream capture).  All calls on a device share the array: calls that may overlap on the GPU
 * race and must be serialised by the caller.  It calls no cudaMalloc/cudaFree. */
#define ALLOYB_ATTN_STATIC_BYTES (16 * 1024 * 1024)
int alloyb_attn_decode_static(int layout, const void* q, int64_t q_batch_stride,
                              int64_t q_head_stride, int q_dtype, void* k0, void* k1, void* v0,
                              void* v1, const void* new_k, const void* new_v,
                              int64_t new_batch_stride, int64_t new_head_stride, const int32_t* pos,
                              int pos_count, void* out, int B, int H, int KV_H, int D, int S_max,
                              int64_t num_pages, float scale, int write_kv, void* stream);
/* Status word of the latest alloyb_attn_decode_static call on the current device (bit 0: a
 * position, bit 1: a page id was out of range and skipped); each static call starts it at zero.
 * Synchronises the stream.  No counterpart in the reference. */
int alloyb_attn_static_status(int32_t* status_out, void* stream);

/* ------------------------------------------------------------------ one-launch decode step
 * The whole decode step of a Llama-shape model for ONE token (batch 1, fp16 activations, Q4_K /
 * Q6_K weights, head_dim 128, at most 8 query heads per KV head) as a single persistent launch:
 * per layer RMSNorm + q/k/v, RoPE + KV append + attention, o_proj + residual, RMSNorm + gate/up +
 * SiLU, down + residual, then the final norm and the output head -- the per-step call stack of the
 * reference's serving loop (server/models/attention.py:845-886 for the attention block,
 * torch/ops/linalg.py:462-497 / :726-802 for the linears, metal/std/norm.py:40-73, rope.py:28-84),
 * which the reference runs as one graph of separate dispatches.  Results are those of the
 * separate entry points above (same arithmetic per op).
 *
 * All sizes are this rank's LOCAL sizes when tensor-parallel (heads, kv_heads, ffn and head.N are
 * shards; hidden is whole).  alloyb_decoder_create allocates (cudaMalloc) the device-side phase
 * list and scratch once; alloyb_decoder_step allocates nothing, launches on `stream` (one memset
 * plus one cooperative launch) and can be captured in a CUDA graph.  The caller writes the token's
 * embedding into hidden_io and the token position into *pos before each step; afterwards logits
 * holds head.N fp16 values and the KV caches hold the token's row. */
typedef struct alloyb_matrix {
    int format;              /* ALLOYB_Q4_K or ALLOYB_Q6_K */
    int N;                   /* output rows */
    const void* data;        /* packed rows, 16-byte aligned */
    int64_t row_bytes;       /* pitch, multiple of 16; 0 = dense */
} alloyb_matrix;
typedef struct alloyb_decoder_layer {
    alloyb_matrix wq, wk, wv, wo, wg, wu, wd;
    const void* norm_in;     /* fp16 (hidden) */
    const void* norm_post;
    void* k0; void* k1; void* v0; void* v1;   /* this layer's cache for ONE sequence, as in alloyb_attn_decode */
} alloyb_decoder_layer;
typedef struct alloyb_decoder_desc {
    int n_layers, hidden, ffn, heads, kv_heads, head_dim;
    float eps;
    int kv_layout;           /* ALLOYB_KV_F16 or ALLOYB_KV_Q8_PAGED */
    int S_max;
    int64_t num_pages;
    const alloyb_decoder_layer* layers;
    const void* norm_final;
    alloyb_matrix head;
    const float* inv_freq;   /* fp32 (head_dim / 2) */
    const int32_t* pos;      /* device: position of the token being decoded */
    void* hidden_io;         /* fp16 (hidden) */
    void* logits;            /* fp16 (head.N) */
    const alloyb_tp* tp;     /* NULL, or the exchange the o_proj / down sums go through */
} alloyb_decoder_desc;
int alloyb_decoder_create(const alloyb_decoder_desc* desc, void** handle);
int alloyb_decoder_step(void* handle, void* stream);
int alloyb_decoder_phases(void* handle);     /* phases the step walks (diagnostic) */
int alloyb_decoder_status(void* handle, int32_t* status_out, void* stream);   /* bits as alloyb_attn_workspace_status */
/* Diagnostic: with tracing on, every CTA records four nanosecond clocks per phase (token staged,
 * phase done, next phase's first copies issued, barrier passed); trace_read synchronises the device
 * and copies n_values <= phases * SMs * 4 of them, ordered [phase][CTA][4]. */
int alloyb_decoder_trace(void* handle, int on);
int alloyb_decoder_trace_read(void* handle, uint64_t* out_ns, int n_values);
int alloyb_decoder_destroy(void* handle);

/* ------------------------------------------------------------------ routed experts
 * gguf_moe_routed (torch/custom_ops.py:59-66; kernels metal/std/moe.py:31-228): per token the
 * top_k largest router logits (descending, lowest index on ties) with a softmax over just those;
 * h = silu(x * gate_e^T) * (x * up_e^T) per slot from the fused Q4_K tensor gate_up_blocks
 * (E, 2*I, H/256*144) (gate rows then up rows of each expert); out (T, H) fp32 =
 * sum over slots of w_slot * (h_slot * down_e^T) with down_qweight Q6_K (E, H, I/256*210).
 * hidden (T, H) f16 / bf16 / f32; router_logits (T, E) fp32.  workspace: at least
 * alloyb_moe_workspace_bytes bytes, 256-aligned (routing, weights, per-slot activations). */
size_t alloyb_moe_workspace_bytes(int T, int top_k, int moe_intermediate);
int alloyb_moe_routed(const void* hidden, int hidden_dtype, const float* router_logits,
                      const void* gate_up_blocks, const void* down_qweight, float* out, int T, int H,
                      int num_experts, int top_k, int moe_intermediate, void* workspace,
                      size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ decode-step glue
 * Small fp16/bf16 ops of the decode step (not graded kernels):
 * rms_norm metal/std/norm.py:40-73 (normalise in fp32, cast, then multiply by
 * the weight), rotate-half RoPE metal/std/rope.py:28-84 applied in place to
 * q (B,H,D) and k (B,KV_H,D) at position pos_b with angle = float(pos)*inv_freq[j]
 * (inv_freq fp32 (D/2,)), silu_mul
 * metal/std/elementwise.py:40-43, greedy argmax of
 * server/generation/decode.py:22-61. */
int alloyb_rms_norm(const void* x, const void* weight, void* y, int M, int K, float eps, int dtype,
                    void* stream);
int alloyb_rope_inplace(void* q, void* k, const int32_t* pos, int pos_count, const float* inv_freq,
                        int B, int H, int KV_H, int D, int dtype, void* stream);
int alloyb_silu_mul(const void* gate, const void* up, void* y, int64_t n, int dtype, void* stream);
int alloyb_argmax(const void* logits, int64_t* out_ids, int M, int N, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ALLOY_B200_H */

"""CPU oracle for the quantised-LLM hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module: it is the checker the
CUDA kernels are compared with (tests, the smoke check, and the timed CPU
baseline of the benchmark), never a fallback.

Every function restates, in NumPy, arithmetic the reference defines:

* Q4_K decode: reference ``tests/kernels/test_quant_q4k_native.py:45-70``
  (``_get_scale_min_k4``/``_dequant``) and the kernel-side layout in
  ``packages/alloy-metal/src/alloy/std/quant.py:844-883``.
* Q6_K decode: reference ``packages/alloy-metal/src/alloy/std/quant.py:1216-1270``
  (``embedding_q6_k``, element-wise).
* Q8_0 weights: reference ``packages/alloy-server/src/alloy_server/gguf/quant.py:497-521``
  (split of the 34-byte wire block) and
  ``packages/alloy-metal/src/alloy/std/quant.py:828-832`` (``w = scale*q``).
* q8_0 KV quantise/dequantise: reference ``tests/kernels/test_kv_quant.py:19-30``
  and ``:219-221``; kernel ``packages/alloy-metal/src/alloy/std/kv_quant.py:59-70``.
* decode attention: reference ``tests/kernels/test_kv_quant.py:225-239``
  (float64 softmax over the dequantised cache, GQA ``h // kv_group``,
  causal over positions [0, pos]).
* chunk (prefill / verify) attention: the same per query row, query i of the
  chunk at position start + i (reference ``tests/kernels/test_kv_quant.py:466-479``).
* Q5_0: split of the 22-byte wire block into the three normalised buffers,
  reference ``packages/alloy-server/src/alloy_server/gguf/quant.py:414-490``;
  ``w = scale * ((nibble | fifth << 4) - 16)``.
* routed experts: top-k over raw logits + softmax of the winners, SiLU-gated
  Q4_K gate/up, Q6_K down, routing-weighted sum
  (``packages/alloy-metal/src/alloy/std/moe.py:31-228``; the router identity
  ``renorm(topk(softmax)) == softmax(topk)`` is the one the reference checks in
  ``tests/kernels/test_moe.py:148-175``).

The weight dequantisers' arithmetic lives in the third-party package
``gguf`` 0.19.0 (pinned in the reference's ``uv.lock:809-810``), which is not
part of the reference tree; its published block formats are restated here.

Parity pins: ``tests/test_oracle.py`` checks this module bit-for-bit against
the committed fixtures in ``tests/golden/`` — produced by running the
reference's own test decoders (Q4_K, q8_0 KV, attention) and ``gguf`` 0.19.0
(Q4_K, Q6_K, Q8_0) in a container that holds both (``tests/golden/make_golden.py``).
Q6_K, Q8_0 and Q5_0 weights have no decoder in the reference's own tests; they
are pinned at the ``gguf`` boundary only (Q5_0 additionally against the
reference's own ``split_q5_0_weight``).  The routed-expert op has only
device-side references in the reference's tests: its oracle here is the
composition of the pinned decoders, "parity unpinned" as an op.
"""

from __future__ import annotations

import numpy as np

QK_K = 256
Q4K_BYTES = 144
Q6K_BYTES = 210
Q8_0_BYTES = 34


def _f16_field(blk: np.ndarray, lo: int) -> np.ndarray:
    """fp16 at byte offset ``lo`` of every block, widened (exactly) to fp32."""
    return np.ascontiguousarray(blk[..., lo:lo + 2]).view(np.float16)[..., 0].astype(np.float32)


# --------------------------------------------------------------------------- Q4_K


def q4k_scales_mins(sbytes: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Unpack the 12 scale bytes of each block into eight 6-bit (scale, min) pairs.

    ``sbytes``: (..., 12) uint8 -> two (..., 8) int32 arrays.  Sub-blocks 0-3
    take the low six bits of bytes 0-3 (scale) and 4-7 (min); sub-blocks 4-7
    take a nibble of bytes 8-11 plus the top two bits of bytes 0-3 / 4-7.
    """
    s = sbytes.astype(np.int32)
    sc = np.empty(s.shape[:-1] + (8,), np.int32)
    mn = np.empty_like(sc)
    for g in range(8):
        if g < 4:
            sc[..., g] = s[..., g] & 63
            mn[..., g] = s[..., g + 4] & 63
        else:
            sc[..., g] = (s[..., g + 4] & 15) | ((s[..., g - 4] >> 6) << 4)
            mn[..., g] = (s[..., g + 4] >> 4) | ((s[..., g] >> 6) << 4)
    return sc, mn


def dequant_q4_k(blocks: np.ndarray) -> np.ndarray:
    """(N, NB*144) uint8 -> (N, NB*256) float32; ``w = d*sc*nib - dmin*m`` in fp32."""
    n = blocks.shape[0]
    nb = blocks.shape[1] // Q4K_BYTES
    b = blocks.reshape(n, nb, Q4K_BYTES)
    d = _f16_field(b, 0)
    dmin = _f16_field(b, 2)
    sc, mn = q4k_scales_mins(b[:, :, 4:16])
    qs = b[:, :, 16:144]
    p = np.arange(QK_K)
    g, l = p // 32, p % 32
    byte = qs[:, :, (g // 2) * 32 + l]                       # (n, nb, 256)
    nib = np.where(g & 1, byte >> 4, byte & 15).astype(np.float32)
    dsc = (d[:, :, None] * sc.astype(np.float32))[:, :, g]   # exact: 11 + 6 bits
    dm = (dmin[:, :, None] * mn.astype(np.float32))[:, :, g]
    w = dsc * nib - dm                                       # one rounding, at the subtract
    return w.astype(np.float32).reshape(n, nb * QK_K)


def dequant_q4_k_scalar(blocks: np.ndarray) -> np.ndarray:
    """Element-by-element Python loop of the same decode (small inputs only)."""
    n = blocks.shape[0]
    nb = blocks.shape[1] // Q4K_BYTES
    out = np.empty((n, nb * QK_K), np.float32)
    for r in range(n):
        for ib in range(nb):
            blk = blocks[r, ib * Q4K_BYTES:(ib + 1) * Q4K_BYTES]
            d = np.float32(blk[0:2].view(np.float16)[0])
            dmin = np.float32(blk[2:4].view(np.float16)[0])
            s = [int(v) for v in blk[4:16]]
            for p in range(QK_K):
                g, l = divmod(p, 32)
                if g < 4:
                    sc, m = s[g] & 63, s[g + 4] & 63
                else:
                    sc = (s[g + 4] & 15) | ((s[g - 4] >> 6) << 4)
                    m = (s[g + 4] >> 4) | ((s[g] >> 6) << 4)
                byte = int(blk[16 + (g // 2) * 32 + l])
                nib = (byte >> 4) if (g & 1) else (byte & 15)
                out[r, ib * QK_K + p] = np.float32(d * np.float32(sc) * np.float32(nib)) - \
                    np.float32(dmin * np.float32(m))
    return out


# --------------------------------------------------------------------------- Q6_K


def dequant_q6_k(blocks: np.ndarray) -> np.ndarray:
    """(N, NB*210) uint8 -> (N, NB*256) float32; ``w = d * sc[p//16] * (q - 32)``."""
    n = blocks.shape[0]
    nb = blocks.shape[1] // Q6K_BYTES
    b = blocks.reshape(n, nb, Q6K_BYTES)
    ql = b[:, :, 0:128]
    qh = b[:, :, 128:192]
    sc = b[:, :, 192:208].view(np.int8).astype(np.float32)
    d = _f16_field(b, 208)
    p = np.arange(QK_K)
    g, l = p // 32, p % 32
    qlb = ql[:, :, (g // 4) * 64 + (g % 2) * 32 + l]
    nib = np.where((g % 4) >= 2, qlb >> 4, qlb & 15).astype(np.int32)
    hi = ((qh[:, :, (g // 4) * 32 + l].astype(np.int32)) >> ((g % 4) * 2)) & 3
    q = ((nib | (hi << 4)) - 32).astype(np.float32)
    w = (d[:, :, None] * sc[:, :, p // 16]) * q              # all products exact in fp32
    return w.astype(np.float32).reshape(n, nb * QK_K)


# --------------------------------------------------------------------------- Q8_0 weights


def split_q8_0(wire: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """(N, K/32*34) uint8 wire blocks -> int8 (N, K) codes + fp16 (N, K/32) scales."""
    n = wire.shape[0]
    g = wire.shape[1] // Q8_0_BYTES
    b = np.ascontiguousarray(wire).reshape(n, g, Q8_0_BYTES)
    scales = np.ascontiguousarray(b[:, :, 0:2]).view(np.float16).reshape(n, g).copy()
    codes = np.ascontiguousarray(b[:, :, 2:]).view(np.int8).reshape(n, g * 32).copy()
    return codes, scales


def dequant_q8_0(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """int8 (N,K) and fp16 (N,K/32) -> (N,K) float32; ``w = scale*q`` (exact)."""
    s = np.repeat(scales.astype(np.float32), 32, axis=-1)
    return (codes.astype(np.float32) * s).astype(np.float32)


# --------------------------------------------------------------------------- Q5_0 weights

Q5_0_BYTES = 22


def split_q5_0(wire: np.ndarray) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(N, K/32*22) uint8 wire blocks ``{fp16 d; u8 qh[4]; u8 qs[16]}`` -> the three
    K-sequential buffers: qweight (N, K/2) with element k in the low and k+1 in the high
    nibble of byte k/2, qhigh (N, K/2) with their fifth bits in bit 0 / bit 4, fp16 scales
    (N, K/32).  Wire element l < 16 is ``qs[l] & 15`` with fifth bit ``qh32 >> l``; element
    l + 16 is ``qs[l] >> 4`` with fifth bit ``qh32 >> (l + 16)``."""
    n = wire.shape[0]
    g = wire.shape[1] // Q5_0_BYTES
    b = np.ascontiguousarray(wire).reshape(n, g, Q5_0_BYTES)
    scales = np.ascontiguousarray(b[:, :, 0:2]).view(np.float16).reshape(n, g).copy()
    qh32 = np.ascontiguousarray(b[:, :, 2:6]).view(np.uint32).reshape(n, g)
    qs = b[:, :, 6:22]
    nib = np.concatenate([qs & 15, qs >> 4], axis=2)                        # (n, g, 32) in K order
    fifth = ((qh32[:, :, None] >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8)
    qweight = (nib[:, :, 0::2] | (nib[:, :, 1::2] << 4)).astype(np.uint8).reshape(n, g * 16)
    qhigh = (fifth[:, :, 0::2] | (fifth[:, :, 1::2] << 4)).astype(np.uint8).reshape(n, g * 16)
    return qweight, qhigh, scales


def dequant_q5_0(qweight: np.ndarray, qhigh: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """The three normalised buffers -> (N, K) float32; ``w = scale * (q - 16)`` (exact)."""
    n, half = qweight.shape
    nib = np.stack([qweight & 15, qweight >> 4], axis=-1).reshape(n, half * 2).astype(np.int32)
    fifth = np.stack([qhigh & 1, (qhigh >> 4) & 1], axis=-1).reshape(n, half * 2).astype(np.int32)
    q = ((nib | (fifth << 4)) - 16).astype(np.float32)
    return (q * np.repeat(scales.astype(np.float32), 32, axis=-1)).astype(np.float32)


# --------------------------------------------------------------------------- routed experts


def moe_routed_ref(x: np.ndarray, logits: np.ndarray, gate_up: np.ndarray, down: np.ndarray,
                   top_k: int, inter: int) -> np.ndarray:
    """float64 routed-expert output (T, H).  ``gate_up``: (E, 2*I, H/256*144) Q4_K bytes (gate
    rows then up rows per expert); ``down``: (E, H, I/256*210) Q6_K bytes.  Router: softmax over
    all experts, top-k, renormalise (ties: lowest index first)."""
    t_n, hdim = x.shape
    e_n = logits.shape[1]
    out = np.zeros((t_n, hdim), np.float64)
    lg = logits.astype(np.float64)
    for t in range(t_n):
        p = np.exp(lg[t] - lg[t].max())
        p /= p.sum()
        order = np.lexsort((np.arange(e_n), -lg[t]))[:top_k]
        w = p[order] / p[order].sum()
        for e, we in zip(order, w):
            gu = dequant_q4_k(np.ascontiguousarray(gate_up[e]).reshape(2 * inter, -1)).astype(np.float64)
            g = gu[:inter] @ x[t].astype(np.float64)
            u = gu[inter:] @ x[t].astype(np.float64)
            h = (silu(g) * u).astype(np.float32).astype(np.float64)          # the op keeps h in fp32
            dw = dequant_q6_k(np.ascontiguousarray(down[e]).reshape(hdim, -1)).astype(np.float64)
            out[t] += we * (dw @ h)
    return out


# --------------------------------------------------------------------------- matmul refs


def mm_ref(x: np.ndarray, w_f32: np.ndarray) -> np.ndarray:
    """fp32 ``x @ W.T`` with the activations widened from their storage type."""
    return x.astype(np.float32) @ w_f32.T


def mm_ref_f64(x: np.ndarray, w_f32: np.ndarray) -> np.ndarray:
    """float64 ``x @ W.T``: the rounding-free yardstick the tolerance tests use."""
    return x.astype(np.float64) @ w_f32.astype(np.float64).T


def silu(g: np.ndarray) -> np.ndarray:
    """``g / (1 + exp(-g))`` (reference ``std/quant.py:1350-1351``)."""
    g = g.astype(np.float64)
    return g / (1.0 + np.exp(-g))


def gelu_tanh(g: np.ndarray) -> np.ndarray:
    g = g.astype(np.float64)
    return 0.5 * g * (1.0 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))


# --------------------------------------------------------------------------- q8_0 KV


def kv_quantize_q8_0(kv: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Quantise fp16 rows (..., D) in 32-element blocks along the last axis.

    ``m = max|x|`` (fp32); ``scale = fp16(m / 127)``; ``inv = 127 / m`` (0 when
    m == 0) in fp32; ``code = int8(sign(x*inv) * floor(|x*inv| + .5))``.
    Returns int8 codes (..., D) and fp16 scales (..., D/32).
    """
    d = kv.shape[-1]
    x = kv.astype(np.float32).reshape(kv.shape[:-1] + (d // 32, 32))
    m = np.abs(x).max(axis=-1)
    scales = (m / np.float32(127.0)).astype(np.float16)
    with np.errstate(divide="ignore"):
        inv = np.where(m > 0, np.float32(127.0) / m, np.float32(0.0)).astype(np.float32)
    q = (x * inv[..., None]).astype(np.float32)
    codes = (np.sign(q) * np.floor(np.abs(q) + np.float32(0.5))).astype(np.int8)
    return codes.reshape(kv.shape), scales


def kv_dequant_q8_0(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """fp32 ``code * scale`` (reference ``test_kv_quant.py:219-221``)."""
    return codes.astype(np.float32) * np.repeat(scales.astype(np.float32), 32, axis=-1)


def kv_pack_blocks(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """Interleave codes (..., D) and scales (..., D/32) into 34-byte q8_0 blocks
    (..., D/32*34) uint8: fp16 scale then 32 int8 codes."""
    d = codes.shape[-1]
    g = d // 32
    out = np.empty(codes.shape[:-1] + (g, Q8_0_BYTES), np.uint8)
    out[..., 0:2] = np.ascontiguousarray(scales).view(np.uint8).reshape(scales.shape + (2,))
    out[..., 2:] = np.ascontiguousarray(codes).view(np.uint8).reshape(codes.shape[:-1] + (g, 32))
    return out.reshape(codes.shape[:-1] + (g * Q8_0_BYTES,))


def kv_unpack_blocks(raw: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    g = raw.shape[-1] // Q8_0_BYTES
    b = np.ascontiguousarray(raw).reshape(raw.shape[:-1] + (g, Q8_0_BYTES))
    scales = np.ascontiguousarray(b[..., 0:2]).view(np.float16).reshape(raw.shape[:-1] + (g,))
    codes = np.ascontiguousarray(b[..., 2:]).view(np.int8).reshape(raw.shape[:-1] + (g * 32,))
    return codes.copy(), scales.copy()


# --------------------------------------------------------------------------- attention


def attention_decode_ref(k: np.ndarray, v: np.ndarray, q: np.ndarray, pos: int,
                         scale: float | None = None) -> np.ndarray:
    """float64 single-query attention for one sequence.

    ``k``, ``v``: (KV_H, S, D) dequantised (or fp16) cache rows; ``q``: (H, D);
    attends positions [0, pos].  Query head h reads KV head ``h // (H/KV_H)``.
    """
    heads, dim = q.shape
    group = heads // k.shape[0]
    sc = (1.0 / np.sqrt(dim)) if scale is None else scale
    out = np.empty((heads, dim), np.float64)
    for h in range(heads):
        kh = k[h // group, :pos + 1].astype(np.float64)
        vh = v[h // group, :pos + 1].astype(np.float64)
        s = kh @ q[h].astype(np.float64) * sc
        p = np.exp(s - s.max())
        p /= p.sum()
        out[h] = p @ vh
    return out


def attention_chunk_ref(k: np.ndarray, v: np.ndarray, q: np.ndarray, start: int,
                        scale: float | None = None) -> np.ndarray:
    """float64 causal attention of a chunk for one sequence: ``q`` (H, S, D); query i sits at
    position ``start + i`` and attends to cache positions [0, start + i] of ``k``/``v``
    (KV_H, >= start + S, D), which already hold the chunk's rows.  Returns (H, S, D)."""
    heads, s_n, dim = q.shape
    out = np.empty((heads, s_n, dim), np.float64)
    for i in range(s_n):
        out[:, i] = attention_decode_ref(k, v, q[:, i], start + i, scale)
    return out


def gather_pages(pool: np.ndarray, page_ids, n_tokens: int) -> np.ndarray:
    """Collect a sequence's rows from a page pool.

    ``pool``: (num_pages, KV_H, page_tokens, row_bytes-or-D); ``page_ids``: the
    sequence's page numbers in order.  Returns (KV_H, n_tokens, ...).
    """
    pages = pool[np.asarray(page_ids)]                       # (P, KV_H, T, X)
    p, h, t, x = pages.shape
    return pages.transpose(1, 0, 2, 3).reshape(h, p * t, x)[:, :n_tokens]


# --------------------------------------------------------------------------- decode-step glue


def rms_norm_ref(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """``w * cast(x * rsqrt(mean(x^2) + eps))`` with the normalisation in fp32
    and the product in the weight's dtype (reference ``std/norm.py:58-73``)."""
    xf = x.astype(np.float32)
    r = 1.0 / np.sqrt((xf * xf).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps))
    return (w * (xf * r.astype(np.float32)).astype(w.dtype)).astype(w.dtype)


def rope_ref(x: np.ndarray, pos: np.ndarray, theta: float) -> np.ndarray:
    """Rotate-half RoPE (reference ``std/rope.py:28-84``): x (..., T, D), pos (T,)."""
    d = x.shape[-1]
    inv = (1.0 / (theta ** (np.arange(0, d, 2, dtype=np.float32) / np.float32(d)))).astype(np.float32)
    ang = pos.astype(np.float32)[:, None] * inv[None, :]
    c, s = np.cos(ang), np.sin(ang)
    x1, x2 = x[..., : d // 2].astype(np.float32), x[..., d // 2:].astype(np.float32)
    return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], axis=-1)

"""CPU oracle of one Llama-shape Q4_K_M decode step.  TEST INFRASTRUCTURE ONLY.

Restates the reference's decode call stack on NumPy: RMSNorm
(``packages/alloy-metal/src/alloy/std/norm.py:40-73``), q/k/v projections on
dequantised weights, rotate-half RoPE (``std/rope.py:28-84``), KV row write +
softmax attention over [0, pos] (``tests/kernels/test_kv_quant.py:225-239``),
o_proj + residual, SwiGLU MLP (``std/quant.py:1350-1351``), final norm, head and
greedy argmax (``packages/alloy-server/src/alloy_server/generation/decode.py:22-61``).
Matmuls and softmax run in float64; every op's output is rounded to fp16, the
activation type the reference serves in, so differences from the device path
come from accumulation order only.
"""

from __future__ import annotations

import numpy as np

from . import blocks as O


def _h(a):
    return np.asarray(a).astype(np.float16)


def _rms(x, w, eps):
    xf = x.astype(np.float32)
    r = (1.0 / np.sqrt((xf.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps)).astype(np.float32)
    return _h(w.astype(np.float32) * _h(xf * r).astype(np.float32))


def _rope(x, pos, inv_freq):
    d = x.shape[-1]
    ang = (np.float32(pos) * inv_freq.astype(np.float32)).astype(np.float32)
    c, s = np.cos(ang.astype(np.float64)), np.sin(ang.astype(np.float64))
    x1, x2 = x[..., : d // 2].astype(np.float64), x[..., d // 2:].astype(np.float64)
    return _h(np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1))


def decode_step(ids, pos, embed_w, layers, norm_final, head_w, inv_freq, k_caches, v_caches,
                heads, kv_heads, head_dim, eps, kv_q8=False):
    """``layers``: dicts of dequantised fp32 matrices wq wk wv wo wg wu wd and fp16 norm_in
    norm_post.  ``k_caches``/``v_caches``: per layer fp32 (B, KV_H, S, D) arrays, updated in
    place at ``pos``.  ``kv_q8``: the new rows go through the q8_0 KV quantiser first (what a q8_0
    cache stores and attention later reads).  Returns (logits fp16 (B, vocab), next ids, hidden)."""
    b = len(ids)
    h = _h(embed_w[np.asarray(ids)])
    for li, lw in enumerate(layers):
        xn = _rms(h, lw["norm_in"], eps)
        q = _h(O.mm_ref_f64(xn, lw["wq"])).reshape(b, heads, head_dim)
        k = _h(O.mm_ref_f64(xn, lw["wk"])).reshape(b, kv_heads, head_dim)
        v = _h(O.mm_ref_f64(xn, lw["wv"])).reshape(b, kv_heads, head_dim)
        q, k = _rope(q, pos, inv_freq), _rope(k, pos, inv_freq)
        if kv_q8:
            k_caches[li][:, :, pos] = O.kv_dequant_q8_0(*O.kv_quantize_q8_0(k))
            v_caches[li][:, :, pos] = O.kv_dequant_q8_0(*O.kv_quantize_q8_0(v))
        else:
            k_caches[li][:, :, pos] = k.astype(np.float32)
            v_caches[li][:, :, pos] = v.astype(np.float32)
        a = np.stack([O.attention_decode_ref(k_caches[li][i], v_caches[li][i], q[i], pos)
                      for i in range(b)])
        a = _h(a).reshape(b, heads * head_dim)
        h = _h(h.astype(np.float32) + _h(O.mm_ref_f64(a, lw["wo"])).astype(np.float32))
        xn = _rms(h, lw["norm_post"], eps)
        g = O.mm_ref_f64(xn, lw["wg"])
        u = O.mm_ref_f64(xn, lw["wu"])
        act = _h(O.silu(g) * u)
        h = _h(h.astype(np.float32) + _h(O.mm_ref_f64(act, lw["wd"])).astype(np.float32))
    xn = _rms(h, norm_final, eps)
    logits = _h(O.mm_ref_f64(xn, head_w))
    return logits, logits.astype(np.float32).argmax(-1), h

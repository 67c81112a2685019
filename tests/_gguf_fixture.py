"""Writes a tiny Llama-architecture GGUF with ``gguf.GGUFWriter`` (the package the reference reads
checkpoints with) from seeded synthetic blocks; returns the rotate-half-order arrays it holds."""

import numpy as np

from alloy_b200 import synth

TINY_META = dict(layers=2, hidden=512, ffn=1024, heads=8, kv_heads=2, head_dim=64, vocab=640,
                 rope_theta=10000.0, eps=1e-5)


def permute_rows(w: np.ndarray, n_head: int) -> np.ndarray:
    """llama.cpp's checkpoint order of q/k rows (interleaved RoPE), applied to packed rows."""
    n = w.shape[0]
    return w.reshape(n_head, 2, n // n_head // 2, w.shape[1]).swapaxes(1, 2).reshape(n, w.shape[1])


def write_tiny_llama(path, seed: int = 0, tied_head: bool = True, d_scale: float = 0.05):
    import gguf
    from gguf import GGMLQuantizationType as T

    m = TINY_META
    rng = np.random.default_rng(seed)
    hd, kvd = m["heads"] * m["head_dim"], m["kv_heads"] * m["head_dim"]

    def q4(n, k):
        b = synth.q4k_blocks(rng, n, k)
        v = b.reshape(n, k // 256, 144)
        for off in (0, 2):                         # d, dmin scaled down: activations stay in fp16 range
            h = v[:, :, off:off + 2].copy().view(np.float16).astype(np.float32) * d_scale
            v[:, :, off:off + 2] = h.astype(np.float16).view(np.uint8)
        return np.ascontiguousarray(v.reshape(n, -1))

    def q6(n, k):
        b = synth.q6k_blocks(rng, n, k)
        v = b.reshape(n, k // 256, 210)
        h = v[:, :, 208:210].copy().view(np.float16).astype(np.float32) * d_scale
        v[:, :, 208:210] = h.astype(np.float16).view(np.uint8)
        return np.ascontiguousarray(v.reshape(n, -1))

    arrays = {"embed": ("q4_k", q4(m["vocab"], m["hidden"])), "layers": []}
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_block_count(m["layers"])
    w.add_embedding_length(m["hidden"])
    w.add_feed_forward_length(m["ffn"])
    w.add_head_count(m["heads"])
    w.add_head_count_kv(m["kv_heads"])
    w.add_rope_freq_base(m["rope_theta"])
    w.add_layer_norm_rms_eps(m["eps"])
    w.add_vocab_size(m["vocab"])
    w.add_context_length(256)
    w.add_tensor("token_embd.weight", arrays["embed"][1], raw_dtype=T.Q4_K)
    TY = {"q4_k": T.Q4_K, "q6_k": T.Q6_K}
    for i in range(m["layers"]):
        # like Q4_K_M checkpoints, v / down are Q6_K in some layers and Q4_K in others
        fv = "q6_k" if i % 2 == 0 else "q4_k"
        mk = {"q4_k": q4, "q6_k": q6}
        lay = {
            "wq": ("q4_k", q4(hd, m["hidden"])), "wk": ("q4_k", q4(kvd, m["hidden"])),
            "wv": (fv, mk[fv](kvd, m["hidden"])), "wo": ("q4_k", q4(m["hidden"], hd)),
            "wg": ("q4_k", q4(m["ffn"], m["hidden"])), "wu": ("q4_k", q4(m["ffn"], m["hidden"])),
            "wd": (fv, mk[fv](m["hidden"], m["ffn"])),
            "norm_in": (1.0 + 0.02 * rng.standard_normal(m["hidden"])).astype(np.float32),
            "norm_post": (1.0 + 0.02 * rng.standard_normal(m["hidden"])).astype(np.float32),
        }
        arrays["layers"].append(lay)
        p = f"blk.{i}."
        w.add_tensor(p + "attn_q.weight", permute_rows(lay["wq"][1], m["heads"]), raw_dtype=T.Q4_K)
        w.add_tensor(p + "attn_k.weight", permute_rows(lay["wk"][1], m["kv_heads"]), raw_dtype=T.Q4_K)
        w.add_tensor(p + "attn_v.weight", lay["wv"][1], raw_dtype=TY[fv])
        w.add_tensor(p + "attn_output.weight", lay["wo"][1], raw_dtype=T.Q4_K)
        w.add_tensor(p + "ffn_gate.weight", lay["wg"][1], raw_dtype=T.Q4_K)
        w.add_tensor(p + "ffn_up.weight", lay["wu"][1], raw_dtype=T.Q4_K)
        w.add_tensor(p + "ffn_down.weight", lay["wd"][1], raw_dtype=TY[fv])
        w.add_tensor(p + "attn_norm.weight", lay["norm_in"])
        w.add_tensor(p + "ffn_norm.weight", lay["norm_post"])
    arrays["norm_final"] = (1.0 + 0.02 * rng.standard_normal(m["hidden"])).astype(np.float32)
    w.add_tensor("output_norm.weight", arrays["norm_final"])
    if tied_head:
        arrays["head"] = arrays["embed"]
    else:
        arrays["head"] = ("q6_k", q6(m["vocab"], m["hidden"]))
        w.add_tensor("output.weight", arrays["head"][1], raw_dtype=T.Q6_K)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return arrays

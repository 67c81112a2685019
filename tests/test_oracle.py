"""The CPU oracle against the committed golden vectors (bit-exact) and, where the
``gguf`` package is importable, against ``gguf.quants.dequantize`` on fresh
seeded blocks of the benchmark distribution."""

import numpy as np
import pytest

from alloy_b200 import synth
from oracle import blocks as O


def _same_bits(a, b):
    assert a.dtype == b.dtype == np.float32
    return np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_q4k_golden(golden):
    g = golden["q4k"]
    assert _same_bits(O.dequant_q4_k(g["blocks_signed"]), g["w_signed"])
    assert _same_bits(O.dequant_q4_k(g["blocks"]), g["w"])
    assert _same_bits(O.dequant_q4_k_scalar(g["blocks"][:2]), g["w"][:2])
    np.testing.assert_allclose(O.mm_ref(g["x"], g["w"]), g["y"], rtol=1e-5, atol=1e-5)


def test_q6k_golden(golden):
    g = golden["q6k"]
    assert _same_bits(O.dequant_q6_k(g["blocks"]), g["w"])


def test_q8_0_golden(golden):
    g = golden["q8_0"]
    codes, scales = O.split_q8_0(g["wire"])
    assert codes.dtype == np.int8 and scales.dtype == np.float16
    assert _same_bits(O.dequant_q8_0(codes, scales), g["w"])


def test_kv_q8_golden(golden):
    g = golden["kv_q8"]
    for name in ("k", "v"):
        codes, scales = O.kv_quantize_q8_0(g[name])
        assert np.array_equal(codes, g[f"{name}_codes"])
        assert np.array_equal(scales.view(np.uint16), g[f"{name}_scales"].view(np.uint16))
    # planted cases: zero block, and exact .5 ties rounding away from zero
    assert g["k_scales"][0, 0, 0] == 0 and not g["k_codes"][0, 0, :32].any()
    assert g["k_codes"][1, 3, 33] == 3 and g["k_codes"][1, 3, 34] == -1


def test_kv_pack_roundtrip(golden):
    g = golden["kv_q8"]
    raw = O.kv_pack_blocks(g["k_codes"], g["k_scales"])
    assert raw.shape[-1] == 128 // 32 * 34
    c, s = O.kv_unpack_blocks(raw)
    assert np.array_equal(c, g["k_codes"]) and np.array_equal(s, g["k_scales"])


def test_kv_q8_requantise_idempotent(golden):
    g = golden["kv_q8"]
    deq = O.kv_dequant_q8_0(g["k_codes"], g["k_scales"]).astype(np.float16)
    c2, s2 = O.kv_quantize_q8_0(deq)
    d2 = O.kv_dequant_q8_0(c2, s2).astype(np.float16)
    c3, s3 = O.kv_quantize_q8_0(d2)
    assert np.array_equal(c2, c3) and np.array_equal(s2, s3)


def test_attention_golden(golden):
    g = golden["kv_q8"]
    dk = O.kv_dequant_q8_0(g["k_codes"], g["k_scales"])
    dv = O.kv_dequant_q8_0(g["v_codes"], g["v_scales"])
    out = O.attention_decode_ref(dk, dv, g["q"].astype(np.float32), int(g["pos"]))
    np.testing.assert_allclose(out, g["attn"], rtol=1e-12, atol=1e-12)


def test_gather_pages():
    rng = np.random.default_rng(0)
    pool = rng.integers(0, 255, size=(7, 2, 4, 3), dtype=np.uint8)
    ids = [5, 0, 3]
    got = O.gather_pages(pool, ids, 10)
    assert got.shape == (2, 10, 3)
    assert np.array_equal(got[1, 4:8], pool[0, 1])
    assert np.array_equal(got[0, 8:10], pool[3, 0, :2])


@pytest.mark.parametrize("fmt", ["q4k", "q6k", "q8_0"])
def test_against_gguf_package(fmt):
    gguf = pytest.importorskip("gguf")
    from gguf.quants import dequantize
    T = gguf.GGMLQuantizationType
    rng = np.random.default_rng(11)
    if fmt == "q4k":
        b = synth.q4k_blocks(rng, 32, 1024)
        ref = dequantize(b.reshape(-1, 144), T.Q4_K).reshape(32, 1024)
        got = O.dequant_q4_k(b)
    elif fmt == "q6k":
        b = synth.q6k_blocks(rng, 32, 1024)
        ref = dequantize(b.reshape(-1, 210), T.Q6_K).reshape(32, 1024)
        got = O.dequant_q6_k(b)
    else:
        b = synth.q8_0_wire(rng, 32, 1024)
        ref = dequantize(b.reshape(-1, 34), T.Q8_0).reshape(32, 1024)
        got = O.dequant_q8_0(*O.split_q8_0(b))
    assert _same_bits(got, ref.astype(np.float32))


def test_q5_0_golden(golden):
    """Q5_0: the oracle's wire split equals the reference's own split_q5_0_weight, and its decode of
    the three buffers equals gguf's decode of the wire blocks, bit for bit."""
    g = golden["q5_0"]
    qw, qh, sc = O.split_q5_0(g["wire"])
    assert np.array_equal(qw, g["qweight"]) and np.array_equal(qh, g["qhigh"])
    assert np.array_equal(sc.view(np.uint16), g["scales"].view(np.uint16))
    w = O.dequant_q5_0(qw, qh, sc)
    assert w.dtype == np.float32 and np.array_equal(w.view(np.uint32), g["w"].view(np.uint32))


def test_attention_chunk_golden(golden):
    """Causal chunk attention: the oracle against the reference's _ref_attention applied per query row."""
    g = golden["attn_chunk"]
    kc, ks = O.kv_quantize_q8_0(g["k"])
    vc, vs = O.kv_quantize_q8_0(g["v"])
    out = O.attention_chunk_ref(O.kv_dequant_q8_0(kc, ks), O.kv_dequant_q8_0(vc, vs),
                                g["q"].astype(np.float32), int(g["start"]))
    assert out.shape == g["attn"].shape
    assert np.abs(out - g["attn"]).max() < 1e-12


def test_moe_router_identity_and_composition():
    """softmax over the top-k raw logits == renormalised top-k of the full softmax (the identity the
    reference's router relies on), and a one-expert, top-1 routed op equals the plain gated MLP."""
    import torch

    rng = np.random.default_rng(11)
    t_n, e_n, k = 5, 16, 4
    logits = rng.standard_normal((t_n, e_n)).astype(np.float32)
    p = torch.softmax(torch.from_numpy(logits).double(), -1)
    top, idx = torch.topk(p, k, dim=-1)
    w_hf = (top / top.sum(-1, keepdim=True)).numpy()
    for t in range(t_n):
        order = np.lexsort((np.arange(e_n), -logits[t].astype(np.float64)))[:k]
        assert order.tolist() == idx[t].tolist()
        sel = logits[t, order].astype(np.float64)
        w = np.exp(sel - sel[0])
        assert np.allclose(w / w.sum(), w_hf[t], rtol=1e-12, atol=0)
    hdim, inter = 256, 256
    gu = synth.q4k_blocks(rng, 2 * inter, hdim)[None]
    dn = synth.q6k_blocks(rng, hdim, inter)[None]
    x = rng.standard_normal((2, hdim)).astype(np.float32)
    y = O.moe_routed_ref(x, np.zeros((2, 1), np.float32), gu, dn, 1, inter)
    wgu = O.dequant_q4_k(gu[0]).astype(np.float64)
    h = (O.silu(wgu[:inter] @ x.T.astype(np.float64)) * (wgu[inter:] @ x.T.astype(np.float64))).astype(np.float32)
    ref = (O.dequant_q6_k(dn[0]).astype(np.float64) @ h.astype(np.float64)).T
    assert np.allclose(y, ref, rtol=1e-12, atol=1e-12)

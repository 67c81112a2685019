"""GPU parity: q8_0 KV quantise/append (bit-exact) and decode attention (tolerance)
vs the oracle, through torch.ops.alloy.* and the C ABI."""

import ctypes as C

import numpy as np
import pytest
import torch

from alloy_b200 import _lib, kv, ops, synth
from oracle import blocks as O
from tests._util import assert_close, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _quantize_range(src, codes, scales, start, n):
    b, h, s_max, d = codes.shape
    L = _lib.load()
    _lib.check(L.alloyb_kv_quantize_q8(src.data_ptr(), src.stride(0), src.stride(1), src.stride(2),
                                       codes.data_ptr(), scales.data_ptr(), b, h, s_max, d, start, n,
                                       torch.cuda.current_stream().cuda_stream), "kv_quantize")


def test_kv_quantize_golden_bit_exact(golden):
    g = golden["kv_q8"]
    h, s, d = g["k"].shape
    for name in ("k", "v"):
        src = _dev(g[name]).reshape(1, h, s, d)
        codes = torch.full((1, h, 64, d), 99, dtype=torch.int8, device=DEV)
        scales = torch.full((1, h, 64, d // 32), 7.0, dtype=torch.float16, device=DEV)
        _quantize_range(src, codes, scales, 5, s)
        assert np.array_equal(codes[0, :, 5:5 + s].cpu().numpy(), g[f"{name}_codes"])
        assert np.array_equal(scales[0, :, 5:5 + s].cpu().numpy().view(np.uint16),
                              g[f"{name}_scales"].view(np.uint16))
        # rows outside [start, start+n) untouched
        assert (codes[0, :, :5] == 99).all() and (codes[0, :, 5 + s:] == 99).all()
        assert (scales[0, :, :5] == 7.0).all()


def test_kv_quantize_seeded_strided_and_dequant():
    rng = np.random.default_rng(3)
    b, h, s, d = 2, 3, 37, 128
    big = synth.kv_rows(rng, (b, s, h, d), 3.0)          # (B, S, H, D) storage, viewed (B, H, S, D)
    big[0, 0, 0, :32] = 0
    src = _dev(big).permute(0, 2, 1, 3)
    codes = torch.zeros((b, h, 48, d), dtype=torch.int8, device=DEV)
    scales = torch.zeros((b, h, 48, d // 32), dtype=torch.float16, device=DEV)
    _quantize_range(src, codes, scales, 0, s)
    rc, rs = O.kv_quantize_q8_0(big.transpose(0, 2, 1, 3))
    assert np.array_equal(codes[:, :, :s].cpu().numpy(), rc)
    assert np.array_equal(scales[:, :, :s].cpu().numpy().view(np.uint16), rs.view(np.uint16))
    out = torch.zeros((b, h, 48, d), dtype=torch.float16, device=DEV)
    L = _lib.load()
    _lib.check(L.alloyb_kv_dequant_q8(codes.data_ptr(), scales.data_ptr(), out.data_ptr(), b, h, 48, d,
                                      s, torch.cuda.current_stream().cuda_stream), "kv_dequant")
    ref = O.kv_dequant_q8_0(rc, rs).astype(np.float16)
    assert np.array_equal(out[:, :, :s].cpu().numpy().view(np.uint16), ref.view(np.uint16))
    assert not out[:, :, s:].any()
    # round-trip bound of the reference's test: |x - deq| <= d*(1/2 + 127*2^-11) + |x|*2^-10
    x = big.transpose(0, 2, 1, 3).astype(np.float32)
    dd = np.repeat(rs.astype(np.float32), 32, axis=-1)
    assert (np.abs(x - ref.astype(np.float32)) <= dd * (0.5 + 127 * 2.0**-11) + np.abs(x) * 2.0**-10).all()


def _ref_decode(k_rows, v_rows, q, pos_list, scale=None):
    """k_rows/v_rows: per sequence (KV_H, S, D) fp32 dequantised; q (B,H,D)."""
    return np.stack([O.attention_decode_ref(k_rows[b], v_rows[b], q[b], pos_list[b], scale)
                     for b in range(q.shape[0])])


@pytest.mark.parametrize("d,group,kv_h,s_max,pos", [(128, 4, 2, 512, 400), (64, 2, 2, 512, 400),
                                                     (128, 1, 3, 256, 0), (256, 8, 1, 512, 511),
                                                     (128, 4, 8, 2048, 2047)])
def test_attention_cache_q8_fused_write(d, group, kv_h, s_max, pos):
    rng = np.random.default_rng([d, group, pos])
    b, h = 2, kv_h * group
    hist_k = synth.kv_rows(rng, (b, kv_h, s_max, d), 2.0)
    hist_v = synth.kv_rows(rng, (b, kv_h, s_max, d), 2.0)
    kc, ks = O.kv_quantize_q8_0(hist_k)
    vc, vs = O.kv_quantize_q8_0(hist_v)
    new_k = synth.kv_rows(rng, (b, kv_h, 1, d), 2.0)
    new_v = synth.kv_rows(rng, (b, kv_h, 1, d), 2.0)
    q = synth.activations(rng, b * h, d).reshape(b, h, 1, d)
    t = [_dev(a) for a in (kc, ks, vc, vs)]
    out = torch.ops.alloy.attention_cache_q8(_dev(q), _dev(new_k), _dev(new_v),
                                             torch.tensor([pos], device=DEV), *t)
    assert out.shape == (b, h, 1, d) and out.dtype == torch.float16
    # the write is bit-exact and only touches row `pos`
    nkc, nks = O.kv_quantize_q8_0(new_k)
    nvc, nvs = O.kv_quantize_q8_0(new_v)
    kc2, ks2, vc2, vs2 = kc.copy(), ks.copy(), vc.copy(), vs.copy()
    kc2[:, :, pos], ks2[:, :, pos] = nkc[:, :, 0], nks[:, :, 0]
    vc2[:, :, pos], vs2[:, :, pos] = nvc[:, :, 0], nvs[:, :, 0]
    for got, ref in zip(t, (kc2, ks2, vc2, vs2)):
        assert np.array_equal(got.cpu().numpy().view(np.uint8), ref.view(np.uint8))
    ref = _ref_decode(O.kv_dequant_q8_0(kc2, ks2), O.kv_dequant_q8_0(vc2, vs2), q[:, :, 0], [pos] * b)
    assert np.abs(to_np(out)[:, :, 0] - ref).max() < 2e-3          # the reference test's bound
    assert_close(to_np(out)[:, :, 0], ref, torch.float16, "attention_cache_q8")


def test_attention_golden(golden):
    g = golden["kv_q8"]
    kv_h, s, d = g["k"].shape
    pos, group = int(g["pos"]), int(g["group"])
    t = [_dev(g[n][None]) for n in ("k_codes", "k_scales", "v_codes", "v_scales")]
    q = _dev(g["q"]).reshape(1, kv_h * group, 1, d).float()   # fp32 in/out like the reference test
    dummy = torch.zeros((1, kv_h, 1, d), dtype=torch.float16, device=DEV)
    out = torch.ops.alloy.attention_cache_q8(q, dummy, dummy, torch.tensor([pos], device=DEV), *t,
                                             write_kv=False)
    assert out.dtype == torch.float32
    assert np.abs(to_np(out)[0, :, 0] - g["attn"]).max() < 2e-3
    out16 = torch.ops.alloy.attention_cache_q8(q.half(), dummy, dummy, torch.tensor([pos], device=DEV),
                                               *t, write_kv=False)
    assert_close(to_np(out16)[0, :, 0], g["attn"], torch.float16, "golden attention fp16")


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_attention_cache_f16(dtype):
    rng = np.random.default_rng(9)
    b, kv_h, group, d, s_max, pos = 3, 2, 4, 128, 300, 257
    h = kv_h * group
    k = synth.kv_rows(rng, (b, kv_h, s_max, d))
    v = synth.kv_rows(rng, (b, kv_h, s_max, d))
    new_k = synth.kv_rows(rng, (b, 1, kv_h, d))
    new_v = synth.kv_rows(rng, (b, 1, kv_h, d))
    q = synth.activations(rng, b * h, d).reshape(b, h, 1, d)
    kd, vd = _dev(k), _dev(v)
    # new_k/new_v arrive as transposed views of (B, 1, KV_H, D), as the model produces them
    out = torch.ops.alloy.attention_cache(_dev(q).to(dtype), _dev(new_k).transpose(1, 2),
                                          _dev(new_v).transpose(1, 2),
                                          torch.tensor([pos], device=DEV, dtype=torch.int64), kd, vd,
                                          1.0 / np.sqrt(d))
    k2, v2 = k.copy(), v.copy()
    k2[:, :, pos], v2[:, :, pos] = new_k[:, 0], new_v[:, 0]
    assert np.array_equal(kd.cpu().numpy().view(np.uint16), k2.view(np.uint16))
    assert np.array_equal(vd.cpu().numpy().view(np.uint16), v2.view(np.uint16))
    ref = _ref_decode(k2.astype(np.float32), v2.astype(np.float32), q[:, :, 0], [pos] * b)
    assert out.dtype == dtype
    assert_close(to_np(out)[:, :, 0], ref, dtype, "attention_cache f16")


def _build_paged(rng, b, kv_h, d, lens, extra_pages=5):
    """Random page placement; returns pool store, the oracle's per-sequence rows."""
    pages_per = [(n + 1 + 15) // 16 for n in lens]
    total = sum(pages_per) + extra_pages
    order = rng.permutation(total).tolist()
    store = kv.PagedKVPool(total, kv_h, d, b, max(pages_per), DEV, free_order=order)
    host = np.zeros(tuple(store.pool.shape), np.uint8)
    seq_rows = []
    for s in range(b):
        store.reserve(s, lens[s] + 1)
        n_tok = pages_per[s] * 16
        k = synth.kv_rows(rng, (kv_h, n_tok, d), 1.0)
        v = synth.kv_rows(rng, (kv_h, n_tok, d), 1.0)
        kc, ks = O.kv_quantize_q8_0(k)
        vc, vs = O.kv_quantize_q8_0(v)
        kraw, vraw = O.kv_pack_blocks(kc, ks), O.kv_pack_blocks(vc, vs)
        for i, pg in enumerate(store.pages_of(s)):
            host[pg, 0] = kraw[:, i * 16:(i + 1) * 16]
            host[pg, 1] = vraw[:, i * 16:(i + 1) * 16]
        seq_rows.append((kc, ks, vc, vs))
    store.pool.copy_(torch.from_numpy(host))
    return store, host, seq_rows


@pytest.mark.parametrize("b,kv_h,group,d,lo,hi", [(4, 2, 4, 128, 1, 700), (3, 8, 4, 128, 900, 2100),
                                                   (2, 1, 8, 64, 15, 17)])
def test_attention_paged_q8(b, kv_h, group, d, lo, hi):
    rng = np.random.default_rng([b, kv_h, hi])
    h = kv_h * group
    lens = rng.integers(lo, hi + 1, size=b).tolist()     # tokens already cached; new token at pos=len
    store, host, seq_rows = _build_paged(rng, b, kv_h, d, lens)
    new_k = synth.kv_rows(rng, (b, kv_h, 1, d))
    new_v = synth.kv_rows(rng, (b, kv_h, 1, d))
    q = synth.activations(rng, b * h, d).reshape(b, h, 1, d)
    pos = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.ops.alloy.attention_cache_q8_paged(_dev(q), _dev(new_k), _dev(new_v), pos,
                                                   store.page_table, store.pool)
    assert ops.attn_status(ops.attn_workspace(torch.device(DEV, 0), b, h, d)) == 0
    nkc, nks = O.kv_quantize_q8_0(new_k)
    nvc, nvs = O.kv_quantize_q8_0(new_v)
    got_pool = store.pool.cpu().numpy()
    k_rows, v_rows = [], []
    for s in range(b):
        kc, ks, vc, vs = (a.copy() for a in seq_rows[s])
        p = lens[s]
        kc[:, p], ks[:, p], vc[:, p], vs[:, p] = nkc[s, :, 0], nks[s, :, 0], nvc[s, :, 0], nvs[s, :, 0]
        pg = store.pages_of(s)[p // 16]
        host[pg, 0, :, p % 16] = O.kv_pack_blocks(nkc[s, :, 0], nks[s, :, 0])
        host[pg, 1, :, p % 16] = O.kv_pack_blocks(nvc[s, :, 0], nvs[s, :, 0])
        k_rows.append(O.kv_dequant_q8_0(kc, ks))
        v_rows.append(O.kv_dequant_q8_0(vc, vs))
    assert np.array_equal(got_pool, host)                 # append bit-exact, nothing else touched
    # the oracle gathers pages to contiguous rows and runs the same attention math
    s0 = 0
    gathered = O.gather_pages(got_pool[:, 0], store.pages_of(s0), lens[s0] + 1)
    gc, gs = O.kv_unpack_blocks(gathered)
    assert np.array_equal(O.kv_dequant_q8_0(gc, gs), k_rows[s0][:, :lens[s0] + 1])
    ref = _ref_decode(k_rows, v_rows, q[:, :, 0], lens)
    assert np.abs(to_np(out)[:, :, 0] - ref).max() < 2e-3
    assert_close(to_np(out)[:, :, 0], ref, torch.float16, "paged q8")


def test_attention_paged_q8_full_size_properties():
    """Batch 64, contexts 4096..32768 (2.4 GB of q8_0 KV): properties that need no CPU reference.

    1. Physical page placement does not matter: the same sequences stored under another page
       permutation give bit-identical outputs.
    2. With every V row of a head equal to one vector, the output is that vector for every query
       (the softmax weights sum to one), whatever K holds.
    """
    from alloy_b200.kv import PagedKVPool
    b, kv_h, group, d = 64, 8, 4, 128
    cpu = torch.Generator().manual_seed(5)
    gen = torch.Generator(device=DEV).manual_seed(5)
    lens = torch.randint(4096, 32768 + 1, (b,), generator=cpu)
    pages_per = [(int(n) + 16) // 16 for n in lens]
    total = sum(pages_per)
    order = torch.randperm(total, generator=cpu).tolist()
    store = PagedKVPool(total, kv_h, d, b, max(pages_per), DEV, free_order=order)
    for i in range(b):
        store.reserve(i, int(lens[i]) + 1)
    store.pool.copy_(torch.randint(0, 256, store.pool.shape, dtype=torch.uint8, device=DEV, generator=gen))
    blocks = store.pool.view(-1, 34)
    sc = torch.empty(blocks.shape[0], device=DEV).uniform_(0.015, 0.03, generator=gen).half()
    blocks[:, 0:2] = sc.view(torch.uint8).view(-1, 2)
    h = kv_h * group
    q = torch.randn((b, h, 1, d), device=DEV, generator=gen).half()
    nk = torch.randn((b, kv_h, 1, d), device=DEV, generator=gen).half()
    nv = torch.randn((b, kv_h, 1, d), device=DEV, generator=gen).half()
    pos = lens.to(torch.int32).to(DEV)
    base_pool = store.pool.clone()
    out1 = torch.ops.alloy.attention_cache_q8_paged(q, nk, nv, pos, store.page_table, store.pool).clone()
    assert torch.isfinite(out1.float()).all()

    # 0. the float64 oracle on sampled (sequence, query head) pairs, the shortest and the longest
    #    sequence among them: pages gathered from the pool as the call left it (new token appended)
    order_by_len = torch.argsort(lens).tolist()
    picks = [(order_by_len[0], 0), (order_by_len[0], h - 1), (order_by_len[-1], 5), (order_by_len[-1], 30),
             (order_by_len[b // 2], 17), (7, 9), (40, 22)]
    out_np = out1.float().cpu().numpy()
    for seq, head in picks:
        n_tok = int(lens[seq]) + 1
        kvh = head // group
        pages = torch.tensor(store.pages_of(seq), device=DEV)
        slabs = store.pool[pages][:, :, kvh].cpu().numpy()                # (P, 2, 16, 136)
        rows = []
        for which in (0, 1):
            raw = slabs[:, which].reshape(-1, slabs.shape[-1])[:n_tok]    # (tokens, 136)
            c, sc_ = O.kv_unpack_blocks(raw)
            rows.append(O.kv_dequant_q8_0(c, sc_)[None])                  # (1, tokens, D)
        ref = O.attention_decode_ref(rows[0], rows[1], q[seq, head, 0].float().cpu().numpy()[None], n_tok - 1)
        assert np.abs(out_np[seq, head, 0] - ref[0]).max() < 2e-3, (seq, head)
        assert_close(out_np[seq, head, 0], ref[0], torch.float16, f"full-size paged, sequence {seq} head {head}")

    # 1. another physical placement of the same pages
    perm = torch.randperm(total, generator=cpu).to(DEV)
    pool2 = torch.empty_like(base_pool)
    pool2[perm] = base_pool
    table2 = store.page_table.clone()
    valid = table2 >= 0
    table2[valid] = perm[table2[valid].long()].to(table2.dtype)
    out2 = torch.ops.alloy.attention_cache_q8_paged(q, nk, nv, pos, table2, pool2)
    assert torch.equal(out1, out2)
    del pool2

    # 2. constant V rows per head: one q8_0 row (4 blocks of 34 bytes) repeated over all tokens
    store.pool.copy_(base_pool)
    row = store.pool[0, 1, :, 0].clone()                                  # (kv_h, 136) of page 0, V slab
    store.pool[:, 1] = row[None, :, None, :]
    nv_const = torch.empty((kv_h, d), device=DEV)
    rb = row.view(kv_h, 4, 34)
    scale = rb[:, :, 0:2].contiguous().view(torch.float16).float()        # (kv_h, 4, 1)
    codes = rb[:, :, 2:].contiguous().view(torch.int8).float()            # (kv_h, 4, 32)
    vconst = (codes * scale).reshape(kv_h, d)                             # dequantised V row per head
    # the appended token's V must be that vector too: pass the dequantised row (it re-quantises to itself)
    nv2 = vconst.half()[None, :, None, :].expand(b, kv_h, 1, d).contiguous()
    out3 = torch.ops.alloy.attention_cache_q8_paged(q, nk, nv2, pos, store.page_table, store.pool)
    want = vconst[:, None, :].expand(kv_h, group, d).reshape(1, h, 1, d).expand(b, h, 1, d)
    err = (out3.float() - want).abs().max() / want.abs().max()
    assert float(err) < 2e-3, float(err)


@pytest.mark.parametrize("layout", ["f16", "q8_split", "paged"])
def test_rope_kv_append_equals_rope_then_append(layout):
    """The fused RoPE + append launch leaves q and the cache exactly as rope_inplace followed by the
    attention op's own append does (bit-identical), and attention with write_kv=False then matches."""
    rng = np.random.default_rng(len(layout))
    b, kv_h, group, d, s_max = 3, 2, 4, 128, 256
    h = kv_h * group
    lens = [17, 200, 64]
    q = torch.from_numpy(synth.activations(rng, b * h, d).reshape(b, h, d)).to(DEV)
    nk = torch.from_numpy(synth.kv_rows(rng, (b, kv_h, d))).to(DEV)
    nv = torch.from_numpy(synth.kv_rows(rng, (b, kv_h, d))).to(DEV)
    inv = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    pos = torch.tensor(lens, dtype=torch.int32, device=DEV)

    def caches():
        g = torch.Generator(device=DEV).manual_seed(7)
        if layout == "f16":
            return [torch.randn((b, kv_h, s_max, d), device=DEV, generator=g).half() for _ in range(2)]
        if layout == "q8_split":
            mk = lambda: (torch.randint(-127, 128, (b, kv_h, s_max, d), device=DEV, generator=g, dtype=torch.int8),
                          torch.rand((b, kv_h, s_max, d // 32), device=DEV, generator=g).mul(0.02).half())
            (kc, ks), (vc, vs) = mk(), mk()
            return [kc, ks, vc, vs]
        store = kv.PagedKVPool(b * (s_max // 16), kv_h, d, b, s_max // 16, DEV)
        for i in range(b):
            store.reserve(i, lens[i] + 1)
        store.pool.copy_(torch.randint(0, 256, store.pool.shape, dtype=torch.uint8, device=DEV, generator=g))
        blk = store.pool.view(-1, 34)
        blk[:, 0:2] = torch.full((blk.shape[0],), 0.02, device=DEV).half().view(torch.uint8).view(-1, 2)
        return [store]

    def attend(qr, kr, c, write):
        q4, k4, v4 = qr.unsqueeze(2), kr.unsqueeze(2), nv.unsqueeze(2)
        if layout == "f16":                      # one shared position for the fp16 op: use sequence 0's
            return torch.ops.alloy.attention_cache(q4, k4, v4, pos[:1], c[0], c[1], -1.0, 0, write)
        if layout == "q8_split":
            return torch.ops.alloy.attention_cache_q8(q4, k4, v4, pos[:1], c[0], c[1], c[2], c[3], -1.0, 0, write)
        return torch.ops.alloy.attention_cache_q8_paged(q4, k4, v4, pos, c[0].page_table, c[0].pool, -1.0, write)

    p_arg = pos if layout == "paged" else pos[:1]
    # two steps: rope, then the op's own append
    c1 = caches()
    q1, k1 = q.clone(), nk.clone()
    ops.rope_inplace(q1, k1, p_arg, inv)
    out1 = attend(q1, k1, c1, True)
    # fused
    c2 = caches()
    q2 = q.clone()
    if layout == "f16":
        ops.rope_kv_append(q2, nk, nv, p_arg, inv, k_cache=c2[0], v_cache=c2[1])
    elif layout == "q8_split":
        ops.rope_kv_append(q2, nk, nv, p_arg, inv, q8_split=tuple(c2))
    else:
        ops.rope_kv_append(q2, nk, nv, p_arg, inv, paged=(c2[0].page_table, c2[0].pool))
    out2 = attend(q2, nk, c2, False)
    assert torch.equal(q1, q2)
    a = [t if isinstance(t, torch.Tensor) else t.pool for t in c1]
    bb = [t if isinstance(t, torch.Tensor) else t.pool for t in c2]
    for x, y in zip(a, bb):
        assert torch.equal(x, y)
    assert torch.equal(out1, out2)
    # all three steps in one launch: same cache, same output, q left unrotated
    c3 = caches()
    q3 = q.clone()
    if layout == "f16":
        out3 = ops.rope_attention_decode(q3, nk, nv, p_arg, inv, k_cache=c3[0], v_cache=c3[1])
    elif layout == "q8_split":
        out3 = ops.rope_attention_decode(q3, nk, nv, p_arg, inv, q8_split=tuple(c3))
    else:
        out3 = ops.rope_attention_decode(q3, nk, nv, p_arg, inv, paged=(c3[0].page_table, c3[0].pool))
    assert torch.equal(q3, q)
    for x, y in zip(a, [t if isinstance(t, torch.Tensor) else t.pool for t in c3]):
        assert torch.equal(x, y)
    assert torch.equal(out1.squeeze(2), out3)


def test_paged_append_entry_and_bad_page_is_skipped():
    rng = np.random.default_rng(5)
    b, kv_h, d = 2, 2, 128
    store = kv.PagedKVPool(8, kv_h, d, b, 2, DEV)
    store.reserve(0, 20)
    store.reserve(1, 3)
    new_k = _dev(synth.kv_rows(rng, (b, kv_h, d)))
    new_v = _dev(synth.kv_rows(rng, (b, kv_h, d)))
    pos = torch.tensor([19, 2], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    L = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    args = (new_k.data_ptr(), new_v.data_ptr(), new_k.stride(0), new_k.stride(1), store.pool.data_ptr(),
            store.page_table.data_ptr(), 2, 8, pos.data_ptr(), b, kv_h, d, status.data_ptr(), st)
    _lib.check(L.alloyb_kv_append_q8_paged(*args), "append")
    assert int(status.item()) == 0
    kc, ks = O.kv_quantize_q8_0(new_k.cpu().numpy())
    pg = store.pages_of(0)[1]
    assert np.array_equal(store.pool[pg, 0, :, 3].cpu().numpy(), O.kv_pack_blocks(kc[0], ks[0]))
    # sequence 1 asks for position 20 whose page is unmapped (-1): skipped, flagged, no fault
    before = store.pool.clone()
    pos2 = torch.tensor([19, 20], dtype=torch.int32, device=DEV)
    args2 = args[:8] + (pos2.data_ptr(),) + args[9:]
    _lib.check(L.alloyb_kv_append_q8_paged(*args2), "append")
    assert int(status.item()) == 2
    assert torch.equal(before[store.pages_of(1)[0]], store.pool[store.pages_of(1)[0]])


def test_attention_argument_errors():
    q = torch.zeros((1, 4, 1, 100), dtype=torch.float16, device=DEV)
    z = torch.zeros((1, 2, 1, 100), dtype=torch.float16, device=DEV)
    c = torch.zeros((1, 2, 8, 100), dtype=torch.int8, device=DEV)
    s = torch.zeros((1, 2, 8, 3), dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        torch.ops.alloy.attention_cache_q8(q, z, z, torch.tensor([0], device=DEV), c, s, c, s)
    with pytest.raises(ValueError):
        torch.ops.alloy.attention_cache_q8(q[0], z, z, torch.tensor([0], device=DEV), c, s, c, s)


@pytest.mark.parametrize("pos0", [0, 63, 64, 2047])
def test_rope_attention_decode_positions_and_fallback(pos0):
    """The one-launch attention step at the first position, at both sides of a split boundary and at the
    last position of the cache; a head_dim the fused kernel does not cover takes the two-launch route."""
    rng = np.random.default_rng(pos0)
    b, kv_h, group, s_max = 2, 2, 4, 2048
    for d in (128, 64):
        h = kv_h * group
        q = torch.from_numpy(synth.activations(rng, b * h, d).reshape(b, h, d)).to(DEV)
        nk = torch.from_numpy(synth.kv_rows(rng, (b, kv_h, d))).to(DEV)
        nv = torch.from_numpy(synth.kv_rows(rng, (b, kv_h, d))).to(DEV)
        inv = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
        pos = torch.tensor([pos0], dtype=torch.int32, device=DEV)
        g = torch.Generator(device=DEV).manual_seed(11)
        base = [torch.randn((b, kv_h, s_max, d), device=DEV, generator=g).half() for _ in range(2)]
        c1, c2 = [t.clone() for t in base], [t.clone() for t in base]
        q1 = q.clone()
        ops.rope_kv_append(q1, nk, nv, pos, inv, k_cache=c1[0], v_cache=c1[1])
        want = torch.ops.alloy.attention_cache(q1.unsqueeze(2), nk.unsqueeze(2), nv.unsqueeze(2), pos, c1[0], c1[1],
                                               -1.0, 0, False).squeeze(2)
        got = ops.rope_attention_decode(q, nk, nv, pos, inv, k_cache=c2[0], v_cache=c2[1])
        assert torch.equal(c1[0], c2[0]) and torch.equal(c1[1], c2[1])
        assert torch.equal(want, got)

"""GPU parity of the multi-token branches of the cache-attention ops: prefill chunks and the 2..16
token verify step over fp16, split-q8 and paged-q8 caches, against the float64 oracle."""

import numpy as np
import pytest
import torch

from alloy_b200 import kv, ops, synth
from oracle import blocks as O
from tests._util import assert_close, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _deq16(codes, scales):
    """What a chunk reads from a q8_0 cache: fp16(code * scale), the rounding of the reference's
    dequantise-to-scratch step (packages/alloy-metal/src/alloy/std/kv_quant.py:73-108)."""
    return O.kv_dequant_q8_0(codes, scales).astype(np.float16).astype(np.float32)


def test_attention_cache_q8_prefill_branch_reference_case():
    """The reference's own prefill case (tests/kernels/test_kv_quant.py:389-480): KV_H 2, group 2,
    D 64, S_MAX 512, 200 cached tokens, a 64-token chunk, cache_pos an arange, fp32 q.  The chunk
    is quantised into the caches; history AND chunk are read back from the codes."""
    kv_h, group, d, s_max, start, chunk = 2, 2, 64, 512, 200, 64
    heads = kv_h * group
    rng = np.random.default_rng(7)
    hist_k = (rng.standard_normal((kv_h, start, d)) * 2).astype(np.float16)
    hist_v = (rng.standard_normal((kv_h, start, d)) * 2).astype(np.float16)
    new_k = (rng.standard_normal((kv_h, chunk, d)) * 2).astype(np.float16)
    new_v = (rng.standard_normal((kv_h, chunk, d)) * 2).astype(np.float16)
    q = rng.standard_normal((heads, chunk, d)).astype(np.float32)
    caches = kv.alloc_quantized_kv(1, kv_h, s_max, d, DEV)
    hc_k, hs_k = O.kv_quantize_q8_0(hist_k)
    hc_v, hs_v = O.kv_quantize_q8_0(hist_v)
    caches[0][0, :, :start], caches[1][0, :, :start] = _dev(hc_k), _dev(hs_k)
    caches[2][0, :, :start], caches[3][0, :, :start] = _dev(hc_v), _dev(hs_v)
    pos = torch.arange(start, start + chunk, dtype=torch.int32, device=DEV)
    out = torch.ops.alloy.attention_cache_q8(_dev(q)[None], _dev(new_k)[None], _dev(new_v)[None], pos, *caches)
    assert out.shape == (1, heads, chunk, d) and out.dtype == torch.float32
    # durable write: the chunk's codes and scales sit at [start, start + chunk), bit-exact
    nc_k, ns_k = O.kv_quantize_q8_0(new_k)
    nc_v, ns_v = O.kv_quantize_q8_0(new_v)
    assert np.array_equal(caches[0][0, :, start:start + chunk].cpu().numpy(), nc_k)
    assert np.array_equal(caches[3][0, :, start:start + chunk].cpu().numpy().view(np.uint16), ns_v.view(np.uint16))
    assert not caches[0][0, :, start + chunk:].any()
    k_full = O.kv_dequant_q8_0(np.concatenate([hc_k, nc_k], 1), np.concatenate([hs_k, ns_k], 1))
    v_full = O.kv_dequant_q8_0(np.concatenate([hc_v, nc_v], 1), np.concatenate([hs_v, ns_v], 1))
    q16 = q.astype(np.float16).astype(np.float64)
    got = out[0].cpu().numpy()
    # the reference test's own yardstick and bound: unrounded code * scale, max abs < 2e-2
    assert np.abs(got - O.attention_chunk_ref(k_full, v_full, q16, start)).max() < 2e-2
    # the path's semantics (K/V rounded to fp16 as the reference's scratch holds them): parity tolerance
    kc, ksc = np.concatenate([hc_k, nc_k], 1), np.concatenate([hs_k, ns_k], 1)
    vc, vsc = np.concatenate([hc_v, nc_v], 1), np.concatenate([hs_v, ns_v], 1)
    assert_close(got, O.attention_chunk_ref(_deq16(kc, ksc), _deq16(vc, vsc), q16, start), torch.float32,
                 "q8 prefill branch")


def test_attention_chunk_golden_fixture(golden):
    """The committed reference-derived fixture, read-only attention over pre-filled q8 caches."""
    g = golden["attn_chunk"]
    kv_h, n, d = g["k"].shape
    start, group = int(g["start"]), int(g["group"])
    chunk = n - start
    kc, ks = O.kv_quantize_q8_0(g["k"])
    vc, vs = O.kv_quantize_q8_0(g["v"])
    caches = [_dev(a)[None] for a in (kc, ks, vc, vs)]
    dummy = torch.zeros((1, kv_h, chunk, d), dtype=torch.float16, device=DEV)
    out = torch.ops.alloy.attention_cache_q8(_dev(g["q"])[None], dummy, dummy,
                                             torch.tensor([start], device=DEV), *caches, -1.0, 0, False)
    assert np.array_equal(caches[0][0].cpu().numpy(), kc)                 # write_kv=False: untouched
    assert np.abs(to_np(out)[0] - g["attn"]).max() < 2e-2
    ref16 = O.attention_chunk_ref(_deq16(kc, ks), _deq16(vc, vs), g["q"].astype(np.float64), start)
    assert np.abs(ref16 - g["attn"]).max() < 5e-3          # the fp16 rounding of K/V is all that separates them
    assert_close(to_np(out)[0], ref16, torch.float16, "chunk golden")


@pytest.mark.parametrize("b,kv_h,group,d,start,chunk,dtype", [
    (2, 2, 4, 128, 300, 70, torch.float16),       # ragged chunk (not a tile multiple), D 128
    (1, 8, 4, 128, 0, 257, torch.bfloat16),       # cold prefill from position 0
    (3, 1, 8, 64, 17, 5, torch.float16),          # verify-sized chunk, 8 heads per KV head
    (1, 2, 12, 64, 33, 9, torch.float16),         # 12 heads per KV head: two CTAs per KV head
    (2, 2, 1, 256, 40, 33, torch.float32),        # MHA, D 256, fp32 queries
])
def test_attention_cache_f16_chunk(b, kv_h, group, d, start, chunk, dtype):
    rng = np.random.default_rng([b, kv_h, d, chunk])
    h, s_max = kv_h * group, start + chunk + 13
    k = synth.kv_rows(rng, (b, kv_h, s_max, d))
    v = synth.kv_rows(rng, (b, kv_h, s_max, d))
    new_k = synth.kv_rows(rng, (b, chunk, kv_h, d))                     # (B, S, KV_H, D) storage, as a model makes it
    new_v = synth.kv_rows(rng, (b, chunk, kv_h, d))
    q = synth.activations(rng, b * h * chunk, d).reshape(b, h, chunk, d)
    kd, vd = _dev(k), _dev(v)
    pos = torch.arange(start, start + chunk, device=DEV)
    out = torch.ops.alloy.attention_cache(_dev(q).to(dtype), _dev(new_k).transpose(1, 2), _dev(new_v).transpose(1, 2),
                                          pos, kd, vd, 1.0 / np.sqrt(d))
    k2, v2 = k.copy(), v.copy()
    k2[:, :, start:start + chunk] = new_k.transpose(0, 2, 1, 3)
    v2[:, :, start:start + chunk] = new_v.transpose(0, 2, 1, 3)
    assert np.array_equal(kd.cpu().numpy().view(np.uint16), k2.view(np.uint16))
    assert np.array_equal(vd.cpu().numpy().view(np.uint16), v2.view(np.uint16))
    q16 = torch.from_numpy(q).to(dtype).to(torch.float16).double().numpy()
    ref = np.stack([O.attention_chunk_ref(k2[i].astype(np.float32), v2[i].astype(np.float32), q16[i], start)
                    for i in range(b)])
    assert out.shape == (b, h, chunk, d) and out.dtype == dtype
    assert_close(to_np(out), ref, dtype, "f16 chunk")


def test_attention_kv_update_multi_is_the_verify_step():
    """attention_kv_update_multi (2..16 new tokens) == writing the rows and decoding them one by one."""
    rng = np.random.default_rng(21)
    b, kv_h, group, d, start, n = 2, 2, 4, 128, 95, 6
    h, s_max = kv_h * group, 128
    k = synth.kv_rows(rng, (b, kv_h, s_max, d))
    v = synth.kv_rows(rng, (b, kv_h, s_max, d))
    nk, nv = synth.kv_rows(rng, (b, kv_h, n, d)), synth.kv_rows(rng, (b, kv_h, n, d))
    q = synth.activations(rng, b * h * n, d).reshape(b, h, n, d)
    kd, vd = _dev(k), _dev(v)
    out = torch.ops.alloy.attention_kv_update_multi(_dev(q), _dev(nk), _dev(nv), torch.tensor([start], device=DEV),
                                                    kd, vd)
    k2, v2 = _dev(k), _dev(v)
    for i in range(n):
        one = torch.ops.alloy.attention_kv_update(_dev(q[:, :, i:i + 1]), _dev(nk[:, :, i:i + 1]),
                                                  _dev(nv[:, :, i:i + 1]), torch.tensor([start + i], device=DEV), k2, v2)
        assert (out[:, :, i].float() - one[:, :, 0].float()).abs().max() < 2e-3
    assert torch.equal(kd, k2) and torch.equal(vd, v2)


def test_attention_paged_q8_chunk_per_sequence_starts():
    """Chunk prefill into the paged pool: each sequence has its own start; the chunk rows are
    quantised into the right pages (bit-exact) and attention reads history + chunk from the codes."""
    from tests.test_gpu_kv_attn import _build_paged

    rng = np.random.default_rng(33)
    b, kv_h, group, d, chunk = 3, 2, 4, 128, 40
    h = kv_h * group
    starts = [0, 21, 300]
    lens = [s + chunk - 1 for s in starts]            # _build_paged reserves lens + 1 tokens
    store, host, seq_rows = _build_paged(rng, b, kv_h, d, lens)
    nk, nv = synth.kv_rows(rng, (b, kv_h, chunk, d)), synth.kv_rows(rng, (b, kv_h, chunk, d))
    q = synth.activations(rng, b * h * chunk, d).reshape(b, h, chunk, d)
    pos = torch.tensor(starts, dtype=torch.int32, device=DEV)
    out = torch.ops.alloy.attention_cache_q8_paged(_dev(q), _dev(nk), _dev(nv), pos, store.page_table, store.pool)
    assert ops.attn_status(ops.attn_workspace(torch.device(DEV, 0), b, h, d)) == 0
    nkc, nks = O.kv_quantize_q8_0(nk)
    nvc, nvs = O.kv_quantize_q8_0(nv)
    refs = []
    for s in range(b):
        kc, ks, vc, vs = (a.copy() for a in seq_rows[s])
        sl = slice(starts[s], starts[s] + chunk)
        kc[:, sl], ks[:, sl], vc[:, sl], vs[:, sl] = nkc[s], nks[s], nvc[s], nvs[s]
        kraw, vraw = O.kv_pack_blocks(kc, ks), O.kv_pack_blocks(vc, vs)
        for i, pg in enumerate(store.pages_of(s)):
            host[pg, 0], host[pg, 1] = kraw[:, i * 16:(i + 1) * 16], vraw[:, i * 16:(i + 1) * 16]
        refs.append(O.attention_chunk_ref(_deq16(kc, ks), _deq16(vc, vs), q[s].astype(np.float64), starts[s]))
    assert np.array_equal(store.pool.cpu().numpy(), host)
    assert np.abs(to_np(out) - np.stack(refs)).max() < 2e-2
    assert_close(to_np(out), np.stack(refs), torch.float16, "paged chunk")


def test_chunk_attention_errors():
    d = 64
    q = torch.zeros((1, 4, 3, d), dtype=torch.float16, device=DEV)
    nk = torch.zeros((1, 2, 3, d), dtype=torch.float16, device=DEV)
    cache = torch.zeros((1, 2, 32, d), dtype=torch.float16, device=DEV)
    pos = torch.tensor([0], device=DEV)
    with pytest.raises(NotImplementedError, match="last_real"):
        torch.ops.alloy.attention_cache(q, nk, nk, pos, cache, cache, 0.125, 0, True, torch.tensor([2], device=DEV))
    with pytest.raises(NotImplementedError, match="sliding"):
        torch.ops.alloy.attention_cache(q, nk, nk, pos, cache, cache, 0.125, 16)
    with pytest.raises(ValueError, match="v cache"):
        torch.ops.alloy.attention_cache(q, nk, nk, pos, cache, cache[:, :, :, :32].contiguous(), 0.125)
    with pytest.raises(ValueError, match="new_k"):
        torch.ops.alloy.attention_cache(q, nk[:, :, :2], nk, pos, cache, cache, 0.125)
    # a chunk that would run past the cache is reported in the status word, not written out of bounds
    torch.ops.alloy.attention_cache(q, nk, nk, torch.tensor([31], device=DEV), cache, cache, 0.125)
    assert ops.attn_status(ops.attn_workspace(torch.device(DEV, 0), 1, 4, d)) & 1
    ops._workspaces.clear()

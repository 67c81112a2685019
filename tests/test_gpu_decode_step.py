"""GPU parity of the Llama-shape decode step (eager and CUDA-graph replay) vs the CPU oracle."""

import numpy as np
import pytest
import torch

from alloy_b200 import llama
from oracle import blocks as O
from oracle import decode_step as OD
from tests._util import GEMM_MIN_TOKENS, rel_errors, to_np

pytestmark = pytest.mark.gpu

TINY = llama.LlamaShape(layers=2, hidden=512, ffn=1024, heads=8, kv_heads=2, head_dim=64, vocab=640,
                        rope_theta=10000.0, eps=1e-5)


def _r16(w, fmt, gemm):
    """GEMM_MIN_TOKENS and more take the tensor-core GEMM, whose definition rounds the decoded weight to
    fp16 once (Q6_K rows whose pitch is not a multiple of 16 bytes stay on the exact-weight kernels)."""
    k = w.shape[1]
    if gemm and (fmt == "q4_k" or (k // 256 * 210) % 16 == 0):
        return w.astype(np.float16).astype(np.float32)
    return w


def _oracle_inputs(dec, gemm=False):
    q4 = lambda t: _r16(O.dequant_q4_k(t.cpu().numpy()), "q4_k", gemm)
    q6 = lambda t: _r16(O.dequant_q6_k(t.cpu().numpy()), "q6_k", gemm)
    layers = []
    for lw in dec.layers:
        layers.append({
            "wq": q4(lw.wq), "wk": q4(lw.wk), "wv": q6(lw.wv), "wo": q4(lw.wo), "wg": q4(lw.wg), "wu": q4(lw.wu),
            "wd": q6(lw.wd), "norm_in": lw.norm_in.cpu().numpy(), "norm_post": lw.norm_post.cpu().numpy()})
    return layers


@pytest.mark.parametrize("batch", [1, 4])
def test_decode_step_matches_oracle(batch):
    ctx = 96
    # d, dmin scaled down so that fp16 activations stay far from overflow in the oracle too
    dec = llama.QuantLlamaDecoder(TINY, batch, ctx, seed=3, d_scale=0.05)
    rng = np.random.default_rng(0)
    ids = rng.integers(0, TINY.vocab, size=batch)
    dec.ids.copy_(torch.from_numpy(ids))
    kc = [k.float().cpu().numpy() for k in dec.k_cache]
    vc = [v.float().cpu().numpy() for v in dec.v_cache]
    layers = _oracle_inputs(dec)
    ref_logits, ref_next, ref_h = OD.decode_step(
        ids, ctx - 1, O.dequant_q4_k(dec.embed.cpu().numpy()), layers, dec.norm_final.cpu().numpy(),
        O.dequant_q6_k(dec.head.cpu().numpy()), dec.inv_freq.cpu().numpy(), kc, vc, TINY.heads,
        TINY.kv_heads, TINY.head_dim, TINY.eps)
    assert np.isfinite(ref_logits.astype(np.float32)).all()
    dec.step()
    torch.cuda.synchronize()
    got = to_np(dec.logits)
    # Each op is held to max 1e-2 / mean 1e-3 element-wise in its own test.  Through a whole
    # step an fp16 rounding that flips in one op is carried through the ops after it, so the
    # composed step is held to: max |err| <= 1e-2 * rms(logits), mean element-wise rel <= 2e-3.
    _, mean = rel_errors(got, ref_logits.astype(np.float64), torch.float16)
    ref64 = ref_logits.astype(np.float64)
    worst = np.abs(got - ref64).max() / np.sqrt((ref64 ** 2).mean())
    assert worst <= 1e-2 and mean <= 2e-3, (worst, mean)
    # the KV rows written at pos are the oracle's rows (fp16, same rounding points)
    mx, mean = rel_errors(to_np(dec.k_cache[0][:, :, ctx - 1]), kc[0][:, :, ctx - 1].astype(np.float64),
                          torch.float16)
    assert mx <= 1e-2 and mean <= 1e-3, (mx, mean)
    # graph replay gives the same logits as eager
    dec.capture()
    dec.step()
    torch.cuda.synchronize()
    assert torch.equal(dec.logits, torch.from_numpy(got).to(dec.logits))
    assert dec.launches_per_step > 0


MID = llama.LlamaShape(layers=2, hidden=1024, ffn=2048, heads=8, kv_heads=2, head_dim=128, vocab=1024,
                       rope_theta=10000.0, eps=1e-5)


def _paged_caches(dec, ctx):
    """Per layer the dequantised (B, KV_H, ctx, D) K and V rows the paged pools hold."""
    ks, vs = [], []
    for pool in dec.pools:
        host = pool.pool.cpu().numpy()
        per_seq = [[], []]
        for i in range(dec.batch):
            pages = dec.pools[0].pages_of(i)              # one page table serves every layer
            for which in (0, 1):
                raw = O.gather_pages(host[:, which], pages, ctx)
                per_seq[which].append(O.kv_dequant_q8_0(*O.kv_unpack_blocks(raw)))
        ks.append(np.stack(per_seq[0]))
        vs.append(np.stack(per_seq[1]))
    return ks, vs


@pytest.mark.parametrize("batch", [16, 32])
@pytest.mark.parametrize("kv_kind", ["f16", "q8_paged"])
def test_decode_step_big_batch_head_dim_128(batch, kv_kind):
    """Batch 16 and 32 of the decode step on a head_dim-128 shape (the tensor-core attention kernel
    and the 9..64-token linear path), with the fp16 cache and with the paged q8_0 pool."""
    ctx = 96
    # zero-mean weights scaled so that q and k come out near unit rms: with the uncentred blocks of the
    # kernel tests the random model's attention scores have a spread of ~50, its softmax is an argmax,
    # and one fp16 rounding flip in q or k moves a logit by percents in the oracle and on the device alike
    dec = llama.QuantLlamaDecoder(MID, batch, ctx, seed=4, d_scale=0.2, centered=True, kv=kv_kind)
    rng = np.random.default_rng(batch)
    ids = rng.integers(0, MID.vocab, size=batch)
    dec.ids.copy_(torch.from_numpy(ids))
    if kv_kind == "f16":
        kc = [k.float().cpu().numpy() for k in dec.k_cache]
        vc = [v.float().cpu().numpy() for v in dec.v_cache]
    else:
        kc, vc = _paged_caches(dec, ctx)
    ref_logits, _, _ = OD.decode_step(
        ids, ctx - 1, O.dequant_q4_k(dec.embed.cpu().numpy()), _oracle_inputs(dec, gemm=batch >= GEMM_MIN_TOKENS),
        dec.norm_final.cpu().numpy(), _r16(O.dequant_q6_k(dec.head.cpu().numpy()), "q6_k", batch >= GEMM_MIN_TOKENS),
        dec.inv_freq.cpu().numpy(), kc, vc, MID.heads, MID.kv_heads,
        MID.head_dim, MID.eps, kv_q8=(kv_kind == "q8_paged"))
    assert np.isfinite(ref_logits.astype(np.float32)).all()
    dec.step()
    torch.cuda.synchronize()
    got = to_np(dec.logits)
    _, mean = rel_errors(got, ref_logits.astype(np.float64), torch.float16)
    ref64 = ref_logits.astype(np.float64)
    worst = np.abs(got - ref64).max() / np.sqrt((ref64 ** 2).mean())
    # fifteen fp16-rounded ops in a row, each held to mean 1e-3 on its own: the composed step is held to
    # max |err| <= 1e-2 * rms(logits) and a mean element-wise relative error of 4e-3
    assert worst <= 1e-2 and mean <= 4e-3, (worst, mean)


WIDE = llama.LlamaShape(layers=3, hidden=2048, ffn=4096, heads=16, kv_heads=4, head_dim=128, vocab=2048,
                        rope_theta=10000.0, eps=1e-5)


@pytest.mark.parametrize("kv_kind", ["f16", "q8_paged"])
def test_one_launch_step_matches_op_by_op_and_oracle(kv_kind):
    """Batch 1: the whole step as ONE persistent launch (alloyb_decoder_step) against the op-by-op step
    of the same weights and against the oracle, over two consecutive positions, eager and replayed."""
    ctx = 200
    mk = lambda fused: llama.QuantLlamaDecoder(WIDE, 1, ctx, seed=9, d_scale=0.2, centered=True, kv=kv_kind,
                                               one_launch=fused)
    fused, plain = mk(True), mk(False)
    assert fused._fused is not None and plain._fused is None
    assert fused._fused.phases == WIDE.layers * 5 + 1
    if kv_kind == "f16":
        kc = [k.float().cpu().numpy() for k in plain.k_cache]
        vc = [v.float().cpu().numpy() for v in plain.v_cache]
    else:
        kc, vc = _paged_caches(plain, ctx)
    layers = _oracle_inputs(plain)
    embed, head = O.dequant_q4_k(plain.embed.cpu().numpy()), O.dequant_q6_k(plain.head.cpu().numpy())
    rng = np.random.default_rng(2)
    for step, pos in enumerate((ctx - 2, ctx - 1)):
        ids = rng.integers(0, WIDE.vocab, size=1)
        for d in (fused, plain):
            d.ids.copy_(torch.from_numpy(ids))
            d.pos.fill_(pos)
            d.seq_pos.fill_(pos)
            d.step()
        torch.cuda.synchronize()
        ref_logits, _, _ = OD.decode_step(ids, pos, embed, layers, plain.norm_final.cpu().numpy(), head,
                                          plain.inv_freq.cpu().numpy(), kc, vc, WIDE.heads, WIDE.kv_heads,
                                          WIDE.head_dim, WIDE.eps, kv_q8=(kv_kind == "q8_paged"))
        ref64 = ref_logits.astype(np.float64)
        rms = np.sqrt((ref64 ** 2).mean())
        for name, d in (("one launch", fused), ("op by op", plain)):
            got = to_np(d.logits)
            _, mean = rel_errors(got, ref64, torch.float16)
            worst = np.abs(got - ref64).max() / rms
            assert worst <= 1e-2 and mean <= 6e-3, (name, step, worst, mean)
        assert (fused.logits.float() - plain.logits.float()).abs().max() <= 1e-2 * rms
        # first layer: same q/k/v arithmetic, same rotation -> the appended rows are the same bits
        if kv_kind == "f16":
            assert torch.equal(fused.k_cache[0][:, :, pos], plain.k_cache[0][:, :, pos])
            assert torch.equal(fused.v_cache[0][:, :, pos], plain.v_cache[0][:, :, pos])
        else:
            assert torch.equal(fused.pools[0].pool, plain.pools[0].pool)
        if step == 0:
            fused.capture()                               # the second position runs as a graph replay
    from alloy_b200 import _lib
    assert _lib.load().alloyb_device_error(1) == 0


def test_decode_step_from_gguf_file(tmp_path):
    """A Llama-architecture GGUF file (written with gguf.GGUFWriter: permuted q/k rows, Q6_K and Q4_K
    v/down in alternating layers, tied head) served by the decoder equals the oracle's step on the
    arrays the file was made from."""
    from alloy_b200 import gguf_loader
    from tests._gguf_fixture import TINY_META, write_tiny_llama

    path = tmp_path / "tiny.gguf"
    arrays = write_tiny_llama(path, seed=11, tied_head=True)
    batch, ctx = 2, 80
    dec = gguf_loader.load_llama_decoder(path, batch, ctx, seed=5)
    assert dec.shape.layers == TINY_META["layers"] and dec.head_fmt == "q4_k"
    deq = {"q4_k": O.dequant_q4_k, "q6_k": O.dequant_q6_k}
    layers = []
    for lay in arrays["layers"]:
        d = {k: deq[lay[k][0]](lay[k][1]) for k in ("wq", "wk", "wv", "wo", "wg", "wu", "wd")}
        d["norm_in"] = lay["norm_in"].astype(np.float16)
        d["norm_post"] = lay["norm_post"].astype(np.float16)
        layers.append(d)
    rng = np.random.default_rng(1)
    ids = rng.integers(0, TINY_META["vocab"], size=batch)
    dec.ids.copy_(torch.from_numpy(ids))
    kc = [k.float().cpu().numpy() for k in dec.k_cache]
    vc = [v.float().cpu().numpy() for v in dec.v_cache]
    table = deq["q4_k"](arrays["embed"][1])
    ref_logits, _, _ = OD.decode_step(ids, ctx - 1, table, layers, arrays["norm_final"].astype(np.float16), table,
                                      dec.inv_freq.cpu().numpy(), kc, vc, TINY_META["heads"], TINY_META["kv_heads"],
                                      TINY_META["head_dim"], TINY_META["eps"])
    assert np.isfinite(ref_logits.astype(np.float32)).all()
    dec.step()
    torch.cuda.synchronize()
    got = to_np(dec.logits)
    _, mean = rel_errors(got, ref_logits.astype(np.float64), torch.float16)
    ref64 = ref_logits.astype(np.float64)
    worst = np.abs(got - ref64).max() / np.sqrt((ref64 ** 2).mean())
    assert worst <= 1e-2 and mean <= 2e-3, (worst, mean)


@pytest.mark.parametrize("kv_kind,start", [("f16", 0), ("q8_paged", 0), ("f16", 17)])
def test_prefill_matches_token_by_token_oracle(kv_kind, start):
    """A 40-token prompt per sequence as ONE chunk (80 token rows through the tensor-core GEMM, the causal
    chunk attention, K/V written to the cache) against the oracle fed the same tokens one position at
    a time; then one decode step from where the prefill left off."""
    ctx, b, n = 96, 2, 40
    dec = llama.QuantLlamaDecoder(MID, b, ctx, seed=5, d_scale=0.2, centered=True, kv=kv_kind)
    rng = np.random.default_rng(7 + start)
    ids = rng.integers(0, MID.vocab, size=(b, n + 1))
    if kv_kind == "f16":
        kc = [k.float().cpu().numpy() for k in dec.k_cache]
        vc = [v.float().cpu().numpy() for v in dec.v_cache]
    else:
        kc, vc = _paged_caches(dec, ctx)
    gemm = b * n >= GEMM_MIN_TOKENS
    args = (O.dequant_q4_k(dec.embed.cpu().numpy()), _oracle_inputs(dec, gemm=gemm), dec.norm_final.cpu().numpy())
    head = O.dequant_q6_k(dec.head.cpu().numpy())
    inv = dec.inv_freq.cpu().numpy()
    ref_logits = None
    for t in range(n):
        ref_logits, _, _ = OD.decode_step(ids[:, t], start + t, *args, head, inv, kc, vc, MID.heads, MID.kv_heads,
                                          MID.head_dim, MID.eps, kv_q8=(kv_kind == "q8_paged"))
    got = to_np(dec.prefill(torch.from_numpy(ids[:, :n]), start=start))
    torch.cuda.synchronize()
    assert dec.device_error() == 0

    # Through the q8_0 pool every one of the chunk's K / V rows is quantised: a value that lands on the
    # other side of a code boundary than the oracle's moves that element by 1/127 of its block's maximum,
    # and two layers of such rows lift the mean error of the logits to ~6e-3 (the reference holds its own
    # q8 prefill attention to 2e-2).  The fp16 cache keeps the composed-step bounds of the batch tests.
    w_max, m_max = (1.5e-2, 8e-3) if kv_kind == "q8_paged" else (1e-2, 4e-3)

    def check(got, ref, what):
        ref64 = ref.astype(np.float64)
        _, mean = rel_errors(got, ref64, torch.float16)
        worst = np.abs(got - ref64).max() / np.sqrt((ref64 ** 2).mean())
        assert worst <= w_max and mean <= m_max, (what, worst, mean)

    check(got, ref_logits, "prefill logits")
    # the cache rows the chunk wrote are the oracle's rows: element-wise in the first layer (norm, k
    # projection, RoPE), as a composed result in the last one
    if kv_kind == "f16":
        mx, mean = rel_errors(to_np(dec.k_cache[0][:, :, start:start + n]), kc[0][:, :, start:start + n].astype(np.float64),
                              torch.float16)
        assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
        last = len(dec.layers) - 1
        check(to_np(dec.v_cache[last][:, :, start:start + n]), vc[last][:, :, start:start + n], "last layer V rows")
    # decoding continues from the prefilled cache (the oracle starts from the cache the device holds, so
    # this step is held to the single-step bounds; its weights are exact: two token rows)
    if kv_kind == "f16":
        kc = [k.float().cpu().numpy() for k in dec.k_cache]
        vc = [v.float().cpu().numpy() for v in dec.v_cache]
    else:
        kc, vc = _paged_caches(dec, ctx)
    args1 = (args[0], _oracle_inputs(dec, gemm=False), args[2])
    ref1, _, _ = OD.decode_step(ids[:, n], start + n, *args1, head, inv, kc, vc, MID.heads, MID.kv_heads,
                                MID.head_dim, MID.eps, kv_q8=(kv_kind == "q8_paged"))
    assert int(dec.pos.item()) == start + n
    dec.ids.copy_(torch.from_numpy(ids[:, n]))
    dec.step()
    torch.cuda.synchronize()
    w_max, m_max = 1e-2, 4e-3
    check(to_np(dec.logits), ref1, "decode after prefill")

"""GPU parity: dequantisers (bit-exact) and quantised linears (tolerance) vs the oracle,
through torch.ops.alloy.* -> ctypes -> C ABI."""

import numpy as np
import pytest
import torch

from alloy_b200 import _lib, ops, quant, synth
from oracle import blocks as O
from tests._util import GEMM_MIN_TOKENS, assert_close, same_bits_f32, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


# ------------------------------------------------------------------ dequant: bit-exact


def test_dequant_golden_bit_exact(golden):
    g = golden["q4k"]
    for blk, w in ((g["blocks_signed"], g["w_signed"]), (g["blocks"], g["w"])):
        got = ops.dequantize("q4_k", _dev(blk)).cpu().numpy()
        assert same_bits_f32(got, w)
    g6 = golden["q6k"]
    assert same_bits_f32(ops.dequantize("q6_k", _dev(g6["blocks"])).cpu().numpy(), g6["w"])
    g8 = golden["q8_0"]
    codes, scales = O.split_q8_0(g8["wire"])
    assert same_bits_f32(ops.dequantize("q8_0", _dev(codes), _dev(scales)).cpu().numpy(), g8["w"])


@pytest.mark.parametrize("fmt,n,k", [("q4_k", 256, 4096), ("q6_k", 192, 4096), ("q4_k", 33, 2560),
                                     ("q6_k", 17, 14336)])
def test_dequant_seeded_bit_exact(fmt, n, k):
    rng = np.random.default_rng(7)
    if fmt == "q4_k":
        blk = np.concatenate([synth.q4k_blocks(rng, n // 2 + 1, k), synth.q4k_blocks_signed(rng, n // 2, k)])
        ref = O.dequant_q4_k(blk)
    else:
        blk = synth.q6k_blocks(rng, n, k)
        ref = O.dequant_q6_k(blk)
    got = ops.dequantize(fmt, _dev(blk)).cpu().numpy()
    assert same_bits_f32(got, ref)
    # bf16 output = the fp32 value rounded once
    got_bf = ops.dequantize(fmt, _dev(blk), out_dtype=torch.bfloat16).cpu()
    assert torch.equal(got_bf, torch.from_numpy(ref).to(torch.bfloat16))


def test_embedding_ops():
    rng = np.random.default_rng(8)
    ids = torch.tensor([[3, 0], [31, 7]], device=DEV)
    b4 = synth.q4k_blocks(rng, 32, 512)
    e4 = torch.ops.alloy.gguf_q4_k_embedding(ids, _dev(b4))
    assert e4.dtype == torch.float32 and e4.shape == (2, 2, 512)
    assert same_bits_f32(e4.cpu().numpy().reshape(4, 512), O.dequant_q4_k(b4)[[3, 0, 31, 7]])
    b6 = synth.q6k_blocks(rng, 32, 512)
    e6 = torch.ops.alloy.gguf_q6_k_embedding(ids, _dev(b6))
    assert same_bits_f32(e6.cpu().numpy().reshape(4, 512), O.dequant_q6_k(b6)[[3, 0, 31, 7]])
    c8, s8 = O.split_q8_0(synth.q8_0_wire(rng, 32, 512))
    e8 = torch.ops.alloy.gguf_q8_0_embedding(ids, _dev(c8), _dev(s8))
    assert same_bits_f32(e8.cpu().numpy().reshape(4, 512), O.dequant_q8_0(c8, s8)[[3, 0, 31, 7]])


# ------------------------------------------------------------------ linear: tolerance

TORCH_DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def _weights(fmt, rng, n, k):
    if fmt == "q4_k":
        blk = synth.q4k_blocks(rng, n, k)
        return (_dev(blk),), O.dequant_q4_k(blk)
    if fmt == "q6_k":
        blk = synth.q6k_blocks(rng, n, k)
        return (_dev(blk),), O.dequant_q6_k(blk)
    codes, scales = O.split_q8_0(synth.q8_0_wire(rng, n, k))
    return (_dev(codes), _dev(scales)), O.dequant_q8_0(codes, scales)


_MM = {"q4_k": lambda x, w: torch.ops.alloy.gguf_q4_k_mm(x, *w),
       "q6_k": lambda x, w: torch.ops.alloy.gguf_q6_k_mm(x, *w),
       "q8_0": lambda x, w: torch.ops.alloy.gguf_q8_0_mm(x, *w)}


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q8_0"])
@pytest.mark.parametrize("m,n,k,dt", [
    (1, 4096, 4096, "f16"),        # config 0 shape
    (1, 64, 2560, "f16"),          # the reference test's NB=10 tail case
    (5, 64, 2560, "f32"),          # the reference's rows test (M=5, fp32 activations)
    (4, 1000, 4096, "f16"), (16, 1024, 4096, "f16"), (32, 520, 2048, "f16"),
    (3, 77, 512, "bf16"), (8, 4096, 14336, "f16"), (1, 1024, 8192, "bf16"),
    (64, 256, 1024, "f16"),
])
def test_mm_matches_oracle(fmt, m, n, k, dt):
    rng = np.random.default_rng([m, n, k, {'q4_k': 4, 'q6_k': 6, 'q8_0': 8}[fmt]])
    w_dev, w = _weights(fmt, rng, n, k)
    tdt = TORCH_DT[dt]
    x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).to(tdt)
    y = _MM[fmt](x.to(DEV), w_dev)
    assert y.shape == (m, n) and y.dtype == tdt
    if m >= GEMM_MIN_TOKENS and dt != "f32" and (fmt != "q6_k" or (k // 256 * 210) % 16 == 0):
        # GEMM_MIN_TOKENS and more take the tensor-core GEMM, whose definition rounds the decoded weight
        # to the activation type once (Q6_K rows whose pitch is not a multiple of 16 bytes stay on the
        # exact-weight row kernels)
        w = torch.from_numpy(w).to(tdt).float().numpy()
    ref = O.mm_ref_f64(x.float().numpy(), w)
    assert_close(to_np(y), ref, tdt, f"{fmt} m={m} n={n} k={k} {dt}")


# One fp16 token takes the persistent streaming kernel when K is a multiple of 2048: full and
# ragged row counts (partial last tile per SM and per matrix), one- and two-super-block slots
# (K = 2048 / 4096), slices longer than one slot (K = 6144, 14336), stacked matrices, residual.
@pytest.mark.parametrize("fmt", ["q4_k", "q6_k"])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1000, 2048), (77, 4096), (4096, 14336), (50, 14336),
                                 (2100, 6144), (5, 2048), (2367, 4096), (4096, 1024), (2000, 3584), (512, 3072),
                                 (8192, 1280)])
def test_one_token_stream(fmt, n, k):
    rng = np.random.default_rng([n, k, len(fmt), 7])
    w_dev, w = _weights(fmt, rng, n, k)
    x = torch.from_numpy(synth.activations(rng, 1, k))
    y = _MM[fmt](x.to(DEV), w_dev)
    assert_close(to_np(y), O.mm_ref_f64(x.float().numpy(), w), torch.float16, f"stream {fmt} n={n} k={k}")


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k"])
def test_one_token_stream_stacked_and_residual(fmt):
    rng = np.random.default_rng(91)
    k = 4096
    x = torch.from_numpy(synth.activations(rng, 1, k)).to(DEV)
    mk = synth.q4k_blocks if fmt == "q4_k" else synth.q6k_blocks
    dq = O.dequant_q4_k if fmt == "q4_k" else O.dequant_q6_k
    ws = [mk(rng, n, k) for n in (4096, 1024, 1000, 24)]
    outs = ops.linear_multi(x, [(fmt, _dev(w), None) for w in ws])
    for w, y in zip(ws, outs):
        assert_close(to_np(y), O.mm_ref_f64(x.cpu().float().numpy(), dq(w)), torch.float16, f"stacked {fmt}")
    r = synth.activations(rng, 1, 1000)
    y = torch.ops.alloy.linear_residual(x, _dev(ws[2]), None, _dev(r), fmt)
    lin = torch.from_numpy(O.mm_ref_f64(x.cpu().float().numpy(), dq(ws[2]))).to(torch.float16).double().numpy()
    assert_close(to_np(y), lin + r.astype(np.float64), torch.float16, f"residual {fmt}")


@pytest.mark.parametrize("n,k", [(1000, 2048), (14336, 4096), (333, 6144)])
def test_one_token_stream_gated(n, k):
    rng = np.random.default_rng([n, k, 13])
    g, u = synth.q4k_blocks(rng, n, k), synth.q4k_blocks(rng, n, k)
    x = synth.activations(rng, 1, k)
    y = torch.ops.alloy.gguf_q4_k_silu(_dev(x), _dev(g), _dev(u))
    ref = O.silu(O.mm_ref_f64(x, O.dequant_q4_k(g))) * O.mm_ref_f64(x, O.dequant_q4_k(u))
    assert_close(to_np(y), ref, torch.float16, f"stream gated n={n} k={k}")


# RMSNorm folded into the consuming linear: fused inside the one-token streaming launch (m = 1,
# fp16), two launches through the caller's scratch otherwise; the oracle is rms_norm_ref (fp16
# out) followed by the float64 product.
@pytest.mark.parametrize("m,dt", [(1, "f16"), (4, "f16"), (1, "bf16")])
def test_linear_normed_qkv_and_gate_up(m, dt):
    rng = np.random.default_rng([m, len(dt), 17])
    k, eps = 4096, 1e-5
    tdt = TORCH_DT[dt]
    x = torch.from_numpy((3.0 * synth.activations(rng, m, k, np.float32))).to(tdt)
    nw = torch.from_numpy((1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)).to(tdt)
    xn = torch.from_numpy(O.rms_norm_ref(x.float().numpy().astype(np.float32), nw.float().numpy().astype(np.float32), eps))
    # the oracle normalises in fp32 and narrows twice, as the kernels do
    xr = (x.float() * torch.rsqrt((x.float() ** 2).mean(dim=1, keepdim=True) + eps)).to(tdt)
    xn = (nw.float() * xr.float()).to(tdt).float().numpy()
    wq, wk, wv = synth.q4k_blocks(rng, 1024, k), synth.q4k_blocks(rng, 200, k), synth.q6k_blocks(rng, 256, k)
    outs = ops.linear_multi(x.to(DEV), [("q4_k", _dev(wq), None), ("q4_k", _dev(wk), None), ("q6_k", _dev(wv), None)],
                            norm=(nw.to(DEV), eps))
    for y, wf in zip(outs, (O.dequant_q4_k(wq), O.dequant_q4_k(wk), O.dequant_q6_k(wv))):
        assert_close(to_np(y), O.mm_ref_f64(xn, wf), tdt, f"normed qkv m={m} {dt}")
    head = synth.q6k_blocks(rng, 3000, k)
    y = ops.linear_multi(x.to(DEV), [("q6_k", _dev(head), None)], norm=(nw.to(DEV), eps))[0]
    assert_close(to_np(y), O.mm_ref_f64(xn, O.dequant_q6_k(head)), tdt, f"normed head m={m} {dt}")
    g, u = synth.q4k_blocks(rng, 1000, k), synth.q4k_blocks(rng, 1000, k)
    y = ops.gated_normed(x.to(DEV), nw.to(DEV), eps, _dev(g), _dev(u))
    ref = O.silu(O.mm_ref_f64(xn, O.dequant_q4_k(g))) * O.mm_ref_f64(xn, O.dequant_q4_k(u))
    assert_close(to_np(y), ref, tdt, f"normed gate/up m={m} {dt}")


# One token against Q4_K and Q6_K matrices in a single streaming launch (q/k and v of a decode step): rows
# of both formats shared out by cost, ragged row counts, the Q6_K matrix named first, two matrices per
# format, a K of 32 super-blocks (fragments not cached), with and without the fused RMSNorm.
@pytest.mark.parametrize("k,q4_rows,q6_rows,normed", [
    (4096, (4096, 1024), (1024,), True),
    (4096, (200, 40), (7,), False),
    (8192, (1024, 136), (520, 24), True),
    (4096, (16,), (2048, 1000), False),
])
def test_mixed_formats_one_launch(k, q4_rows, q6_rows, normed):
    rng = np.random.default_rng([k, len(q4_rows), q6_rows[0]])
    eps = 1e-5
    x = torch.from_numpy(2.0 * synth.activations(rng, 1, k, np.float32)).to(torch.float16)
    w4 = [synth.q4k_blocks(rng, n, k) for n in q4_rows]
    w6 = [synth.q6k_blocks(rng, n, k) for n in q6_rows]
    # Q6_K first: the launch sorts by format, the outputs keep the caller's order
    specs = [("q6_k", _dev(w), None) for w in w6] + [("q4_k", _dev(w), None) for w in w4]
    refs = [O.dequant_q6_k(w) for w in w6] + [O.dequant_q4_k(w) for w in w4]
    if normed:
        nw = torch.from_numpy((1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32)).to(torch.float16)
        xr = (x.float() * torch.rsqrt((x.float() ** 2).mean(dim=1, keepdim=True) + eps)).to(torch.float16)
        xin = (nw.float() * xr.float()).to(torch.float16).float().numpy()
        outs = ops.linear_multi(x.to(DEV), specs, norm=(nw.to(DEV), eps))
    else:
        xin = x.float().numpy()
        outs = ops.linear_multi(x.to(DEV), specs)
    torch.cuda.synchronize()
    assert _lib.load().alloyb_device_error(1) == 0
    for y, wf in zip(outs, refs):
        assert y.shape == (1, wf.shape[0])
        assert_close(to_np(y), O.mm_ref_f64(xin, wf), torch.float16, f"mixed k={k} rows={wf.shape[0]}")


# Row-parallel linear with the all-reduce inside the launch: with one rank the exchange
# degenerates to "deliver to myself, wait for my own flag, add the residual", which runs the
# whole device path (epochs, both slot sets, flags) on a single GPU.  The 2-GPU sum is checked
# in the tensor-parallel bench run (logits against the NCCL path).
@pytest.mark.parametrize("fmt,n,k", [("q4_k", 4096, 4096), ("q6_k", 4096, 14336), ("q4_k", 8192, 1024), ("q6_k", 1000, 2048)])
def test_linear_allreduce_single_rank(fmt, n, k):
    from alloy_b200 import tp
    rng = np.random.default_rng([n, k, len(fmt), 23])
    w_dev, w = _weights(fmt, rng, n, k)
    ex = tp.PeerExchange(max_n=8192)
    try:
        for call in range(3):                       # epochs 1..3: both slot sets, flag reuse
            x = synth.activations(rng, 1, k)
            r = synth.activations(rng, 1, n)
            y = ops.linear_allreduce(_dev(x), fmt, w_dev[0], _dev(r), ex)
            assert y is not None
            lin = torch.from_numpy(O.mm_ref_f64(x, w)).to(torch.float16).double().numpy()
            assert_close(to_np(y), lin + r.astype(np.float64), torch.float16, f"allreduce w=1 {fmt} call {call}")
        assert ops.linear_allreduce(_dev(synth.activations(rng, 3, k)), fmt, w_dev[0], None, ex) is None
    finally:
        torch.cuda.synchronize()
        ex.close()


def test_peer_wait_runs_out_and_is_reported():
    """A peer that never delivers: a two-rank descriptor on ONE GPU whose second buffer nobody writes,
    with a short spin limit.  The kernel must come back, the sticky device error word must be set
    (the host then drops the peer path), and the next call on a sound exchange must be clean."""
    import ctypes as C

    from alloy_b200 import _lib, tp
    rng = np.random.default_rng(5)
    n, k = 4096, 4096
    w_dev, w = _weights("q4_k", rng, n, k)
    L = _lib.load()
    assert L.alloyb_device_error(1) == 0
    mine, silent = tp.PeerExchange(max_n=n), tp.PeerExchange(max_n=n)
    try:
        peers = (C.c_void_p * 8)(mine.desc.peer[0], silent.desc.peer[0], *([None] * 6))
        desc = _lib.TP(2, 0, n, 5000, peers)
        x = _dev(synth.activations(rng, 1, k))
        y = torch.empty((1, n), dtype=torch.float16, device=DEV)
        wd = (_lib.Weight * 1)(_lib.Weight(_lib.Q4_K, n, w_dev[0].data_ptr(), None, 0, y.data_ptr(), 0))
        rc = L.alloyb_linear_allreduce(x.data_ptr(), 1, k, _lib.F16, wd, None, C.byref(desc),
                                       torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()                       # the launch returned: no hang
        assert L.alloyb_device_error(1) != 0           # ... and said so
        assert L.alloyb_device_error(0) == 0           # cleared by the read above
        # a misaligned activation pointer under an exchange is a hard error, never "not taken"
        xo = torch.zeros(k + 8, dtype=torch.float16, device=DEV)[1:k + 1]
        rc = L.alloyb_linear_allreduce(xo.data_ptr(), 1, k, _lib.F16, wd, None, C.byref(desc),
                                       torch.cuda.current_stream().cuda_stream)
        assert rc == -2
    finally:
        torch.cuda.synchronize()
        mine.close()
        silent.close()
    ex = tp.PeerExchange(max_n=n)
    try:
        x = synth.activations(rng, 1, k)
        y = ops.linear_allreduce(_dev(x), "q4_k", w_dev[0], None, ex)
        assert_close(to_np(y), O.mm_ref_f64(x, w), torch.float16, "after a timed-out call")
        assert L.alloyb_device_error(1) == 0
    finally:
        torch.cuda.synchronize()
        ex.close()


# A K shard whose rows are not a multiple of 16 bytes long (Q6_K, 14 super-blocks = 2940 bytes)
# keeps a 16-byte pitch: the op takes the strided view as it is.
@pytest.mark.parametrize("world", [2, 4])
def test_column_shard_padded_pitch(world):
    from alloy_b200 import tp
    rng = np.random.default_rng(world)
    n, k = 600, 3584 * world
    full = synth.q6k_blocks(rng, n, k)
    x = synth.activations(rng, 1, k)
    wf = O.dequant_q6_k(full)
    acc = np.zeros((1, n))
    for r in range(world):
        shard = tp.shard_cols(_dev(full), "q6_k", r, world)
        assert shard.stride(0) % 16 == 0 and shard.shape[1] == 14 * 210
        ks = tp.k_slice(k, r, world)
        y = torch.ops.alloy.gguf_q6_k_mm(_dev(np.ascontiguousarray(x[:, ks])), shard)
        part = O.mm_ref_f64(x[:, ks], wf[:, ks])
        assert_close(to_np(y), part, torch.float16, f"padded shard {r}/{world}")
        acc += part
    assert np.allclose(acc, O.mm_ref_f64(x, wf), rtol=1e-9, atol=1e-9)


def test_q4k_mm_golden(golden):
    g = golden["q4k"]
    y = torch.ops.alloy.gguf_q4_k_mm(_dev(g["x"]), _dev(g["blocks"]))
    assert_close(to_np(y), g["y"].astype(np.float64), torch.float16, "golden q4k")


@pytest.mark.parametrize("m", [1, 3, 8])
def test_batched_and_mixed(m):
    rng = np.random.default_rng(21)
    k = 2048
    x = torch.from_numpy(synth.activations(rng, m, k)).to(DEV)
    ws = [synth.q4k_blocks(rng, n, k) for n in (512, 128, 136, 40, 72)]
    outs = torch.ops.alloy.batched_gguf_q4_k_mm(x, [_dev(w) for w in ws])
    assert len(outs) == 5
    for w, y in zip(ws, outs):
        assert_close(to_np(y), O.mm_ref_f64(x.cpu().float().numpy(), O.dequant_q4_k(w)), torch.float16)
    w6 = [synth.q6k_blocks(rng, n, k) for n in (128, 64)]
    for w, y in zip(w6, torch.ops.alloy.batched_gguf_q6_k_mm(x, [_dev(w) for w in w6])):
        assert_close(to_np(y), O.mm_ref_f64(x.cpu().float().numpy(), O.dequant_q6_k(w)), torch.float16)
    w8 = [O.split_q8_0(synth.q8_0_wire(rng, n, k)) for n in (96, 32)]
    outs8 = torch.ops.alloy.batched_gguf_q8_0_mm(x, [_dev(c) for c, _ in w8], [_dev(s) for _, s in w8])
    for (c, s), y in zip(w8, outs8):
        assert_close(to_np(y), O.mm_ref_f64(x.cpu().float().numpy(), O.dequant_q8_0(c, s)), torch.float16)
    # q/k (Q4_K) + v (Q6_K) in one launch
    mixed = ops.linear_multi(x, [("q4_k", _dev(ws[0]), None), ("q4_k", _dev(ws[1]), None),
                                 ("q6_k", _dev(w6[0]), None)])
    for y, wf in zip(mixed, (O.dequant_q4_k(ws[0]), O.dequant_q4_k(ws[1]), O.dequant_q6_k(w6[0]))):
        assert_close(to_np(y), O.mm_ref_f64(x.cpu().float().numpy(), wf), torch.float16)


@pytest.mark.parametrize("m,n,k", [(1, 14336, 4096), (4, 1024, 2560), (16, 512, 1024), (5, 64, 2560)])
@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_q4k_gated(m, n, k, act):
    rng = np.random.default_rng(31 + m)
    g, u = synth.q4k_blocks(rng, n, k), synth.q4k_blocks(rng, n, k)
    x = synth.activations(rng, m, k)
    op = torch.ops.alloy.gguf_q4_k_silu if act == "silu" else torch.ops.alloy.gguf_q4_k_gelu
    y = op(_dev(x), _dev(g), _dev(u))
    wg, wu = O.dequant_q4_k(g), O.dequant_q4_k(u)
    if m >= GEMM_MIN_TOKENS:
        # that many tokens take the tensor-core GEMM, which rounds the decoded weight to the
        # activation type once (as the reference's tiled GEMM does from five tokens up)
        wg, wu = (w.astype(np.float16).astype(np.float32) for w in (wg, wu))
    gate = O.mm_ref_f64(x, wg)
    up = O.mm_ref_f64(x, wu)
    ref = (O.silu(gate) if act == "silu" else O.gelu_tanh(gate)) * up
    assert_close(to_np(y), ref, torch.float16, f"gated {act} m={m}")


def test_q8_gated():
    rng = np.random.default_rng(41)
    n, k, m = 256, 1024, 3
    (gc, gs), (uc, us) = (O.split_q8_0(synth.q8_0_wire(rng, n, k)) for _ in range(2))
    x = synth.activations(rng, m, k)
    y = torch.ops.alloy.gguf_q8_0_silu(_dev(x), _dev(gc), _dev(gs), _dev(uc), _dev(us))
    ref = O.silu(O.mm_ref_f64(x, O.dequant_q8_0(gc, gs))) * O.mm_ref_f64(x, O.dequant_q8_0(uc, us))
    assert_close(to_np(y), ref, torch.float16, "q8 gated")


def test_linear_residual():
    rng = np.random.default_rng(51)
    n, k, m = 512, 1024, 4
    w = synth.q6k_blocks(rng, n, k)
    x, r = synth.activations(rng, m, k), synth.activations(rng, m, n)
    y = torch.ops.alloy.linear_residual(_dev(x), _dev(w), None, _dev(r), "q6_k")
    lin = torch.from_numpy(O.mm_ref_f64(x, O.dequant_q6_k(w))).to(torch.float16).double().numpy()
    assert_close(to_np(y), lin + r.astype(np.float64), torch.float16, "residual")


def test_modules_and_errors():
    rng = np.random.default_rng(61)
    blk = synth.q4k_blocks(rng, 64, 512)
    lin = quant.GGUFQ4_KLinear(in_features=512, out_features=64, blocks=torch.from_numpy(blk)).to(DEV)
    x = torch.from_numpy(synth.activations(rng, 6, 512)).to(DEV).reshape(2, 3, 512)
    y = lin(x)
    assert y.shape == (2, 3, 64)
    assert_close(to_np(y).reshape(6, 64),
                 O.mm_ref_f64(x.cpu().float().numpy().reshape(6, 512), O.dequant_q4_k(blk)), torch.float16)
    with pytest.raises(ValueError):
        quant.GGUFQ4_KLinear(in_features=500, out_features=64, blocks=torch.from_numpy(blk))
    with pytest.raises(TypeError):
        quant.GGUFQ4_KLinear(in_features=512, out_features=64, blocks=torch.from_numpy(blk).to(torch.int8))
    with pytest.raises(ValueError):
        torch.ops.alloy.gguf_q4_k_mm(x.reshape(6, 512)[:, :256].contiguous(), lin.blocks)
    assert torch.ops.alloy.gguf_q4_k_mm(x.reshape(6, 512)[:0], lin.blocks).shape == (0, 64)


def test_no_device_error_recorded():
    """No kernel of this module ran out a bounded wait."""
    from alloy_b200 import _lib
    assert _lib.load().alloyb_device_error(0) == 0

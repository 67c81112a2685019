"""GPU parity of the dequant-GEMM (tcgen05 path, 28 tokens and more) against the oracle.

The GEMM's definition includes ONE rounding of the exactly-decoded fp32 weight to the activation
type (bf16 / fp16) before the tensor-core product, so the oracle here is
float64( X ) @ float64( round_to_type( dequant_fp32(W) ) ).T, rounded to the output type.
"""

import numpy as np
import pytest
import torch

from alloy_b200 import _lib, ops, synth
from oracle import blocks as O
from tests._util import assert_close, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"bf16": torch.bfloat16, "f16": torch.float16}


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _ref(x_t, w_f32, dt):
    w_r = torch.from_numpy(w_f32).to(dt).double().numpy()      # one rounding of the decoded weight
    return x_t.double().cpu().numpy() @ w_r.T


# Q6_K rows are 16-byte aligned (what the bulk copies need) only when K is a multiple of 2048;
# other Q6_K shapes take the exact-weight row kernels and are covered in test_gpu_linear.py.
@pytest.mark.parametrize("fmt,m,n,k,dt", [
    ("q4_k", 256, 128, 256, "bf16"), ("q4_k", 64, 256, 512, "bf16"), ("q4_k", 300, 200, 1024, "bf16"),
    ("q4_k", 512, 384, 2048, "f16"), ("q4_k", 1000, 136, 4096, "bf16"),
    ("q6_k", 256, 128, 2048, "bf16"), ("q6_k", 64, 256, 2048, "bf16"), ("q6_k", 300, 200, 4096, "bf16"),
    ("q6_k", 512, 384, 2048, "f16"), ("q6_k", 1000, 136, 6144, "bf16"),
    ("q8_0", 256, 128, 256, "bf16"), ("q8_0", 64, 200, 1024, "f16"), ("q8_0", 1000, 136, 4096, "bf16")])
def test_gemm_matches_oracle(fmt, m, n, k, dt):
    rng = np.random.default_rng([m, n, k, len(fmt)])
    tdt = DT[dt]
    if fmt == "q8_0":
        codes, scales = O.split_q8_0(synth.q8_0_wire(rng, n, k))
        w = O.dequant_q8_0(codes, scales)
        x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).to(tdt).to(DEV)
        y = torch.ops.alloy.gguf_q8_0_mm(x, _dev(codes), _dev(scales))
        assert y.shape == (m, n) and y.dtype == tdt
        assert_close(to_np(y), _ref(x, w, tdt), tdt, f"gemm {fmt} {m}x{n}x{k} {dt}")
        assert _lib.load().alloyb_device_error(0) == 0
        return
    if fmt == "q4_k":
        blk = synth.q4k_blocks(rng, n, k)
        w = O.dequant_q4_k(blk)
        op = torch.ops.alloy.gguf_q4_k_mm
    else:
        blk = synth.q6k_blocks(rng, n, k)
        w = O.dequant_q6_k(blk)
        op = torch.ops.alloy.gguf_q6_k_mm
    x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).to(tdt).to(DEV)
    y = op(x, _dev(blk))
    assert y.shape == (m, n) and y.dtype == tdt
    assert_close(to_np(y), _ref(x, w, tdt), tdt, f"gemm {fmt} {m}x{n}x{k} {dt}")
    assert _lib.load().alloyb_device_error(0) == 0


def test_gemm_rows_agree_with_gemv_path():
    """The same matrix through the GEMV family (M=8) and the GEMM (M=64, first 8 rows equal inputs)."""
    rng = np.random.default_rng(77)
    n, k = 256, 1024
    blk = _dev(synth.q4k_blocks(rng, n, k))
    x = torch.from_numpy(synth.activations(rng, 64, k)).to(DEV)
    big = torch.ops.alloy.gguf_q4_k_mm(x, blk)
    small = torch.ops.alloy.gguf_q4_k_mm(x[:8].contiguous(), blk)
    # GEMV keeps fp32-exact weights, the GEMM rounds them to fp16 once: close, not identical
    a, b = to_np(big[:8]).astype(np.float64), to_np(small).astype(np.float64)
    assert np.abs(a - b).max() <= 1e-2 * np.sqrt((b * b).mean())


@pytest.mark.parametrize("m", [128, 200])
def test_gated_prefill(m):
    """Up to 128 tokens gate and up stay fp32 accumulators of one launch; beyond, two GEMMs round each to
    the activation type before the activation kernel multiplies them."""
    rng = np.random.default_rng(78)
    n, k = 256, 512
    g, u = synth.q4k_blocks(rng, n, k), synth.q4k_blocks(rng, n, k)
    x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).to(torch.bfloat16).to(DEV)
    y = torch.ops.alloy.gguf_q4_k_silu(x, _dev(g), _dev(u))
    gate, up = _ref(x, O.dequant_q4_k(g), torch.bfloat16), _ref(x, O.dequant_q4_k(u), torch.bfloat16)
    if m > 128:
        gate = torch.from_numpy(gate).to(torch.bfloat16).double().numpy()
        up = torch.from_numpy(up).to(torch.bfloat16).double().numpy()
    assert_close(to_np(y), O.silu(gate) * up, torch.bfloat16, "prefill gate/up")


@pytest.mark.parametrize("fmt,n,k", [("q4_k", 14336, 4096), ("q6_k", 4096, 14336)])
def test_gemm_full_size_sampled_columns(fmt, n, k):
    """The benchmark-sized prefill GEMM (4096 tokens), checked on 48 sampled output columns."""
    rng = np.random.default_rng(5)
    m = 4096
    gen = torch.Generator(device=DEV).manual_seed(3)
    blk = (synth.q4k_blocks_device if fmt == "q4_k" else synth.q6k_blocks_device)(n, k, gen, DEV)
    x = torch.randn((m, k), device=DEV, generator=gen).to(torch.bfloat16)
    op = torch.ops.alloy.gguf_q4_k_mm if fmt == "q4_k" else torch.ops.alloy.gguf_q6_k_mm
    y = op(x, blk)
    cols = np.sort(rng.choice(n, size=48, replace=False))
    sub = blk[torch.from_numpy(cols).to(DEV)].cpu().numpy()
    w = O.dequant_q4_k(sub) if fmt == "q4_k" else O.dequant_q6_k(sub)
    assert_close(to_np(y[:, torch.from_numpy(cols).to(DEV)]), _ref(x, w, torch.bfloat16), torch.bfloat16,
                 f"full-size {fmt}")
    assert _lib.load().alloyb_device_error(0) == 0


def _weights(fmt, rng, n, k):
    if fmt == "q8_0":
        codes, scales = O.split_q8_0(synth.q8_0_wire(rng, n, k))
        return (_dev(codes), _dev(scales)), O.dequant_q8_0(codes, scales)
    blk = synth.q4k_blocks(rng, n, k) if fmt == "q4_k" else synth.q6k_blocks(rng, n, k)
    return (_dev(blk), None), (O.dequant_q4_k(blk) if fmt == "q4_k" else O.dequant_q6_k(blk))


# Batched-decode and chunk sizes: one token tile of 32 / 64 / 128 columns, ragged token and row
# counts, matrices with fewer row tiles than SMs (K split over several CTAs whose partial tiles
# meet in the fp32 scratch), with and without a residual.  Every case runs twice: the second call
# finds the scratch and the tile counters as the first one left them.
@pytest.mark.parametrize("fmt,m,n,k,dt", [
    ("q4_k", 28, 4096, 4096, "f16"), ("q4_k", 31, 1024, 4096, "bf16"), ("q4_k", 32, 4096, 14336, "f16"),
    ("q4_k", 64, 14336, 4096, "f16"), ("q4_k", 128, 200, 1024, "bf16"), ("q4_k", 129, 200, 1024, "bf16"),
    ("q6_k", 50, 1024, 4096, "f16"), ("q6_k", 100, 4096, 14336, "bf16"), ("q6_k", 29, 130, 2048, "f16"),
    ("q8_0", 33, 520, 2048, "f16"), ("q8_0", 30, 4096, 4096, "bf16")])
def test_gemm_few_tokens_split_k_and_residual(fmt, m, n, k, dt):
    rng = np.random.default_rng([m, n, k, len(fmt), 5])
    tdt = DT[dt]
    (wd, sd), w = _weights(fmt, rng, n, k)
    x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).to(tdt).to(DEV)
    res = torch.from_numpy(synth.activations(rng, m, n, np.float32)).to(tdt).to(DEV)
    ref = _ref(x, w, tdt)
    name = {"q4_k": "q4_k", "q6_k": "q6_k", "q8_0": "q8_0"}[fmt]
    for rep in range(2):
        y = (torch.ops.alloy.gguf_q8_0_mm(x, wd, sd) if fmt == "q8_0" else
             (torch.ops.alloy.gguf_q4_k_mm if fmt == "q4_k" else torch.ops.alloy.gguf_q6_k_mm)(x, wd))
        assert y.shape == (m, n) and y.dtype == tdt
        assert_close(to_np(y), ref, tdt, f"gemm {fmt} {m}x{n}x{k} {dt} call {rep}")
        yr = torch.ops.alloy.linear_residual(x, wd, sd, res, name)
        # residual: type(residual + type(acc)).  Two roundings, each relative to its own operand: where
        # residual and product cancel the error is bounded by their magnitudes, not by the sum's
        acc = torch.from_numpy(ref).to(tdt).double().numpy()
        r64 = res.double().cpu().numpy()
        err = np.abs(to_np(yr).astype(np.float64) - (r64 + acc))
        ulp = 2.0 ** (-8 if tdt == torch.bfloat16 else -11)
        bound = ulp * (2.0 * np.abs(acc) + np.abs(r64 + acc)) + 1e-3 * np.sqrt((ref ** 2).mean())
        assert (err <= bound).all(), f"gemm+residual {fmt} {m}x{n}x{k} {dt} call {rep}: worst {np.max(err / bound):.2f} x bound"
        assert err.mean() <= ulp * (np.abs(acc) + np.abs(r64 + acc)).mean()
    assert _lib.load().alloyb_device_error(0) == 0


# Gate/up pairs up to 128 tokens keep two accumulators in tensor memory; few row tiles split K over
# two planes of the scratch.
@pytest.mark.parametrize("m,n,k,dt", [(32, 14336, 4096, "f16"), (64, 1024, 4096, "bf16"), (128, 3584, 2048, "f16"),
                                      (29, 200, 1024, "f16")])
@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_gemm_gated_few_tokens(m, n, k, dt, act):
    rng = np.random.default_rng([m, n, k, 7])
    tdt = DT[dt]
    g, u = synth.q4k_blocks(rng, n, k), synth.q4k_blocks(rng, n, k)
    x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).to(tdt).to(DEV)
    op = torch.ops.alloy.gguf_q4_k_silu if act == "silu" else torch.ops.alloy.gguf_q4_k_gelu
    gate, up = _ref(x, O.dequant_q4_k(g), tdt), _ref(x, O.dequant_q4_k(u), tdt)
    ref = (O.silu(gate) if act == "silu" else O.gelu_tanh(gate)) * up
    gd, ud = _dev(g), _dev(u)
    for rep in range(2):
        y = op(x, gd, ud)
        assert y.shape == (m, n) and y.dtype == tdt
        assert_close(to_np(y), ref, tdt, f"gated gemm {act} {m}x{n}x{k} {dt} call {rep}")
    assert _lib.load().alloyb_device_error(0) == 0


def test_gemm_gated_q8_few_tokens():
    rng = np.random.default_rng(43)
    m, n, k = 40, 640, 2048
    (gc, gs), (uc, us) = (O.split_q8_0(synth.q8_0_wire(rng, n, k)) for _ in range(2))
    x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).half().to(DEV)
    y = torch.ops.alloy.gguf_q8_0_silu(x, _dev(gc), _dev(gs), _dev(uc), _dev(us))
    ref = O.silu(_ref(x, O.dequant_q8_0(gc, gs), torch.float16)) * _ref(x, O.dequant_q8_0(uc, us), torch.float16)
    assert_close(to_np(y), ref, torch.float16, "q8 gated gemm")
    assert _lib.load().alloyb_device_error(0) == 0


# Two matrices of one format whose packed rows lie back to back in one buffer (q and k of a layer) run as ONE
# GEMM with two outputs: each output against the oracle, with and without a K split, ragged second matrix.
@pytest.mark.parametrize("fmt,m,nq,nk,k", [("q4_k", 40, 256, 200, 1024), ("q4_k", 64, 4096, 1024, 4096),
                                           ("q6_k", 33, 128, 72, 2048), ("q4_k", 200, 384, 128, 512)])
def test_gemm_two_stacked_matrices_one_launch(fmt, m, nq, nk, k):
    rng = np.random.default_rng([m, nq, nk, k])
    make = synth.q4k_blocks if fmt == "q4_k" else synth.q6k_blocks
    deq = O.dequant_q4_k if fmt == "q4_k" else O.dequant_q6_k
    wq, wk = make(rng, nq, k), make(rng, nk, k)
    both = torch.from_numpy(np.concatenate([wq, wk], 0)).to(DEV)
    x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).to(torch.float16)
    yq, yk = ops.linear_multi(x.to(DEV), [(fmt, both[:nq], None), (fmt, both[nq:], None)])
    torch.cuda.synchronize()
    assert _lib.load().alloyb_device_error(1) == 0
    for y, w in ((yq, wq), (yk, wk)):
        assert y.shape == (m, w.shape[0])
        assert_close(to_np(y), _ref(x, deq(w), torch.float16), torch.float16, f"stacked {fmt} m={m} rows={w.shape[0]}")

"""GPU parity of the adjacent formats/ops: Q5_0 (decode bit-exact, matmul within tolerance) and the
routed mixture-of-experts op, against the oracle."""

import numpy as np
import pytest
import torch

from alloy_b200 import quant, synth
from oracle import blocks as O
from tests._util import assert_close, same_bits_f32, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _q5_wire(rng, n, k):
    wire = rng.integers(0, 256, size=(n, k // 32, 22), dtype=np.uint8)
    d = rng.uniform(1e-4, 2e-3, size=(n, k // 32)).astype(np.float16)
    wire[:, :, 0:2] = d.view(np.uint8).reshape(n, k // 32, 2)
    return wire.reshape(n, -1)


def test_q5_0_embedding_golden_bit_exact(golden):
    g = golden["q5_0"]
    n, k = g["w"].shape
    ids = torch.tensor([[3, 0], [5, 3]], device=DEV)
    out = torch.ops.alloy.gguf_q5_0_embedding(ids, _dev(g["qweight"]), _dev(g["qhigh"]), _dev(g["scales"]))
    assert out.dtype == torch.float32 and out.shape == (2, 2, k)
    assert same_bits_f32(out.cpu().numpy().reshape(4, k), g["w"][[3, 0, 5, 3]])


@pytest.mark.parametrize("m,n,k,dt", [(1, 96, 1024, torch.float16), (5, 40, 4096, torch.bfloat16),
                                      (3, 17, 64, torch.float32)])
def test_q5_0_mm_matches_oracle(m, n, k, dt):
    rng = np.random.default_rng([m, n, k])
    wire = _q5_wire(rng, n, k)
    qw, qh, sc = quant.split_q5_0_weight(weights=wire, in_features=k, out_features=n)
    w = O.dequant_q5_0(*O.split_q5_0(wire))
    x = torch.from_numpy(synth.activations(rng, m, k, np.float32)).to(dt)
    lin = quant.GGUFQ5_0Linear(in_features=k, out_features=n, qweight=qw.to(DEV), qhigh=qh.to(DEV),
                               scales=sc.to(DEV))
    y = lin(x.to(DEV))
    assert y.dtype == dt and y.shape == (m, n)
    assert_close(to_np(y), O.mm_ref_f64(x.double().numpy(), w), dt, "q5_0 mm")
    ys = torch.ops.alloy.batched_gguf_q5_0_mm(x.to(DEV), [qw.to(DEV)] * 2, [qh.to(DEV)] * 2, [sc.to(DEV)] * 2)
    assert len(ys) == 2 and torch.equal(ys[0], y) and torch.equal(ys[1], y)


@pytest.mark.parametrize("t_n,dt", [(1, torch.float32), (3, torch.float16)])
def test_moe_routed_matches_oracle(t_n, dt):
    """The reference's handler case (tests/kernels/test_moe.py:89-146: H 256, I 512, 4 experts, top 2,
    small block scales), at one and several tokens, against the float64 composition of the decoders."""
    hdim, inter, e_n, top_k = 256, 512, 4, 2
    rng = np.random.default_rng(7)
    gu = rng.integers(0, 256, size=(e_n, 2 * inter, hdim // 256, 144), dtype=np.uint8)
    gu[..., 0:2] = (rng.standard_normal((e_n, 2 * inter, 1)) * 0.002).astype(np.float16).view(np.uint8).reshape(
        e_n, 2 * inter, 1, 2)
    gu[..., 2:4] = (rng.standard_normal((e_n, 2 * inter, 1)) * 0.001).astype(np.float16).view(np.uint8).reshape(
        e_n, 2 * inter, 1, 2)
    gu = gu.reshape(e_n, 2 * inter, -1)
    down = rng.integers(0, 256, size=(e_n, hdim, inter // 256, 210), dtype=np.uint8)
    down[..., 208:210] = np.array([0.02], np.float16).view(np.uint8)
    down = down.reshape(e_n, hdim, -1)
    x = torch.from_numpy(rng.standard_normal((t_n, hdim)).astype(np.float32)).to(dt)
    logits = rng.standard_normal((t_n, e_n)).astype(np.float32)
    logits[0, 1] = logits[0, 3]                       # a tie: the lower index wins
    y = torch.ops.alloy.gguf_moe_routed(x.to(DEV), _dev(logits), _dev(gu), _dev(down), e_n, top_k, inter)
    assert y.dtype == torch.float32 and y.shape == (t_n, hdim)
    ref = O.moe_routed_ref(x.double().numpy(), logits, gu, down, top_k, inter)
    got = y.cpu().numpy().astype(np.float64)
    assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()           # the reference test's metric
    assert_close(got, ref, torch.float32, "moe routed")

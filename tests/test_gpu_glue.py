"""GPU parity of the small decode-step ops (RMSNorm, RoPE, SiLU*up, greedy argmax) vs the oracle."""

import numpy as np
import pytest
import torch

from alloy_b200 import ops
from oracle import blocks as O
from tests._util import assert_close, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("m,k", [(1, 4096), (5, 512), (3, 8192)])
def test_rms_norm(m, k):
    rng = np.random.default_rng([m, k])
    x = rng.standard_normal((m, k)).astype(np.float16)
    w = (1.0 + 0.1 * rng.standard_normal(k)).astype(np.float16)
    y = ops.rms_norm(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), 1e-5)
    assert_close(to_np(y), O.rms_norm_ref(x, w, 1e-5).astype(np.float64), torch.float16, "rms_norm")


def test_rope_inplace():
    rng = np.random.default_rng(5)
    b, h, kvh, d, theta = 3, 8, 2, 128, 500000.0
    q = rng.standard_normal((b, h, d)).astype(np.float16)
    k = rng.standard_normal((b, kvh, d)).astype(np.float16)
    pos = np.array([7, 1000, 31], dtype=np.int32)
    inv = (1.0 / (theta ** (np.arange(0, d, 2, dtype=np.float32) / np.float32(d)))).astype(np.float32)
    qd, kd = torch.from_numpy(q).to(DEV), torch.from_numpy(k).to(DEV)
    ops.rope_inplace(qd, kd, torch.from_numpy(pos).to(DEV), torch.from_numpy(inv).to(DEV))
    for got, src in ((qd, q), (kd, k)):
        ref = np.stack([O.rope_ref(src[i][:, None, :], pos[i:i + 1], theta)[:, 0] for i in range(b)])
        assert_close(to_np(got), ref.astype(np.float64), torch.float16, "rope")


@pytest.mark.parametrize("shape,dt", [((4, 1000), torch.float16), ((3, 1001), torch.float16), ((64, 1024), torch.bfloat16),
                                      ((5, 333), torch.float32)])
def test_silu_mul(shape, dt):
    """Whole multiples of eight 16-bit elements take the 16-byte-vector kernel, the rest one element per
    thread: same numbers."""
    rng = np.random.default_rng(6)
    g = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dt)
    u = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dt)
    y = ops.silu_mul(g.to(DEV), u.to(DEV))
    ref = O.silu(g.double().numpy()) * u.double().numpy()
    assert_close(to_np(y), ref, dt, "silu_mul")
    # an unaligned view of the same data goes through the scalar kernel and agrees bit for bit
    gp = torch.zeros(g.numel() + 1, dtype=dt, device=DEV)[1:].view(shape).copy_(g)
    up = torch.zeros(u.numel() + 1, dtype=dt, device=DEV)[1:].view(shape).copy_(u)
    assert torch.equal(ops.silu_mul(gp, up), y)


@pytest.mark.parametrize("m,n,dt", [(1, 128256, torch.float16), (4, 32000, torch.float16), (3, 1000, torch.float32),
                                     (2, 7, torch.bfloat16)])
def test_argmax_first_maximum(m, n, dt):
    gen = torch.Generator().manual_seed(m * 131 + n)
    x = torch.randn((m, n), generator=gen).to(dt)
    # a tie at the maximum: the smaller index wins
    top = x.float().max(dim=1).values
    for r in range(m):
        i, j = sorted(torch.randint(0, n, (2,), generator=gen).tolist())
        x[r, i] = top[r] + 1.0
        x[r, j] = top[r] + 1.0
    got = ops.argmax(x.to(DEV)).cpu()
    xf = x.float()
    want = torch.tensor([int(torch.nonzero(xf[r] == xf[r].max())[0]) for r in range(m)])
    assert torch.equal(got, want)

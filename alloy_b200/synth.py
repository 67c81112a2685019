"""Seeded synthetic GGUF blocks, activations and KV data of the benchmark shapes.

Two families:

* NumPy generators (``np.random.default_rng(seed)``) for tests and small
  cases.  ``q4k_blocks`` / ``q6k_blocks`` / ``q8_0_weight`` draw block contents
  the way the benchmark configurations specify: fp16 ``d`` (and ``dmin``)
  uniform in [1e-4, 2e-3], every packed byte uniform, so the 6-bit scales/mins
  are uniform in 0..63 and the nibbles uniform in 0..15.
  ``q4k_blocks_signed`` mirrors the generator of the reference's kernel tests
  (``tests/kernels/test_quant_q4k_native.py:35-42``: ``d ~ N(0, .02)``,
  ``dmin ~ N(0, .01)``, signed) and is kept for unit tests only.
* torch generators that fill device memory directly for the full-size
  benchmark matrices (gigabytes of blocks are not staged through the host).

The Q6_K int8 sub-block scales are drawn uniform over -128..127; the
benchmark configuration leaves that range open.
"""

from __future__ import annotations

import numpy as np
import torch

Q4K_BLOCK_BYTES = 144
Q6K_BLOCK_BYTES = 210
Q8_0_BLOCK_BYTES = 34
QK_K = 256
D_LO, D_HI = 1e-4, 2e-3


def _check_k(k: int, align: int = QK_K) -> int:
    if k % align != 0:
        raise ValueError(f"contraction dim {k} not divisible by {align}")
    return k // align


# --------------------------------------------------------------------------- numpy


def q4k_blocks(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """(n, k/256*144) uint8 Q4_K super-blocks, benchmark distribution."""
    nb = _check_k(k)
    blk = rng.integers(0, 256, size=(n, nb, Q4K_BLOCK_BYTES), dtype=np.uint8)
    d = rng.uniform(D_LO, D_HI, size=(n, nb)).astype(np.float16)
    dmin = rng.uniform(D_LO, D_HI, size=(n, nb)).astype(np.float16)
    blk[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    blk[:, :, 2:4] = dmin.view(np.uint8).reshape(n, nb, 2)
    return blk.reshape(n, nb * Q4K_BLOCK_BYTES)


def q4k_blocks_signed(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """Q4_K blocks with signed normal d/dmin, as the reference's tests draw them."""
    nb = _check_k(k)
    blk = rng.integers(0, 256, size=(n, nb, Q4K_BLOCK_BYTES), dtype=np.uint8)
    d = (rng.standard_normal((n, nb)) * 0.02).astype(np.float16)
    dmin = (rng.standard_normal((n, nb)) * 0.01).astype(np.float16)
    blk[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    blk[:, :, 2:4] = dmin.view(np.uint8).reshape(n, nb, 2)
    return blk.reshape(n, nb * Q4K_BLOCK_BYTES)


def q6k_blocks(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """(n, k/256*210) uint8 Q6_K super-blocks: ql[128] qh[64] int8 sc[16] f16 d."""
    nb = _check_k(k)
    blk = rng.integers(0, 256, size=(n, nb, Q6K_BLOCK_BYTES), dtype=np.uint8)
    d = rng.uniform(D_LO, D_HI, size=(n, nb)).astype(np.float16)
    blk[:, :, 208:210] = d.view(np.uint8).reshape(n, nb, 2)
    return blk.reshape(n, nb * Q6K_BLOCK_BYTES)


def q8_0_wire(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """(n, k/32*34) uint8 Q8_0 wire blocks: f16 d + 32 int8 codes."""
    g = _check_k(k, 32)
    blk = rng.integers(0, 256, size=(n, g, Q8_0_BLOCK_BYTES), dtype=np.uint8)
    d = rng.uniform(D_LO, D_HI, size=(n, g)).astype(np.float16)
    blk[:, :, 0:2] = d.view(np.uint8).reshape(n, g, 2)
    return blk.reshape(n, g * Q8_0_BLOCK_BYTES)


def activations(rng: np.random.Generator, m: int, k: int, dtype=np.float16) -> np.ndarray:
    """(m, k) N(0,1) activations."""
    return rng.standard_normal((m, k)).astype(dtype)


def kv_rows(rng: np.random.Generator, shape, scale: float = 1.0) -> np.ndarray:
    """fp16 N(0, scale) K or V rows of the given shape (last axis = head_dim)."""
    return (rng.standard_normal(shape) * scale).astype(np.float16)


# --------------------------------------------------------------------------- torch (device)


def _uniform_f16_bytes(shape, gen: torch.Generator, device, d_scale: float = 1.0) -> torch.Tensor:
    d = torch.empty(shape, dtype=torch.float32, device=device).uniform_(D_LO, D_HI, generator=gen)
    return (d * d_scale).to(torch.float16).view(torch.uint8)


def q4k_blocks_device(n: int, k: int, gen: torch.Generator, device="cuda",
                      d_scale: float = 1.0, centered: bool = False) -> torch.Tensor:
    """Device-side Q4_K blocks with the benchmark distribution (d, dmin times ``d_scale``).

    ``centered``: every sub-block gets min == scale and the block dmin = 7.5 d, so that a weight is
    d * sc * (q - 7.5): zero-mean like a quantised model's weights (a stack of random layers then
    keeps its residual stream inside fp16).  Uncentered blocks have a large positive mean.
    """
    nb = _check_k(k)
    blk = torch.randint(0, 256, (n, nb, Q4K_BLOCK_BYTES), dtype=torch.uint8, device=device,
                        generator=gen)
    d = _uniform_f16_bytes((n, nb), gen, device, d_scale)
    blk[:, :, 0:2] = d.view(n, nb, 2)
    if centered:
        blk[:, :, 2:4] = (d.view(torch.float16).float() * 7.5).to(torch.float16).view(torch.uint8).view(n, nb, 2)
        blk[:, :, 8:12] = blk[:, :, 4:8]                      # mins 0-3 (and the high bits of 4-7) = scales
        lo = blk[:, :, 12:16] & 0x0F
        blk[:, :, 12:16] = lo | (lo << 4)                     # low bits of mins 4-7 = those of scales 4-7
    else:
        blk[:, :, 2:4] = _uniform_f16_bytes((n, nb), gen, device, d_scale).view(n, nb, 2)
    return blk.view(n, nb * Q4K_BLOCK_BYTES)


def q6k_blocks_device(n: int, k: int, gen: torch.Generator, device="cuda",
                      d_scale: float = 1.0) -> torch.Tensor:
    """Device-side Q6_K blocks with the benchmark distribution (d times ``d_scale``)."""
    nb = _check_k(k)
    blk = torch.randint(0, 256, (n, nb, Q6K_BLOCK_BYTES), dtype=torch.uint8, device=device,
                        generator=gen)
    blk[:, :, 208:210] = _uniform_f16_bytes((n, nb), gen, device, d_scale).view(n, nb, 2)
    return blk.view(n, nb * Q6K_BLOCK_BYTES)


def q8_0_weight_device(n: int, k: int, gen: torch.Generator, device="cuda"):
    """Device-side normalised Q8_0 weight: int8 (n,k) codes + fp16 (n,k/32) scales."""
    g = _check_k(k, 32)
    q = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=device, generator=gen)
    s = torch.empty((n, g), dtype=torch.float32, device=device).uniform_(D_LO, D_HI, generator=gen)
    return q, s.to(torch.float16)

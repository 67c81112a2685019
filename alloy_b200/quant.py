"""Quantised ``Linear`` / ``Embedding`` modules over GGUF-native packed buffers.

Interface of the reference's ``packages/alloy-server/src/alloy_server/gguf/quant.py``: the
format table ``QUANT_FORMATS`` (:49-82), ``validate_quant_buffers`` (:84-105), the
``GGUFQ*Linear`` / ``GGUFQ*Embedding`` classes with keyword-only constructors taking the
format's buffers by name (:108-228), and the wire-block splitters ``split_q8_0_weight``
(:497-521) and ``split_q5_0_weight`` (:414-490).  The names, buffer layouts and exception
types are that interface; the implementation is this package's own.  The reference's module
itself also runs unchanged on top of ``alloy_b200.ops`` (it only binds ``torch.ops.alloy.*``).

Every forward is one ``torch.ops.alloy`` call: on a CUDA device the sm_100a kernels, anywhere
else ``NotImplementedError`` (there is no CPU path).
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass

import numpy as np
import torch

from . import ops  # noqa: F401  (registers torch.ops.alloy.*)

_A = torch.ops.alloy


@dataclass(frozen=True)
class QuantBuffer:
    """A packed buffer of a format: module attribute, element type, columns for a given K."""

    name: str
    dtype: torch.dtype
    cols: Callable[[int], int]


@dataclass(frozen=True)
class QuantFormat:
    name: str
    align: int                       # K must be a multiple of this
    mm_op: Callable
    embed_op: Callable
    buffers: tuple[QuantBuffer, ...]

    @property
    def buffer_names(self) -> tuple[str, ...]:
        return tuple(b.name for b in self.buffers)

    def shapes(self, rows: int, dim: int) -> dict[str, tuple[int, int]]:
        return {b.name: (rows, b.cols(dim)) for b in self.buffers}


def _per(numer: int, denom: int) -> Callable[[int], int]:
    """Columns = K // denom * numer (bytes or elements per K elements)."""
    return lambda k: k // denom * numer


# name: (K alignment, mm op, embedding op, [(buffer, dtype, columns per K)])
_TABLE = {
    "q8_0": (32, _A.gguf_q8_0_mm, _A.gguf_q8_0_embedding,
             [("qweight", torch.int8, _per(1, 1)), ("scales", torch.float16, _per(1, 32))]),
    "q4_k": (256, _A.gguf_q4_k_mm, _A.gguf_q4_k_embedding, [("blocks", torch.uint8, _per(144, 256))]),
    "q5_0": (32, _A.gguf_q5_0_mm, _A.gguf_q5_0_embedding,
             [("qweight", torch.uint8, _per(1, 2)), ("qhigh", torch.uint8, _per(1, 2)),
              ("scales", torch.float16, _per(1, 32))]),
    "q6_k": (256, _A.gguf_q6_k_mm, _A.gguf_q6_k_embedding, [("qweight", torch.uint8, _per(210, 256))]),
}
QUANT_FORMATS: dict[str, QuantFormat] = {
    name: QuantFormat(name, align, mm.default, emb.default, tuple(QuantBuffer(*b) for b in bufs))
    for name, (align, mm, emb, bufs) in _TABLE.items()
}


def validate_quant_buffers(fmt: QuantFormat, buffers: dict[str, torch.Tensor], *, rows: int, dim: int,
                           kind: str) -> None:
    """``ValueError`` for a wrong buffer set, K alignment, rank or shape; ``TypeError`` for a dtype."""
    who = f"{fmt.name} {kind}"
    missing = [n for n in fmt.buffer_names if n not in buffers]
    extra = [n for n in buffers if n not in fmt.buffer_names]
    if missing or extra:
        raise ValueError(f"{who} takes buffers {fmt.buffer_names}; missing {missing}, unexpected {extra}")
    if dim % fmt.align:
        raise ValueError(f"{who}: dim {dim} is not a multiple of {fmt.align}")
    want = fmt.shapes(rows, dim)
    for spec in fmt.buffers:
        t = buffers[spec.name]
        if t.dtype is not spec.dtype:
            raise TypeError(f"{who}: buffer {spec.name!r} must be {spec.dtype}, is {t.dtype}")
        if t.ndim != 2 or tuple(t.shape) != want[spec.name]:
            raise ValueError(f"{who}: buffer {spec.name!r} must have shape {want[spec.name]} for rows={rows} "
                             f"dim={dim}, has {tuple(t.shape)}")


class _PackedModule(torch.nn.Module):
    FORMAT: QuantFormat

    def _adopt(self, buffers: dict[str, torch.Tensor], rows: int, dim: int, kind: str) -> None:
        validate_quant_buffers(self.FORMAT, buffers, rows=rows, dim=dim, kind=kind)
        for name in self.FORMAT.buffer_names:
            self.register_buffer(name, buffers[name].contiguous())

    def _packed(self) -> list[torch.Tensor]:
        return [getattr(self, name) for name in self.FORMAT.buffer_names]


class GGUFQuantLinear(_PackedModule):
    """``y = x W^T (+ bias)`` on packed weights; a subclass fixes ``FORMAT``."""

    def __init__(self, *, in_features: int, out_features: int, bias: torch.nn.Parameter | None = None,
                 **buffers: torch.Tensor) -> None:
        super().__init__()
        self.in_features, self.out_features = int(in_features), int(out_features)
        self._adopt(buffers, self.out_features, self.in_features, "linear")
        self.register_parameter("bias", bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = self.FORMAT.mm_op(x.reshape(-1, self.in_features).contiguous(), *self._packed())
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)


class GGUFQuantEmbedding(_PackedModule):
    """Row gather + dequantise to float32 (the reference's embedding ops return float32)."""

    def __init__(self, *, num_embeddings: int, embedding_dim: int, embed_scale: float = 1.0,
                 **buffers: torch.Tensor) -> None:
        super().__init__()
        self.num_embeddings, self.embedding_dim = int(num_embeddings), int(embedding_dim)
        self.embed_scale = float(embed_scale)
        self._adopt(buffers, self.num_embeddings, self.embedding_dim, "embedding")

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        rows = self.FORMAT.embed_op(input_ids, *self._packed())
        return rows if self.embed_scale == 1.0 else rows * self.embed_scale


def _pin(base: type, fmt: str, name: str) -> type:
    return type(name, (base,), {"FORMAT": QUANT_FORMATS[fmt], "__module__": __name__,
                                "__doc__": f"{base.__name__} over {fmt} buffers."})


GGUFQ8_0Linear = _pin(GGUFQuantLinear, "q8_0", "GGUFQ8_0Linear")
GGUFQ4_KLinear = _pin(GGUFQuantLinear, "q4_k", "GGUFQ4_KLinear")
GGUFQ5_0Linear = _pin(GGUFQuantLinear, "q5_0", "GGUFQ5_0Linear")
GGUFQ6_KLinear = _pin(GGUFQuantLinear, "q6_k", "GGUFQ6_KLinear")
GGUFQ8_0Embedding = _pin(GGUFQuantEmbedding, "q8_0", "GGUFQ8_0Embedding")
GGUFQ4_KEmbedding = _pin(GGUFQuantEmbedding, "q4_k", "GGUFQ4_KEmbedding")
GGUFQ5_0Embedding = _pin(GGUFQuantEmbedding, "q5_0", "GGUFQ5_0Embedding")
GGUFQ6_KEmbedding = _pin(GGUFQuantEmbedding, "q6_k", "GGUFQ6_KEmbedding")


def _wire_blocks(weights: np.ndarray, in_features: int, out_features: int, block_bytes: int, fmt: str) -> np.ndarray:
    if weights.dtype != np.uint8:
        raise TypeError(f"{fmt} weights must be uint8 bytes, got {weights.dtype}")
    if in_features % 32:
        raise ValueError(f"{fmt} in_features must be divisible by 32, got {in_features}")
    want = (out_features, in_features // 32 * block_bytes)
    if tuple(weights.shape) != want:
        raise ValueError(f"{fmt} packed weight is {tuple(weights.shape)}, expected {want}")
    return np.ascontiguousarray(weights).reshape(out_features, in_features // 32, block_bytes)


def split_q8_0_weight(*, weights: np.ndarray, in_features: int,
                      out_features: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Q8_0 wire blocks ``{fp16 d; int8 q[32]}`` (N, K/32*34) -> int8 codes (N, K) + fp16 scales (N, K/32)."""
    blk = _wire_blocks(weights, in_features, out_features, 34, "Q8_0")
    scales = blk[:, :, :2].copy().view(np.float16)[:, :, 0]
    codes = blk[:, :, 2:].copy().view(np.int8).reshape(out_features, in_features)
    return torch.from_numpy(codes), torch.from_numpy(np.ascontiguousarray(scales))


def split_q5_0_weight(*, weights: np.ndarray, in_features: int,
                      out_features: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Q5_0 wire blocks ``{fp16 d; u8 qh[4]; u8 qs[16]}`` (N, K/32*22) -> K-sequential qweight (N, K/2),
    qhigh (N, K/2) and fp16 scales (N, K/32): byte k/2 holds element k in its low nibble (fifth bit in
    bit 0 of qhigh) and element k+1 in its high nibble (fifth bit in bit 4)."""
    blk = _wire_blocks(weights, in_features, out_features, 22, "Q5_0")
    scales = blk[:, :, :2].copy().view(np.float16)[:, :, 0]
    bits = np.unpackbits(blk[:, :, 2:6], axis=-1, bitorder="little")          # element l's fifth bit at [l]
    nib = np.concatenate([blk[:, :, 6:] & 15, blk[:, :, 6:] >> 4], axis=-1)   # wire order -> K order
    pack = lambda a: (a[:, :, 0::2] | (a[:, :, 1::2] << 4)).reshape(out_features, in_features // 2)
    return (torch.from_numpy(pack(nib)), torch.from_numpy(pack(bits)),
            torch.from_numpy(np.ascontiguousarray(scales)))

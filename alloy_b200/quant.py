"""GGUF-native quantised modules: the module/buffer contract of the reference's
``packages/alloy-server/src/alloy_server/gguf/quant.py`` (``QuantFormat`` and
``QUANT_FORMATS`` :49-82, ``validate_quant_buffers`` :84-105, ``GGUFQuantLinear``
:108-141, ``GGUFQuantEmbedding`` :144-172, ``split_q8_0_weight`` :497-521) for
the three formats of the hot path.  The modules call ``torch.ops.alloy.*``, so
on a CUDA device they run the sm_100a kernels and anywhere else they raise.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass

import numpy as np
import torch

from . import ops  # noqa: F401  (registers torch.ops.alloy.*)


@dataclass(frozen=True)
class QuantBuffer:
    """One packed buffer of a format: attribute name, dtype, columns as a function of K."""

    name: str
    dtype: torch.dtype
    cols: Callable[[int], int]


@dataclass(frozen=True)
class QuantFormat:
    name: str
    align: int
    mm_op: Callable
    embed_op: Callable
    buffers: tuple[QuantBuffer, ...]

    @property
    def buffer_names(self) -> tuple[str, ...]:
        return tuple(b.name for b in self.buffers)


QUANT_FORMATS: dict[str, QuantFormat] = {
    "q8_0": QuantFormat("q8_0", 32, torch.ops.alloy.gguf_q8_0_mm.default,
                        torch.ops.alloy.gguf_q8_0_embedding.default, (
        QuantBuffer("qweight", torch.int8, lambda k: k),
        QuantBuffer("scales", torch.float16, lambda k: k // 32),
    )),
    "q4_k": QuantFormat("q4_k", 256, torch.ops.alloy.gguf_q4_k_mm.default,
                        torch.ops.alloy.gguf_q4_k_embedding.default, (
        QuantBuffer("blocks", torch.uint8, lambda k: (k // 256) * 144),
    )),
    "q6_k": QuantFormat("q6_k", 256, torch.ops.alloy.gguf_q6_k_mm.default,
                        torch.ops.alloy.gguf_q6_k_embedding.default, (
        QuantBuffer("qweight", torch.uint8, lambda k: (k // 256) * 210),
    )),
}


def validate_quant_buffers(fmt: QuantFormat, buffers: dict[str, torch.Tensor], *, rows: int,
                           dim: int, kind: str) -> None:
    if set(buffers) != set(fmt.buffer_names):
        raise ValueError(f"{fmt.name} {kind} expects buffers {fmt.buffer_names}, got {tuple(buffers)}")
    if dim % fmt.align != 0:
        raise ValueError(f"{fmt.name} {kind} dim {dim} not divisible by {fmt.align}")
    for b in fmt.buffers:
        t = buffers[b.name]
        if t.dtype is not b.dtype:
            raise TypeError(f"{fmt.name} {kind} buffer {b.name!r} requires {b.dtype}, got {t.dtype}")
        if t.ndim != 2:
            raise ValueError(f"{fmt.name} {kind} buffer {b.name!r} must be rank-2, got {tuple(t.shape)}")
        expected = (rows, b.cols(dim))
        if tuple(t.shape) != expected:
            raise ValueError(f"{fmt.name} {kind} buffer {b.name!r} shape {tuple(t.shape)} != {expected} "
                             f"(rows={rows} dim={dim})")


class GGUFQuantLinear(torch.nn.Module):
    """Linear over GGUF-native packed weights; subclasses pin ``FORMAT``."""

    FORMAT: QuantFormat

    def __init__(self, *, in_features: int, out_features: int,
                 bias: torch.nn.Parameter | None = None, **buffers: torch.Tensor) -> None:
        super().__init__()
        validate_quant_buffers(self.FORMAT, buffers, rows=out_features, dim=in_features, kind="linear")
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        for b in self.FORMAT.buffers:
            self.register_buffer(b.name, buffers[b.name].contiguous())
        if bias is not None:
            self.bias = bias
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x_shape = x.shape
        flat = x.reshape(-1, self.in_features).contiguous()
        out = self.FORMAT.mm_op(flat, *(self._buffers[b.name] for b in self.FORMAT.buffers))
        if self.bias is not None:
            out = out + self.bias
        return out.reshape(*x_shape[:-1], self.out_features)


class GGUFQuantEmbedding(torch.nn.Module):
    """Embedding over GGUF-native packed weights; returns float32 like the reference."""

    FORMAT: QuantFormat

    def __init__(self, *, num_embeddings: int, embedding_dim: int, embed_scale: float = 1.0,
                 **buffers: torch.Tensor) -> None:
        super().__init__()
        validate_quant_buffers(self.FORMAT, buffers, rows=num_embeddings, dim=embedding_dim,
                               kind="embedding")
        self.num_embeddings = int(num_embeddings)
        self.embedding_dim = int(embedding_dim)
        self.embed_scale = float(embed_scale)
        for b in self.FORMAT.buffers:
            self.register_buffer(b.name, buffers[b.name].contiguous())

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        out = self.FORMAT.embed_op(input_ids, *(self._buffers[b.name] for b in self.FORMAT.buffers))
        if self.embed_scale != 1.0:
            out = out * self.embed_scale
        return out


class GGUFQ8_0Linear(GGUFQuantLinear):
    FORMAT = QUANT_FORMATS["q8_0"]


class GGUFQ4_KLinear(GGUFQuantLinear):
    FORMAT = QUANT_FORMATS["q4_k"]


class GGUFQ6_KLinear(GGUFQuantLinear):
    FORMAT = QUANT_FORMATS["q6_k"]


class GGUFQ8_0Embedding(GGUFQuantEmbedding):
    FORMAT = QUANT_FORMATS["q8_0"]


class GGUFQ4_KEmbedding(GGUFQuantEmbedding):
    FORMAT = QUANT_FORMATS["q4_k"]


class GGUFQ6_KEmbedding(GGUFQuantEmbedding):
    FORMAT = QUANT_FORMATS["q6_k"]


def split_q8_0_weight(*, weights: np.ndarray, in_features: int,
                      out_features: int) -> tuple[torch.Tensor, torch.Tensor]:
    """34-byte Q8_0 wire blocks (N, K/32*34) uint8 -> int8 (N,K) codes + fp16 (N,K/32) scales."""
    if weights.dtype != np.uint8:
        raise TypeError(f"Q8_0 weights must be uint8 bytes, got {weights.dtype}")
    if in_features % 32 != 0:
        raise ValueError(f"Q8_0 in_features must be divisible by 32, got {in_features}")
    groups = in_features // 32
    expected = (out_features, groups * 34)
    if weights.shape != expected:
        raise ValueError("Q8_0 packed weight shape does not match linear dimensions: "
                         f"weights={tuple(weights.shape)} expected={expected}")
    wire = np.ascontiguousarray(weights).reshape(out_features, groups, 34)
    scales = np.ascontiguousarray(wire[:, :, :2]).view(np.float16).reshape(out_features, groups)
    codes = np.ascontiguousarray(wire[:, :, 2:]).view(np.int8).reshape(out_features, in_features)
    return torch.from_numpy(codes.copy()), torch.from_numpy(scales.copy())

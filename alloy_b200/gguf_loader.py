"""GGUF file -> packed weight buffers for the quantised decoder.

The counterpart of the reference's load path for causal LMs
(``packages/alloy-server/src/alloy_server/gguf/loader.py:97-250`` walks the GGUF tensor table and
swaps quantised modules in; ``gguf/quant.py:230-348`` maps a tensor's ggml type to a module and
keeps the raw blocks as the module's buffer; ``gguf/meta.py`` caches the parsed header).  Here the
file is parsed directly -- header, metadata, tensor table, aligned data section of GGUF v2/v3 --
and the tensors of a Llama-architecture checkpoint are handed to ``QuantLlamaDecoder`` as they
are on disk: Q4_K / Q6_K rows are the wire format of the kernels, nothing is repacked.

Two fix-ups the reference's stack also performs (through ``transformers``' GGUF tensor
processors): q/k rows of Llama checkpoints are stored permuted for interleaved RoPE and are put
back into rotate-half order (a pure row permutation, so it works on packed rows), and a missing
``output.weight`` ties the head to the token embedding.
"""

from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass, field

import numpy as np
import torch

GGUF_MAGIC = 0x46554747  # "GGUF" little-endian
DEFAULT_ALIGNMENT = 32

# ggml type id -> (name, elements per block, bytes per block)
GGML_TYPES = {
    0: ("f32", 1, 4),
    1: ("f16", 1, 2),
    8: ("q8_0", 32, 34),
    12: ("q4_k", 256, 144),
    14: ("q6_k", 256, 210),
    30: ("bf16", 1, 2),
}

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


class GGUFError(ValueError):
    pass


@dataclass
class GGUFTensor:
    name: str
    ggml_type: int
    shape: tuple[int, ...]            # logical shape, outermost first: (N, K) for a matrix
    offset: int                       # byte offset inside the data section
    nbytes: int
    data: np.ndarray | None = None    # uint8 view of the file (set by read_gguf)

    @property
    def type_name(self) -> str:
        return GGML_TYPES[self.ggml_type][0] if self.ggml_type in GGML_TYPES else f"ggml_type_{self.ggml_type}"

    def rows(self) -> np.ndarray:
        """The tensor as rows of packed bytes: (N, row_bytes) uint8 (1-D tensors: one row)."""
        n = self.shape[0] if len(self.shape) > 1 else 1
        return self.data.reshape(n, self.nbytes // n)


@dataclass
class GGUFFile:
    version: int
    metadata: dict
    tensors: dict[str, GGUFTensor]
    alignment: int
    data_offset: int
    _mm: object = field(default=None, repr=False)


class _Cursor:
    def __init__(self, buf) -> None:
        self.buf, self.pos = buf, 0

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GGUFError("truncated GGUF file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += size
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GGUFError("truncated GGUF string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype: int):
        if vtype in _SCALAR:
            return self.take(_SCALAR[vtype])
        if vtype == _T_STRING:
            return self.string()
        if vtype == _T_ARRAY:
            etype = self.take("<I")
            count = self.take("<Q")
            if etype in _SCALAR and etype != 7:
                fmt = _SCALAR[etype]
                size = struct.calcsize(fmt)
                if self.pos + size * count > len(self.buf):
                    raise GGUFError("truncated GGUF array")
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt), count=count, offset=self.pos)
                self.pos += size * count
                return arr
            return [self.value(etype) for _ in range(count)]
        raise GGUFError(f"unknown GGUF metadata value type {vtype}")


def read_gguf(path) -> GGUFFile:
    """Parse a GGUF v2/v3 file; tensor data stay memory-mapped."""
    f = open(path, "rb")
    try:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    finally:
        f.close()
    c = _Cursor(mm)
    if len(mm) < 24 or c.take("<I") != GGUF_MAGIC:
        raise GGUFError(f"{path}: not a GGUF file")
    version = c.take("<I")
    if version not in (2, 3):
        raise GGUFError(f"{path}: GGUF version {version} is not supported (2 and 3 are)")
    n_tensors, n_kv = c.take("<Q"), c.take("<Q")
    meta: dict = {}
    for _ in range(n_kv):
        key = c.string()
        meta[key] = c.value(c.take("<I"))
    align = int(meta.get("general.alignment", DEFAULT_ALIGNMENT))
    if align <= 0 or align & (align - 1):
        raise GGUFError(f"{path}: alignment {align} is not a power of two")
    tensors: dict[str, GGUFTensor] = {}
    for _ in range(n_tensors):
        name = c.string()
        nd = c.take("<I")
        if nd < 1 or nd > 4:
            raise GGUFError(f"{path}: tensor {name!r} has {nd} dimensions")
        ne = [c.take("<Q") for _ in range(nd)]          # ne[0] varies fastest
        gt = c.take("<I")
        off = c.take("<Q")
        n_el = int(np.prod(ne, dtype=np.int64))
        if gt in GGML_TYPES:
            _, per, bb = GGML_TYPES[gt]
            if ne[0] % per:
                raise GGUFError(f"{path}: tensor {name!r}: row of {ne[0]} elements is not whole {per}-element blocks")
            nbytes = n_el // per * bb
        else:
            nbytes = -1                                  # unknown type: listed, not readable
        tensors[name] = GGUFTensor(name, gt, tuple(reversed(ne)), off, nbytes)
    data_offset = (c.pos + align - 1) // align * align
    whole = np.frombuffer(mm, dtype=np.uint8)
    for t in tensors.values():
        if t.nbytes < 0:
            continue
        if t.offset % align:
            raise GGUFError(f"{path}: tensor {t.name!r} is not aligned to {align} bytes")
        lo = data_offset + t.offset
        if lo + t.nbytes > len(mm):
            raise GGUFError(f"{path}: tensor {t.name!r} runs past the end of the file")
        t.data = whole[lo:lo + t.nbytes]
    return GGUFFile(version, meta, tensors, align, data_offset, mm)


# ------------------------------------------------------------------------------- Llama checkpoints


@dataclass
class Packed:
    """One weight as the kernels take it: format name + (N, row_bytes) uint8 (or a dense vector)."""
    fmt: str
    tensor: torch.Tensor


@dataclass
class LlamaWeights:
    embed: Packed
    layers: list[dict[str, Packed]]       # wq wk wv wo wg wu wd norm_in norm_post
    norm_final: Packed
    head: Packed
    tied_head: bool


def llama_shape(meta: dict, tensors: dict[str, GGUFTensor]):
    """``LlamaShape`` from the metadata of a ``general.architecture == 'llama'`` file."""
    from .llama import LlamaShape

    arch = meta.get("general.architecture")
    if arch != "llama":
        raise GGUFError(f"architecture {arch!r} is not supported (llama is)")

    def need(key):
        if f"llama.{key}" not in meta:
            raise GGUFError(f"metadata key llama.{key} is missing")
        return meta[f"llama.{key}"]

    hidden, heads = int(need("embedding_length")), int(need("attention.head_count"))
    kv_heads = int(meta.get("llama.attention.head_count_kv", heads))
    head_dim = int(meta.get("llama.attention.key_length", hidden // heads))
    vocab = int(meta.get("llama.vocab_size", tensors["token_embd.weight"].shape[0]))
    return LlamaShape(layers=int(need("block_count")), hidden=hidden, ffn=int(need("feed_forward_length")),
                      heads=heads, kv_heads=kv_heads, head_dim=head_dim, vocab=vocab,
                      rope_theta=float(meta.get("llama.rope.freq_base", 10000.0)),
                      eps=float(meta.get("llama.attention.layer_norm_rms_epsilon", 1e-5)))


def unpermute_qk_rows(rows: torch.Tensor, n_head: int) -> torch.Tensor:
    """Rows of a q/k projection from the checkpoint's interleaved-RoPE order back to rotate-half
    order: per head, stored row 2i + j is row j * (head_dim / 2) + i.  Works on packed rows."""
    n = rows.shape[0]
    if n % (2 * n_head):
        raise GGUFError(f"{n} rows do not split into {n_head} heads of even size")
    return rows.reshape(n_head, n // n_head // 2, 2, -1).transpose(1, 2).reshape(n, -1).contiguous()


_LINEAR_FORMATS = ("q4_k", "q6_k")


def _matrix(f: GGUFFile, name: str, device, n: int, k: int) -> Packed:
    if name not in f.tensors:
        raise GGUFError(f"tensor {name!r} is missing")
    t = f.tensors[name]
    if t.type_name not in _LINEAR_FORMATS:
        raise GGUFError(f"tensor {name!r} is {t.type_name}; this decoder takes q4_k / q6_k matrices")
    if t.shape != (n, k):
        raise GGUFError(f"tensor {name!r} has shape {t.shape}, expected {(n, k)}")
    return Packed(t.type_name, torch.from_numpy(np.array(t.rows())).to(device))      # a copy: the map is read-only


def _vector(f: GGUFFile, name: str, device, n: int, dtype: torch.dtype) -> Packed:
    if name not in f.tensors:
        raise GGUFError(f"tensor {name!r} is missing")
    t = f.tensors[name]
    if t.shape != (n,):
        raise GGUFError(f"tensor {name!r} has shape {t.shape}, expected {(n,)}")
    if t.type_name == "f32":
        v = torch.from_numpy(np.frombuffer(t.data, dtype=np.float32).copy())
    elif t.type_name == "f16":
        v = torch.from_numpy(np.frombuffer(t.data, dtype=np.float16).copy())
    else:
        raise GGUFError(f"tensor {name!r} is {t.type_name}; norm weights must be f32 or f16")
    return Packed("dense", v.to(dtype).to(device))


def load_llama_weights(f: GGUFFile, device="cuda", dtype: torch.dtype = torch.float16):
    """(LlamaShape, LlamaWeights) of a Llama-architecture GGUF, tensors on ``device``."""
    shape = llama_shape(f.metadata, f.tensors)
    s = shape
    hd, kvd = s.heads * s.head_dim, s.kv_heads * s.head_dim
    embed = _matrix(f, "token_embd.weight", device, s.vocab, s.hidden)
    layers = []
    for i in range(s.layers):
        p = f"blk.{i}."
        wq = _matrix(f, p + "attn_q.weight", device, hd, s.hidden)
        wk = _matrix(f, p + "attn_k.weight", device, kvd, s.hidden)
        wq.tensor = unpermute_qk_rows(wq.tensor, s.heads)
        wk.tensor = unpermute_qk_rows(wk.tensor, s.kv_heads)
        layers.append({
            "wq": wq, "wk": wk,
            "wv": _matrix(f, p + "attn_v.weight", device, kvd, s.hidden),
            "wo": _matrix(f, p + "attn_output.weight", device, s.hidden, hd),
            "wg": _matrix(f, p + "ffn_gate.weight", device, s.ffn, s.hidden),
            "wu": _matrix(f, p + "ffn_up.weight", device, s.ffn, s.hidden),
            "wd": _matrix(f, p + "ffn_down.weight", device, s.hidden, s.ffn),
            "norm_in": _vector(f, p + "attn_norm.weight", device, s.hidden, dtype),
            "norm_post": _vector(f, p + "ffn_norm.weight", device, s.hidden, dtype),
        })
    norm_final = _vector(f, "output_norm.weight", device, s.hidden, dtype)
    tied = "output.weight" not in f.tensors
    head = embed if tied else _matrix(f, "output.weight", device, s.vocab, s.hidden)
    return shape, LlamaWeights(embed, layers, norm_final, head, tied)


def load_llama_decoder(path, batch: int, context: int, *, device="cuda", kv: str = "f16", **kw):
    """``QuantLlamaDecoder`` serving the weights of a Llama-architecture GGUF file."""
    from .llama import QuantLlamaDecoder

    f = read_gguf(path)
    shape, weights = load_llama_weights(f, device)
    return QuantLlamaDecoder(shape, batch, context, device=device, kv=kv, weights=weights, **kw)

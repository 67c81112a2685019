"""``torch.ops.alloy.*`` — the operator surface of the quantised-LLM hot path.

The schemas are the ones the reference declares in
``packages/alloy-torch/src/alloy_torch/custom_ops.py`` (``gguf_q4_k_mm`` :47-49,
``batched_gguf_q4_k_mm`` :50-52, ``gguf_q4_k_silu`` / ``_gelu`` :53-58,
``gguf_q4_k_embedding`` :67-69, ``gguf_q6_k_*`` :96-102, ``gguf_q8_0_*`` :103-111,
``attention_cache`` :136-140, ``attention_cache_q8`` :144-150), so modules
written against the reference call these unchanged.  The reference registers
only ``Meta`` kernels and executes the ops on Metal through an FX handler
table (``packages/alloy-torch/src/alloy_torch/ops/registry.py:280-330``); here
each op has a ``CUDA`` kernel that calls the C ABI of ``liballoy_b200.so`` on
the current stream, plus the same ``Meta`` shape functions.  There is no CPU
implementation, as in the reference: a CPU call raises ``NotImplementedError``.

Two ops have no reference schema: ``attention_cache_q8_paged`` (decode
attention over the 16-token-paged pool of 34-byte q8_0 blocks) and
``linear_residual`` (row-parallel projection with the residual add fused).
"""

from __future__ import annotations

import ctypes as C
import math
from collections.abc import Sequence

import torch

from . import _lib
from ._lib import Weight, check

_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}

lib = torch.library.Library("alloy", "DEF")

lib.define("gguf_q4_k_mm(Tensor activations, Tensor blocks) -> Tensor")
lib.define("batched_gguf_q4_k_mm(Tensor activations, Tensor[] blocks) -> Tensor[]")
lib.define("gguf_q4_k_silu(Tensor activations, Tensor gate_blocks, Tensor up_blocks) -> Tensor")
lib.define("gguf_q4_k_gelu(Tensor activations, Tensor gate_blocks, Tensor up_blocks) -> Tensor")
lib.define("gguf_q4_k_embedding(Tensor input_ids, Tensor blocks) -> Tensor")
lib.define("gguf_q6_k_mm(Tensor activations, Tensor packed_weights) -> Tensor")
lib.define("gguf_q6_k_embedding(Tensor input_ids, Tensor packed_weights) -> Tensor")
lib.define("batched_gguf_q6_k_mm(Tensor activations, Tensor[] packed_weights) -> Tensor[]")
lib.define("gguf_q8_0_embedding(Tensor input_ids, Tensor qweight, Tensor scales) -> Tensor")
lib.define("gguf_q8_0_mm(Tensor activations, Tensor qweight, Tensor scales) -> Tensor")
lib.define("batched_gguf_q8_0_mm(Tensor activations, Tensor[] qweights, Tensor[] scales) -> Tensor[]")
lib.define(
    "gguf_q8_0_silu(Tensor activations, Tensor gate_qweight, Tensor gate_scales, "
    "Tensor up_qweight, Tensor up_scales) -> Tensor"
)
lib.define(
    "attention_cache(Tensor q, Tensor new_k, Tensor new_v, "
    "Tensor cache_pos, Tensor k_cache, Tensor v_cache, float scale, "
    "int sliding_window=0, bool write_kv=True, Tensor? last_real=None) -> Tensor"
)
lib.define(
    "attention_cache_q8(Tensor q, Tensor new_k, Tensor new_v, "
    "Tensor cache_pos, Tensor k_codes, Tensor k_scales, "
    "Tensor v_codes, Tensor v_scales, "
    "float scale=-1.0, int sliding_window=0, bool write_kv=True, "
    "Tensor? last_real=None) -> Tensor"
)
lib.define(
    "attention_kv_update(Tensor q, Tensor new_k, Tensor new_v, "
    "Tensor cache_pos, Tensor k_cache, Tensor v_cache, "
    "float scale=-1.0, int sliding_window=0) -> Tensor"
)
lib.define(
    "attention_kv_update_multi(Tensor q, Tensor new_k, Tensor new_v, "
    "Tensor cache_pos, Tensor k_cache, Tensor v_cache, "
    "float scale=-1.0, int sliding_window=0) -> Tensor"
)
# Q5_0 (three normalised buffers: nibbles, fifth bits, fp16 block scales).
lib.define("gguf_q5_0_mm(Tensor activations, Tensor qweight, Tensor qhigh, Tensor scales) -> Tensor")
lib.define("gguf_q5_0_embedding(Tensor input_ids, Tensor qweight, Tensor qhigh, Tensor scales) -> Tensor")
lib.define(
    "batched_gguf_q5_0_mm(Tensor activations, Tensor[] qweights, "
    "Tensor[] qhighs, Tensor[] scales) -> Tensor[]"
)
lib.define(
    "gguf_moe_routed(Tensor hidden, Tensor router_logits, Tensor gate_up_blocks, "
    "Tensor down_qweight, int num_experts, int top_k, int moe_intermediate) -> Tensor"
)
# New ops (no reference schema).
lib.define(
    "attention_cache_q8_paged(Tensor q, Tensor new_k, Tensor new_v, Tensor seq_pos, "
    "Tensor page_table, Tensor kv_pool, float scale=-1.0, bool write_kv=True) -> Tensor"
)
lib.define(
    "linear_residual(Tensor activations, Tensor weight, Tensor? scales, Tensor residual, "
    "str format) -> Tensor"
)

_FORMATS = {"q4_k": _lib.Q4_K, "q6_k": _lib.Q6_K, "q8_0": _lib.Q8_0}
_BLOCK_BYTES = {_lib.Q4_K: 144, _lib.Q6_K: 210}


_launches = 0


def launch_count() -> int:
    """Number of C-ABI kernel-launching calls made so far (each launches 1-2 kernels)."""
    return _launches


def _stream() -> int:
    global _launches
    _launches += 1
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"activations must be float16, bfloat16 or float32, got {t.dtype}") from None


def _k_of(fmt: int, w: torch.Tensor) -> int:
    if w.ndim != 2:
        raise ValueError(f"packed weight must be rank-2, got {tuple(w.shape)}")
    if fmt == _lib.Q8_0:
        if w.dtype != torch.int8:
            raise TypeError(f"q8_0 qweight requires torch.int8, got {w.dtype}")
        return w.shape[1]
    if w.dtype != torch.uint8:
        raise TypeError(f"packed blocks require torch.uint8, got {w.dtype}")
    bb = _BLOCK_BYTES[fmt]
    if w.shape[1] % bb:
        raise ValueError(f"packed row of {w.shape[1]} bytes is not a whole number of {bb}-byte blocks")
    return w.shape[1] // bb * 256


def _pitched(w: torch.Tensor) -> tuple[torch.Tensor, int]:
    """A packed weight as (tensor, row pitch in bytes; 0 = dense).  Rows may be padded (a column
    shard whose row length is not a multiple of 16 bytes keeps a 16-byte pitch so that the
    tensor-core kernels can copy it); anything else is made contiguous."""
    if w.ndim == 2 and w.stride(1) == 1 and w.stride(0) >= w.shape[1] and w.element_size() == 1:
        return w, (0 if w.stride(0) == w.shape[1] else w.stride(0))
    return w.contiguous(), 0


def _check_acts(x: torch.Tensor, k: int) -> torch.Tensor:
    if x.ndim != 2:
        raise ValueError(f"activations must be (M, K), got {tuple(x.shape)}")
    if x.shape[1] != k:
        raise ValueError(f"activations K={x.shape[1]} does not match the weight's K={k}")
    return x.contiguous()


def _linear(x: torch.Tensor, fmt: int, weights: Sequence[torch.Tensor],
            scales: Sequence[torch.Tensor] | None, residual: torch.Tensor | None = None):
    """One launch for ``len(weights)`` sibling matrices of one format."""
    if len(weights) == 0:
        return []
    k = _k_of(fmt, weights[0])
    x = _check_acts(x, k)
    m = x.shape[0]
    if m == 0:
        return [x.new_empty((0, w.shape[0])) for w in weights]
    outs = []
    descs = (Weight * len(weights))()
    keep = []
    for i, w in enumerate(weights):
        if _k_of(fmt, w) != k:
            raise ValueError("batched matrices must share K")
        w, pitch = _pitched(w)
        y = torch.empty((m, w.shape[0]), dtype=x.dtype, device=x.device)
        s_ptr = None
        if fmt == _lib.Q8_0:
            s = scales[i]
            if s.dtype != torch.float16 or tuple(s.shape) != (w.shape[0], k // 32):
                raise ValueError(f"q8_0 scales must be float16 {(w.shape[0], k // 32)}, "
                                 f"got {s.dtype} {tuple(s.shape)}")
            s = s.contiguous()
            keep.append(s)
            s_ptr = s.data_ptr()
        keep.append(w)
        descs[i] = Weight(fmt, w.shape[0], w.data_ptr(), s_ptr, pitch, y.data_ptr(), 0)
        outs.append(y)
    r_ptr = None
    if residual is not None:
        residual = residual.contiguous()
        if residual.shape != outs[0].shape or residual.dtype != x.dtype:
            raise ValueError("residual must match the output's shape and dtype")
        r_ptr = residual.data_ptr()
    L = _lib.load()
    check(L.alloyb_linear(x.data_ptr(), m, k, _dtype_code(x), descs, len(weights), r_ptr, _stream()),
          "alloyb_linear")
    return outs


def linear_multi(x: torch.Tensor, specs: Sequence[tuple[str, torch.Tensor, torch.Tensor | None]],
                 norm: tuple[torch.Tensor, float] | None = None):
    """Sibling projections of possibly different formats in ONE call.

    ``specs``: (format name, weight, scales-or-None) per matrix, all with the
    same K.  Used for q/k/v where v is Q6_K while q and k are Q4_K.
    ``norm`` = (weight, eps): the projections see RMSNorm(x) (``alloyb_linear_normed``).
    """
    fm0 = _FORMATS[specs[0][0]]
    k = _k_of(fm0, specs[0][1])
    x = _check_acts(x, k)
    m = x.shape[0]
    if m == 0:
        return [x.new_empty((0, w.shape[0])) for _, w, _ in specs]
    descs = (Weight * len(specs))()
    outs = []
    for i, (name, w, s) in enumerate(specs):
        fmt = _FORMATS[name]
        if _k_of(fmt, w) != k:
            raise ValueError("matrices must share K")
        y = torch.empty((m, w.shape[0]), dtype=x.dtype, device=x.device)
        w, pitch = _pitched(w)
        descs[i] = Weight(fmt, w.shape[0], w.data_ptr(), s.data_ptr() if s is not None else None, pitch,
                          y.data_ptr(), 0)
        outs.append(y)
    L = _lib.load()
    if norm is not None:
        nw, eps = norm
        scratch = torch.empty_like(x)
        check(L.alloyb_linear_normed(x.data_ptr(), nw.data_ptr(), float(eps), scratch.data_ptr(), m, k,
                                     _dtype_code(x), descs, len(specs), _stream()), "alloyb_linear_normed")
        return outs
    check(L.alloyb_linear(x.data_ptr(), m, k, _dtype_code(x), descs, len(specs), None, _stream()),
          "alloyb_linear")
    return outs


def linear_allreduce(x: torch.Tensor, fmt_name: str, weight: torch.Tensor, residual: torch.Tensor | None,
                     exchange) -> torch.Tensor | None:
    """Row-parallel linear with the all-reduce inside the launch (``alloyb_linear_allreduce``).

    ``x`` is this rank's K slice of the activations, ``weight`` its K slice of the packed matrix,
    ``exchange`` a ``tp.PeerExchange``.  Returns ``residual + sum over ranks`` or ``None`` when the
    fused kernel does not cover the shape (nothing was launched).
    """
    fmt = _FORMATS[fmt_name]
    k = _k_of(fmt, weight)
    x = _check_acts(x, k)
    m = x.shape[0]
    y = torch.empty((m, weight.shape[0]), dtype=x.dtype, device=x.device)
    weight, pitch = _pitched(weight)
    desc = (Weight * 1)(Weight(fmt, weight.shape[0], weight.data_ptr(), None, pitch, y.data_ptr(), 0))
    L = _lib.load()
    import ctypes as C
    rc = L.alloyb_linear_allreduce(x.data_ptr(), m, k, _dtype_code(x), desc,
                                   residual.data_ptr() if residual is not None else None,
                                   C.byref(exchange.desc), _stream())
    if rc == 1:
        return None
    check(rc, "alloyb_linear_allreduce")
    return y


def gated_normed(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, gate: torch.Tensor, up: torch.Tensor,
                 act: str = "silu") -> torch.Tensor:
    """act(RMSNorm(x) G^T) * (RMSNorm(x) U^T) for Q4_K gate/up (``alloyb_gated_linear_normed``)."""
    k = _k_of(_lib.Q4_K, gate)
    x = _check_acts(x, k)
    y = torch.empty((x.shape[0], gate.shape[0]), dtype=x.dtype, device=x.device)
    if x.shape[0] == 0:
        return y
    scratch = torch.empty_like(x)
    L = _lib.load()
    check(L.alloyb_gated_linear_normed(x.data_ptr(), norm_weight.data_ptr(), float(eps), scratch.data_ptr(),
                                       gate.data_ptr(), None, up.data_ptr(), None, y.data_ptr(), x.shape[0],
                                       gate.shape[0], k, _lib.Q4_K,
                                       _lib.ACT_SILU if act == "silu" else _lib.ACT_GELU_TANH, _dtype_code(x),
                                       _stream()), "alloyb_gated_linear_normed")
    return y


# ------------------------------------------------------------------------------- linear ops


@torch.library.impl(lib, "gguf_q4_k_mm", "CUDA")
def _q4k_mm(activations, blocks):
    return _linear(activations, _lib.Q4_K, [blocks], None)[0]


@torch.library.impl(lib, "gguf_q6_k_mm", "CUDA")
def _q6k_mm(activations, packed_weights):
    return _linear(activations, _lib.Q6_K, [packed_weights], None)[0]


@torch.library.impl(lib, "gguf_q8_0_mm", "CUDA")
def _q8_mm(activations, qweight, scales):
    return _linear(activations, _lib.Q8_0, [qweight], [scales])[0]


@torch.library.impl(lib, "batched_gguf_q4_k_mm", "CUDA")
def _bq4k_mm(activations, blocks):
    return _batched(activations, _lib.Q4_K, blocks, None)


@torch.library.impl(lib, "batched_gguf_q6_k_mm", "CUDA")
def _bq6k_mm(activations, packed_weights):
    return _batched(activations, _lib.Q6_K, packed_weights, None)


@torch.library.impl(lib, "batched_gguf_q8_0_mm", "CUDA")
def _bq8_mm(activations, qweights, scales):
    return _batched(activations, _lib.Q8_0, qweights, scales)


def _batched(x, fmt, ws, ss, group: int = 4):
    out = []
    for i in range(0, len(ws), group):
        out += _linear(x, fmt, ws[i:i + group], ss[i:i + group] if ss is not None else None)
    return out


@torch.library.impl(lib, "linear_residual", "CUDA")
def _linear_residual(activations, weight, scales, residual, format):
    fmt = _FORMATS[format]
    return _linear(activations, fmt, [weight], [scales] if scales is not None else None, residual)[0]


def _gated(x, gate, gs, up, us, fmt, act):
    k = _k_of(fmt, gate)
    if _k_of(fmt, up) != k or gate.shape[0] != up.shape[0]:
        raise ValueError("gate and up must have the same shape")
    x = _check_acts(x, k)
    gate, up = gate.contiguous(), up.contiguous()
    y = torch.empty((x.shape[0], gate.shape[0]), dtype=x.dtype, device=x.device)
    if x.shape[0] == 0:
        return y
    if x.shape[0] > 128 and fmt == _lib.Q4_K and act == _lib.ACT_SILU and x.dtype != torch.float32:
        # prefill: two single GEMMs + silu_mul, the split the reference measured faster than its
        # fused dual-accumulator kernel (packages/alloy-torch/src/alloy_torch/ops/linalg.py:774-780);
        # up to 128 tokens the tensor-core GEMM keeps both accumulators in tensor memory
        g, u = _linear(x, fmt, [gate], None)[0], _linear(x, fmt, [up], None)[0]
        return silu_mul(g, u)
    L = _lib.load()
    check(L.alloyb_gated_linear(x.data_ptr(), gate.data_ptr(), gs.data_ptr() if gs is not None else None,
                                up.data_ptr(), us.data_ptr() if us is not None else None,
                                y.data_ptr(), x.shape[0], gate.shape[0], k, fmt, act,
                                _dtype_code(x), _stream()), "alloyb_gated_linear")
    return y


@torch.library.impl(lib, "gguf_q4_k_silu", "CUDA")
def _q4k_silu(activations, gate_blocks, up_blocks):
    return _gated(activations, gate_blocks, None, up_blocks, None, _lib.Q4_K, _lib.ACT_SILU)


@torch.library.impl(lib, "gguf_q4_k_gelu", "CUDA")
def _q4k_gelu(activations, gate_blocks, up_blocks):
    return _gated(activations, gate_blocks, None, up_blocks, None, _lib.Q4_K, _lib.ACT_GELU_TANH)


@torch.library.impl(lib, "gguf_q8_0_silu", "CUDA")
def _q8_silu(activations, gate_qweight, gate_scales, up_qweight, up_scales):
    return _gated(activations, gate_qweight, gate_scales.contiguous(), up_qweight,
                  up_scales.contiguous(), _lib.Q8_0, _lib.ACT_SILU)


# ------------------------------------------------------------------------------- Q5_0, routed experts


def _q5_check(qweight, qhigh, scales):
    if qweight.dtype != torch.uint8 or qhigh.dtype != torch.uint8 or scales.dtype != torch.float16:
        raise TypeError("q5_0 buffers are uint8 qweight, uint8 qhigh and float16 scales")
    n, half = qweight.shape
    if tuple(qhigh.shape) != (n, half) or tuple(scales.shape) != (n, half // 16) or half % 16:
        raise ValueError(f"q5_0 buffers must be (N, K/2), (N, K/2), (N, K/32); got {tuple(qweight.shape)}, "
                         f"{tuple(qhigh.shape)}, {tuple(scales.shape)}")
    return n, half * 2


@torch.library.impl(lib, "gguf_q5_0_mm", "CUDA")
def _q5_mm(activations, qweight, qhigh, scales):
    n, k = _q5_check(qweight, qhigh, scales)
    x = _check_acts(activations, k)
    y = torch.empty((x.shape[0], n), dtype=x.dtype, device=x.device)
    if x.shape[0] == 0:
        return y
    qweight, qhigh, scales = qweight.contiguous(), qhigh.contiguous(), scales.contiguous()
    check(_lib.load().alloyb_q5_0_mm(x.data_ptr(), qweight.data_ptr(), qhigh.data_ptr(), scales.data_ptr(),
                                     y.data_ptr(), x.shape[0], n, k, _dtype_code(x), _stream()), "alloyb_q5_0_mm")
    return y


@torch.library.impl(lib, "batched_gguf_q5_0_mm", "CUDA")
def _bq5_mm(activations, qweights, qhighs, scales):
    return [_q5_mm(activations, w, h, s) for w, h, s in zip(qweights, qhighs, scales)]


@torch.library.impl(lib, "gguf_q5_0_embedding", "CUDA")
def _q5_emb(input_ids, qweight, qhigh, scales):
    n, k = _q5_check(qweight, qhigh, scales)
    flat = input_ids.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty((flat.numel(), k), dtype=torch.float32, device=qweight.device)
    if flat.numel():
        qweight, qhigh, scales = qweight.contiguous(), qhigh.contiguous(), scales.contiguous()
        check(_lib.load().alloyb_dequant_q5_0(qweight.data_ptr(), qhigh.data_ptr(), scales.data_ptr(),
                                              flat.data_ptr(), out.data_ptr(), flat.numel(), n, k, _lib.F32,
                                              _stream()), "alloyb_dequant_q5_0")
    return out.reshape(tuple(input_ids.shape) + (k,))


@torch.library.impl(lib, "gguf_moe_routed", "CUDA")
def _moe_routed(hidden, router_logits, gate_up_blocks, down_qweight, num_experts, top_k, moe_intermediate):
    if hidden.ndim != 2 or router_logits.ndim != 2 or router_logits.shape != (hidden.shape[0], num_experts):
        raise ValueError("hidden must be (T, H) and router_logits (T, num_experts)")
    t, hdim = hidden.shape
    i = int(moe_intermediate)
    if hdim % 256 or i % 256:
        raise ValueError("hidden size and moe_intermediate must be multiples of 256")
    if gate_up_blocks.dtype != torch.uint8 or down_qweight.dtype != torch.uint8:
        raise TypeError("expert weights are packed uint8 blocks")
    if gate_up_blocks.numel() != num_experts * 2 * i * (hdim // 256) * 144:
        raise ValueError("gate_up_blocks must hold (E, 2*I, H/256*144) Q4_K bytes")
    if down_qweight.numel() != num_experts * hdim * (i // 256) * 210:
        raise ValueError("down_qweight must hold (E, H, I/256*210) Q6_K bytes")
    hidden = hidden.contiguous()
    logits = router_logits.to(torch.float32).contiguous()
    out = torch.empty((t, hdim), dtype=torch.float32, device=hidden.device)
    if t == 0:
        return out
    L = _lib.load()
    n = L.alloyb_moe_workspace_bytes(t, int(top_k), i)
    ws = torch.empty(n, dtype=torch.uint8, device=hidden.device)
    check(L.alloyb_moe_routed(hidden.data_ptr(), _dtype_code(hidden), logits.data_ptr(),
                              gate_up_blocks.contiguous().data_ptr(), down_qweight.contiguous().data_ptr(),
                              out.data_ptr(), t, hdim, int(num_experts), int(top_k), i, ws.data_ptr(), n, _stream()),
          "alloyb_moe_routed")
    return out


# ------------------------------------------------------------------------------- embeddings


def _embedding(ids: torch.Tensor, fmt: int, w: torch.Tensor, scales: torch.Tensor | None,
               out_dtype: torch.dtype = torch.float32, out: torch.Tensor | None = None) -> torch.Tensor:
    k = _k_of(fmt, w)
    w = w.contiguous()
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    if out is None:
        out = torch.empty((flat.numel(), k), dtype=out_dtype, device=w.device)
    elif out.numel() != flat.numel() * k or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor of ids.numel() * K elements")
    else:
        out_dtype = out.dtype
    if flat.numel() == 0:
        return out.reshape(tuple(ids.shape) + (k,))
    L = _lib.load()
    if fmt == _lib.Q4_K:
        rc = L.alloyb_dequant_q4k(w.data_ptr(), flat.data_ptr(), out.data_ptr(), flat.numel(),
                                  w.shape[0], k, _DTYPES[out_dtype], _stream())
    elif fmt == _lib.Q6_K:
        rc = L.alloyb_dequant_q6k(w.data_ptr(), flat.data_ptr(), out.data_ptr(), flat.numel(),
                                  w.shape[0], k, _DTYPES[out_dtype], _stream())
    else:
        scales = scales.contiguous()
        rc = L.alloyb_dequant_q8_0(w.data_ptr(), scales.data_ptr(), flat.data_ptr(), out.data_ptr(),
                                   flat.numel(), w.shape[0], k, _DTYPES[out_dtype], _stream())
    check(rc, "alloyb_dequant")
    return out.reshape(tuple(ids.shape) + (k,))


@torch.library.impl(lib, "gguf_q4_k_embedding", "CUDA")
def _q4k_emb(input_ids, blocks):
    return _embedding(input_ids, _lib.Q4_K, blocks, None)


@torch.library.impl(lib, "gguf_q6_k_embedding", "CUDA")
def _q6k_emb(input_ids, packed_weights):
    return _embedding(input_ids, _lib.Q6_K, packed_weights, None)


@torch.library.impl(lib, "gguf_q8_0_embedding", "CUDA")
def _q8_emb(input_ids, qweight, scales):
    return _embedding(input_ids, _lib.Q8_0, qweight, scales)


def dequantize(fmt: str, w: torch.Tensor, scales: torch.Tensor | None = None,
               out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Decode a whole packed matrix on the device (test hook; bit-exact fp32)."""
    code = _FORMATS[fmt]
    k = _k_of(code, w)
    w = w.contiguous()
    out = torch.empty((w.shape[0], k), dtype=out_dtype, device=w.device)
    L = _lib.load()
    if code == _lib.Q4_K:
        rc = L.alloyb_dequant_q4k(w.data_ptr(), None, out.data_ptr(), w.shape[0], w.shape[0], k,
                                  _DTYPES[out_dtype], _stream())
    elif code == _lib.Q6_K:
        rc = L.alloyb_dequant_q6k(w.data_ptr(), None, out.data_ptr(), w.shape[0], w.shape[0], k,
                                  _DTYPES[out_dtype], _stream())
    else:
        scales = scales.contiguous()
        rc = L.alloyb_dequant_q8_0(w.data_ptr(), scales.data_ptr(), None, out.data_ptr(), w.shape[0],
                                   w.shape[0], k, _DTYPES[out_dtype], _stream())
    check(rc, "alloyb_dequant")
    return out


# ------------------------------------------------------------------------------- attention

_workspaces: dict[tuple[int, int, int, int], torch.Tensor] = {}


def attn_workspace(device: torch.device, b: int, h: int, d: int) -> torch.Tensor:
    """Cached, initialised split-K workspace for (device, B, H, D).

    One workspace serves every call of that shape on the device; calls that
    may overlap on the GPU (different streams) need workspaces of their own
    (``new_attn_workspace``).
    """
    key = (device.index if device.index is not None else torch.cuda.current_device(), b, h, d)
    ws = _workspaces.get(key)
    if ws is None:
        ws = new_attn_workspace(device, b, h, d)
        _workspaces[key] = ws
    return ws


def new_attn_workspace(device: torch.device, b: int, h: int, d: int) -> torch.Tensor:
    L = _lib.load()
    n = L.alloyb_attn_workspace_bytes(b, h, d)
    ws = torch.empty(n, dtype=torch.uint8, device=device)
    check(L.alloyb_attn_workspace_init(ws.data_ptr(), n, b, h, _stream()), "alloyb_attn_workspace_init")
    return ws


def attn_status(ws: torch.Tensor) -> int:
    """Device status word of a workspace (0 = every position/page was in range)."""
    L = _lib.load()
    out = C.c_int32(0)
    check(L.alloyb_attn_workspace_status(ws.data_ptr(), C.byref(out), _stream()),
          "alloyb_attn_workspace_status")
    return int(out.value)


def _pos_i32(pos: torch.Tensor) -> torch.Tensor:
    if pos.dtype != torch.int32:
        pos = pos.to(torch.int32)
    return pos.contiguous()


def _check_cache(layout, b, kv_h, d, k0, k1, v0, v1):
    """Cache tensors against (B, KV_H, D): a mismatch would make the kernels index out of bounds."""
    if layout == _lib.KV_Q8_PAGED:
        pool, table = k0, k1
        if pool.shape[1] != 2 or pool.shape[2] != kv_h or pool.shape[3] != 16 or pool.shape[4] != d // 32 * 34:
            raise ValueError(f"kv_pool must be (pages, 2, {kv_h}, 16, {d // 32 * 34}), got {tuple(pool.shape)}")
        if table.shape[0] < b:
            raise ValueError(f"page_table has {table.shape[0]} rows for batch {b}")
        return
    for name, t in (("k cache", k0), ("v cache", v0)):
        if t.ndim != 4 or t.shape[0] < b or t.shape[1] != kv_h or t.shape[3] != d:
            raise ValueError(f"{name} must be (>= {b}, {kv_h}, S, {d}), got {tuple(t.shape)}")
    if k0.shape != v0.shape:
        raise ValueError("K and V caches must have the same shape")
    if layout == _lib.KV_Q8_SPLIT:
        want = (k0.shape[0], kv_h, k0.shape[2], d // 32)
        for name, t in (("k scales", k1), ("v scales", v1)):
            if tuple(t.shape) != want:
                raise ValueError(f"{name} must be {want}, got {tuple(t.shape)}")


def _cache_attention(layout, q, new_k, new_v, pos, k0, k1, v0, v1, s_max, num_pages, scale,
                     write_kv, workspace=None):
    """Shared body of the cache-attention ops: one query token per sequence runs the split-K decode
    kernels, a chunk of several (prefill, verify) the causal chunk kernel after the chunk's K/V rows
    have been written to the cache (quantised for the q8 layouts) -- the routing of the reference's
    ``_attention_cache_handler`` / ``_attention_cache_q8_handler``
    (packages/alloy-torch/src/alloy_torch/ops/attention.py:886-934, ops/kv_quant.py:58-162)."""
    if q.ndim != 4:
        raise ValueError(f"attention expects 4D Q (B, H, S, D), got {q.ndim}D")
    b, h, s, d = q.shape
    if d % 32 != 0:
        raise ValueError(f"attention needs head_dim % 32 == 0, got {d}")
    if new_k.ndim != 4 or new_v.ndim != 4:
        raise ValueError("new_k / new_v must be 4D (B, KV_H, S, D)")
    kv_h = new_k.shape[1]
    if kv_h <= 0 or h % kv_h:
        raise ValueError(f"{h} query heads do not group over {kv_h} KV heads")
    _check_cache(layout, b, kv_h, d, k0, k1, v0, v1)
    if q.stride(3) != 1:
        q = q.contiguous()
    for name, t in (("new_k", new_k), ("new_v", new_v)):
        if t.dtype != torch.float16:
            raise TypeError(f"{name} must be float16, got {t.dtype}")
        if tuple(t.shape) != (b, kv_h, s, d):
            raise ValueError(f"{name} must be {(b, kv_h, s, d)}, got {tuple(t.shape)}")
    if new_k.stride(3) != 1 or new_v.stride(3) != 1 or new_k.stride() != new_v.stride():
        new_k, new_v = new_k.contiguous(), new_v.contiguous()
    out = torch.empty((b, s, h, d), dtype=q.dtype, device=q.device)
    ws = workspace if workspace is not None else attn_workspace(q.device, b, h, d)
    L = _lib.load()
    ptrs = [t.data_ptr() if t is not None else None for t in (k0, k1, v0, v1)]
    sc = float(scale) if scale is not None else -1.0
    if s == 1:
        check(L.alloyb_attn_decode(
            layout, q.data_ptr(), q.stride(0), q.stride(1), _dtype_code(q), *ptrs,
            new_k.data_ptr(), new_v.data_ptr(), new_k.stride(0), new_k.stride(1),
            pos.data_ptr(), pos.numel(), out.data_ptr(), b, h, kv_h, d, s_max, num_pages,
            sc, 1 if write_kv else 0, ws.data_ptr(), ws.numel(), _stream()), "alloyb_attn_decode")
        return out.transpose(1, 2)
    if d not in (64, 128, 256):
        raise NotImplementedError(f"chunk attention is built for head_dim 64, 128 and 256, got {d}")
    if write_kv:
        check(L.alloyb_kv_write(layout, new_k.data_ptr(), new_v.data_ptr(), new_k.stride(0), new_k.stride(1),
                                new_k.stride(2), *ptrs, pos.data_ptr(), pos.numel(), b, kv_h, d, s_max, num_pages,
                                s, ws.data_ptr(), _stream()), "alloyb_kv_write")
    check(L.alloyb_attn_chunk(layout, q.data_ptr(), q.stride(0), q.stride(1), q.stride(2), _dtype_code(q), *ptrs,
                              pos.data_ptr(), pos.numel(), out.data_ptr(), b, h, kv_h, d, s, s_max, num_pages, sc,
                              ws.data_ptr(), _stream()), "alloyb_attn_chunk")
    return out.transpose(1, 2)


def _norm_scale(scale, d):
    default = 1.0 / math.sqrt(d)
    if scale is None or scale <= 0 or math.isclose(float(scale), default, rel_tol=1e-6, abs_tol=1e-6):
        return -1.0
    return float(scale)


def _no_window(sliding_window, last_real):
    if sliding_window:
        raise NotImplementedError("sliding-window ring caches are outside this build's scope")
    if last_real is not None:
        # the bound the reference applies to padded chunks of a ring cache
        # (packages/alloy-torch/src/alloy_torch/ops/kv_quant.py:70, :110): not computed here, so refuse it
        raise NotImplementedError("last_real (the padded-chunk bound of sliding-window caches) is outside "
                                  "this build's scope")


@torch.library.impl(lib, "attention_cache", "CUDA")
def _attention_cache(q, new_k, new_v, cache_pos, k_cache, v_cache, scale, sliding_window=0,
                     write_kv=True, last_real=None):
    _no_window(sliding_window, last_real)
    if k_cache.dtype != torch.float16 or v_cache.dtype != torch.float16:
        raise TypeError("attention_cache expects float16 K/V caches")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("K/V caches must be contiguous (B, KV_H, S, D)")
    pos = _pos_i32(cache_pos.reshape(-1)[:1])
    return _cache_attention(_lib.KV_F16, q, new_k, new_v, pos, k_cache, None, v_cache, None,
                             k_cache.shape[2], 0, _norm_scale(scale, q.shape[-1]), write_kv)


@torch.library.impl(lib, "attention_kv_update", "CUDA")
def _attention_kv_update(q, new_k, new_v, cache_pos, k_cache, v_cache, scale=-1.0, sliding_window=0):
    return _attention_cache(q, new_k, new_v, cache_pos, k_cache, v_cache, scale, sliding_window, True, None)


@torch.library.impl(lib, "attention_kv_update_multi", "CUDA")
def _attention_kv_update_multi(q, new_k, new_v, cache_pos, k_cache, v_cache, scale=-1.0, sliding_window=0):
    """Speculative-decode verify: 2..16 new tokens written at cache_pos.., each attending causally
    (packages/alloy-torch/src/alloy_torch/ops/attention.py:1255-1275)."""
    return _attention_cache(q, new_k, new_v, cache_pos, k_cache, v_cache, scale, sliding_window, True, None)


@torch.library.impl(lib, "attention_cache_q8", "CUDA")
def _attention_cache_q8(q, new_k, new_v, cache_pos, k_codes, k_scales, v_codes, v_scales,
                        scale=-1.0, sliding_window=0, write_kv=True, last_real=None):
    _no_window(sliding_window, last_real)
    for t, dt in ((k_codes, torch.int8), (v_codes, torch.int8), (k_scales, torch.float16),
                  (v_scales, torch.float16)):
        if t.dtype != dt or not t.is_contiguous():
            raise TypeError("q8 cache tensors must be contiguous int8 codes / float16 scales")
    pos = _pos_i32(cache_pos.reshape(-1)[:1])
    return _cache_attention(_lib.KV_Q8_SPLIT, q, new_k, new_v, pos, k_codes, k_scales, v_codes,
                             v_scales, k_codes.shape[2], 0, _norm_scale(scale, q.shape[-1]), write_kv)


@torch.library.impl(lib, "attention_cache_q8_paged", "CUDA")
def _attention_cache_q8_paged(q, new_k, new_v, seq_pos, page_table, kv_pool, scale=-1.0,
                              write_kv=True):
    if kv_pool.dtype != torch.uint8 or not kv_pool.is_contiguous() or kv_pool.ndim != 5:
        raise TypeError("kv_pool must be contiguous uint8 (pages, 2, KV_H, 16, D/32*34)")
    if page_table.dtype != torch.int32 or not page_table.is_contiguous() or page_table.ndim != 2:
        raise TypeError("page_table must be contiguous int32 (B, max_pages)")
    if page_table.shape[0] != q.shape[0]:
        raise ValueError("page_table needs one row per sequence")
    pos = _pos_i32(seq_pos.reshape(-1))
    return _cache_attention(_lib.KV_Q8_PAGED, q, new_k, new_v, pos, kv_pool, page_table, None, None,
                             page_table.shape[1] * 16, kv_pool.shape[0],
                             _norm_scale(scale, q.shape[-1]), write_kv)


# ------------------------------------------------------------------------------- Meta kernels
# Same shape functions as the reference's Meta registrations
# (packages/alloy-torch/src/alloy_torch/custom_ops.py:285-300, :666-673, :750-785).


def _mm_meta(x, w):
    return torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)


torch.library.impl(lib, "gguf_q4_k_mm", "Meta")(lambda activations, blocks: _mm_meta(activations, blocks))
torch.library.impl(lib, "gguf_q6_k_mm", "Meta")(
    lambda activations, packed_weights: _mm_meta(activations, packed_weights))
torch.library.impl(lib, "gguf_q8_0_mm", "Meta")(
    lambda activations, qweight, scales: _mm_meta(activations, qweight))
torch.library.impl(lib, "batched_gguf_q4_k_mm", "Meta")(
    lambda activations, blocks: [_mm_meta(activations, w) for w in blocks])
torch.library.impl(lib, "batched_gguf_q6_k_mm", "Meta")(
    lambda activations, packed_weights: [_mm_meta(activations, w) for w in packed_weights])
torch.library.impl(lib, "batched_gguf_q8_0_mm", "Meta")(
    lambda activations, qweights, scales: [_mm_meta(activations, w) for w in qweights])
torch.library.impl(lib, "gguf_q4_k_silu", "Meta")(
    lambda activations, gate_blocks, up_blocks: _mm_meta(activations, gate_blocks))
torch.library.impl(lib, "gguf_q4_k_gelu", "Meta")(
    lambda activations, gate_blocks, up_blocks: _mm_meta(activations, gate_blocks))
torch.library.impl(lib, "gguf_q8_0_silu", "Meta")(
    lambda activations, gate_qweight, gate_scales, up_qweight, up_scales:
    _mm_meta(activations, gate_qweight))
torch.library.impl(lib, "linear_residual", "Meta")(
    lambda activations, weight, scales, residual, format: torch.empty_like(residual))
torch.library.impl(lib, "gguf_q4_k_embedding", "Meta")(
    lambda input_ids, blocks: torch.empty(input_ids.shape + ((blocks.shape[1] // 144) * 256,),
                                          dtype=torch.float32, device=input_ids.device))
torch.library.impl(lib, "gguf_q6_k_embedding", "Meta")(
    lambda input_ids, packed_weights: torch.empty(
        input_ids.shape + ((packed_weights.shape[1] // 210) * 256,), dtype=torch.float32,
        device=input_ids.device))
torch.library.impl(lib, "gguf_q8_0_embedding", "Meta")(
    lambda input_ids, qweight, scales: torch.empty(input_ids.shape + (qweight.shape[1],),
                                                   dtype=torch.float32, device=input_ids.device))
torch.library.impl(lib, "gguf_q5_0_mm", "Meta")(
    lambda activations, qweight, qhigh, scales:
    torch.empty((activations.shape[0], scales.shape[0]), dtype=activations.dtype, device=activations.device))
torch.library.impl(lib, "batched_gguf_q5_0_mm", "Meta")(
    lambda activations, qweights, qhighs, scales:
    [torch.empty((activations.shape[0], s.shape[0]), dtype=activations.dtype, device=activations.device)
     for s in scales])
torch.library.impl(lib, "gguf_q5_0_embedding", "Meta")(
    lambda input_ids, qweight, qhigh, scales: torch.empty(input_ids.shape + (qweight.shape[1] * 2,),
                                                          dtype=torch.float32, device=input_ids.device))
torch.library.impl(lib, "gguf_moe_routed", "Meta")(
    lambda hidden, router_logits, gate_up_blocks, down_qweight, num_experts, top_k, moe_intermediate:
    torch.empty((hidden.shape[0], hidden.shape[1]), dtype=torch.float32, device=hidden.device))
torch.library.impl(lib, "attention_kv_update", "Meta")(
    lambda q, new_k, new_v, cache_pos, k_cache, v_cache, scale=-1.0, sliding_window=0: torch.empty_like(q))
torch.library.impl(lib, "attention_kv_update_multi", "Meta")(
    lambda q, new_k, new_v, cache_pos, k_cache, v_cache, scale=-1.0, sliding_window=0: torch.empty_like(q))
torch.library.impl(lib, "attention_cache", "Meta")(
    lambda q, new_k, new_v, cache_pos, k_cache, v_cache, scale, sliding_window=0, write_kv=True,
    last_real=None: torch.empty_like(q))
torch.library.impl(lib, "attention_cache_q8", "Meta")(
    lambda q, new_k, new_v, cache_pos, k_codes, k_scales, v_codes, v_scales, scale=-1.0,
    sliding_window=0, write_kv=True, last_real=None: torch.empty_like(q))
torch.library.impl(lib, "attention_cache_q8_paged", "Meta")(
    lambda q, new_k, new_v, seq_pos, page_table, kv_pool, scale=-1.0, write_kv=True:
    torch.empty_like(q))


# ------------------------------------------------------------------------------- glue


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    y = torch.empty_like(x2)
    L = _lib.load()
    check(L.alloyb_rms_norm(x2.data_ptr(), weight.data_ptr(), y.data_ptr(), x2.shape[0], x2.shape[1],
                            float(eps), _dtype_code(x2), _stream()), "alloyb_rms_norm")
    return y.reshape(x.shape)


def rope_inplace(q: torch.Tensor, k: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor) -> None:
    """Rotate-half RoPE on contiguous q (B,H,D) and k (B,KV_H,D) at pos (int32 (1,) or (B,))."""
    b, h, d = q.shape
    L = _lib.load()
    check(L.alloyb_rope_inplace(q.data_ptr(), k.data_ptr(), pos.data_ptr(), pos.numel(),
                                inv_freq.data_ptr(), b, h, k.shape[1], d, _dtype_code(q), _stream()),
          "alloyb_rope_inplace")


def rope_kv_append(q: torch.Tensor, new_k: torch.Tensor, new_v: torch.Tensor, pos: torch.Tensor,
                   inv_freq: torch.Tensor, *, k_cache: torch.Tensor | None = None, v_cache: torch.Tensor | None = None,
                   q8_split: tuple | None = None, paged: tuple | None = None) -> None:
    """Rotate-half RoPE of the decode token's q (contiguous fp16 (B, H, D), in place) and k, and the
    append of the rotated k and of v at ``pos`` to ONE cache, in one launch
    (``alloyb_rope_kv_append``); run the attention op with ``write_kv=False`` afterwards.

    The cache is ``k_cache``/``v_cache`` (fp16 (B, KV_H, S, D)), ``q8_split`` = (k_codes, k_scales,
    v_codes, v_scales), or ``paged`` = (page_table, kv_pool).  new_k/new_v: fp16 (B, KV_H, D).
    """
    b, h, d = q.shape
    kv_h = new_k.shape[1]
    if q.dtype != torch.float16 or not q.is_contiguous():
        raise ValueError("q must be contiguous float16 (B, H, D)")
    for name, t in (("new_k", new_k), ("new_v", new_v)):
        if t.dtype != torch.float16 or tuple(t.shape) != (b, kv_h, d) or t.stride(2) != 1:
            raise ValueError(f"{name} must be float16 {(b, kv_h, d)} with unit inner stride")
    if new_k.stride() != new_v.stride():
        new_k, new_v = new_k.contiguous(), new_v.contiguous()
    pos = _pos_i32(pos.reshape(-1))
    if k_cache is not None:
        layout, ptrs, s_max, n_pages = _lib.KV_F16, (k_cache, None, v_cache, None), k_cache.shape[2], 0
    elif q8_split is not None:
        layout, ptrs, s_max, n_pages = _lib.KV_Q8_SPLIT, tuple(q8_split), q8_split[0].shape[2], 0
    elif paged is not None:
        table, pool = paged
        layout, ptrs, s_max, n_pages = _lib.KV_Q8_PAGED, (pool, table, None, None), table.shape[1] * 16, pool.shape[0]
    else:
        raise ValueError("one cache must be given")
    _check_cache(layout, b, kv_h, d, *ptrs)
    ws = attn_workspace(q.device, b, h, d)
    L = _lib.load()
    check(L.alloyb_rope_kv_append(layout, q.data_ptr(), new_k.data_ptr(), new_v.data_ptr(), new_k.stride(0),
                                  new_k.stride(1), *[t.data_ptr() if t is not None else None for t in ptrs],
                                  pos.data_ptr(), pos.numel(), inv_freq.data_ptr(), b, h, kv_h, d, s_max, n_pages,
                                  ws.data_ptr(), _stream()), "alloyb_rope_kv_append")


def rope_attention_decode(q: torch.Tensor, new_k: torch.Tensor, new_v: torch.Tensor, pos: torch.Tensor,
                          inv_freq: torch.Tensor, *, k_cache: torch.Tensor | None = None,
                          v_cache: torch.Tensor | None = None, q8_split: tuple | None = None,
                          paged: tuple | None = None, scale: float | None = None) -> torch.Tensor:
    """The decode token's attention step in ONE launch (``alloyb_attn_decode_rope``): RoPE of q and k, the
    append of k / v at ``pos`` to the cache, attention over the cache.  Arguments as ``rope_kv_append``
    (q fp16 (B, H, D), left unrotated); returns (B, H, D).  Same numbers, bit for bit, as
    ``rope_kv_append`` followed by the cache-attention op with ``write_kv=False``; shapes the fused
    kernel does not cover take exactly that route."""
    b, h, d = q.shape
    kv_h = new_k.shape[1]
    if q.dtype != torch.float16 or q.stride(2) != 1:
        raise ValueError("q must be float16 (B, H, D) with unit inner stride")
    for name, t in (("new_k", new_k), ("new_v", new_v)):
        if t.dtype != torch.float16 or tuple(t.shape) != (b, kv_h, d) or t.stride(2) != 1:
            raise ValueError(f"{name} must be float16 {(b, kv_h, d)} with unit inner stride")
    if new_k.stride() != new_v.stride():
        new_k, new_v = new_k.contiguous(), new_v.contiguous()
    pos = _pos_i32(pos.reshape(-1))
    if k_cache is not None:
        layout, ptrs, s_max, n_pages = _lib.KV_F16, (k_cache, None, v_cache, None), k_cache.shape[2], 0
    elif q8_split is not None:
        layout, ptrs, s_max, n_pages = _lib.KV_Q8_SPLIT, tuple(q8_split), q8_split[0].shape[2], 0
    elif paged is not None:
        table, pool = paged
        layout, ptrs, s_max, n_pages = _lib.KV_Q8_PAGED, (pool, table, None, None), table.shape[1] * 16, pool.shape[0]
    else:
        raise ValueError("one cache must be given")
    _check_cache(layout, b, kv_h, d, *ptrs)
    ws = attn_workspace(q.device, b, h, d)
    out = torch.empty((b, h, d), dtype=q.dtype, device=q.device)
    L = _lib.load()
    rc = L.alloyb_attn_decode_rope(layout, q.data_ptr(), q.stride(0), q.stride(1),
                                   *[t.data_ptr() if t is not None else None for t in ptrs],
                                   new_k.data_ptr(), new_v.data_ptr(), new_k.stride(0), new_k.stride(1),
                                   pos.data_ptr(), pos.numel(), inv_freq.data_ptr(), out.data_ptr(), b, h, kv_h, d,
                                   s_max, n_pages, float(scale) if scale is not None else -1.0, ws.data_ptr(),
                                   ws.numel(), _stream())
    if rc == 1:          # not a shape of the fused kernel: the two launches it stands for
        q = q.contiguous()
        rope_kv_append(q, new_k, new_v, pos, inv_freq, k_cache=k_cache, v_cache=v_cache, q8_split=q8_split, paged=paged)
        k0, k1, v0, v1 = ptrs
        return _cache_attention(layout, q.unsqueeze(2), new_k.unsqueeze(2), new_v.unsqueeze(2), pos, k0, k1, v0, v1,
                                s_max, n_pages, scale, False).squeeze(2)
    check(rc, "alloyb_attn_decode_rope")
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    y = torch.empty_like(gate)
    L = _lib.load()
    check(L.alloyb_silu_mul(gate.data_ptr(), up.data_ptr(), y.data_ptr(), gate.numel(),
                            _dtype_code(gate), _stream()), "alloyb_silu_mul")
    return y


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    m, n = logits.shape
    if out is None:
        out = torch.empty((m,), dtype=torch.int64, device=logits.device)
    elif out.shape != (m,) or out.dtype != torch.int64 or not out.is_contiguous() or out.device != logits.device:
        raise ValueError(f"out must be a contiguous int64 tensor of shape ({m},) on {logits.device}")
    L = _lib.load()
    check(L.alloyb_argmax(logits.data_ptr(), out.data_ptr(), m, n, _dtype_code(logits), _stream()),
          "alloyb_argmax")
    return out

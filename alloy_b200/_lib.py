"""ctypes binding of ``liballoy_b200.so`` — the only route from Python to the kernels.

There is no fallback: if the shared library has not been built
(``python -m alloy_b200.build``) loading raises, and every op raises with it.
"""

from __future__ import annotations

import ctypes as C
import pathlib

_HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = _HERE / "liballoy_b200.so"

F16, BF16, F32 = 0, 1, 2
Q4_K, Q6_K, Q8_0 = 0, 1, 2
ACT_SILU, ACT_GELU_TANH = 0, 1
KV_F16, KV_Q8_SPLIT, KV_Q8_PAGED = 0, 1, 2


class AlloyB200Error(RuntimeError):
    """A C-ABI call returned a negative status."""


class Weight(C.Structure):
    """Mirror of ``alloyb_weight`` in ``include/alloy_b200.h``."""

    _fields_ = [
        ("format", C.c_int),
        ("N", C.c_int),
        ("data", C.c_void_p),
        ("scales", C.c_void_p),
        ("row_bytes", C.c_int64),
        ("y", C.c_void_p),
        ("ldy", C.c_int64),
    ]


class TP(C.Structure):
    """Mirror of ``alloyb_tp`` in ``include/alloy_b200.h``."""

    _fields_ = [
        ("world", C.c_int),
        ("rank", C.c_int),
        ("max_n", C.c_int),
        ("spin_limit", C.c_int),
        ("peer", C.c_void_p * 8),
    ]


class Matrix(C.Structure):
    """Mirror of ``alloyb_matrix``."""

    _fields_ = [("format", C.c_int), ("N", C.c_int), ("data", C.c_void_p), ("row_bytes", C.c_int64)]


class DecoderLayer(C.Structure):
    """Mirror of ``alloyb_decoder_layer``."""

    _fields_ = [("wq", Matrix), ("wk", Matrix), ("wv", Matrix), ("wo", Matrix), ("wg", Matrix), ("wu", Matrix),
                ("wd", Matrix), ("norm_in", C.c_void_p), ("norm_post", C.c_void_p), ("k0", C.c_void_p),
                ("k1", C.c_void_p), ("v0", C.c_void_p), ("v1", C.c_void_p)]


class DecoderDesc(C.Structure):
    """Mirror of ``alloyb_decoder_desc``."""

    _fields_ = [("n_layers", C.c_int), ("hidden", C.c_int), ("ffn", C.c_int), ("heads", C.c_int),
                ("kv_heads", C.c_int), ("head_dim", C.c_int), ("eps", C.c_float), ("kv_layout", C.c_int),
                ("S_max", C.c_int), ("num_pages", C.c_int64), ("layers", C.POINTER(DecoderLayer)),
                ("norm_final", C.c_void_p), ("head", Matrix), ("inv_freq", C.c_void_p), ("pos", C.c_void_p),
                ("hidden_io", C.c_void_p), ("logits", C.c_void_p), ("tp", C.POINTER(TP))]


_p, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); must list every symbol the header declares.
SIGNATURES = {
    "alloyb_version": (_i, []),
    "alloyb_error_string": (C.c_char_p, [_i]),
    "alloyb_last_cuda_error": (_i, []),
    "alloyb_device_supported": (_i, []),
    "alloyb_device_error": (_i, [_i]),
    "alloyb_dequant_q4k": (_i, [_p, _p, _p, _i64, _i64, _i, _i, _p]),
    "alloyb_dequant_q6k": (_i, [_p, _p, _p, _i64, _i64, _i, _i, _p]),
    "alloyb_dequant_q8_0": (_i, [_p, _p, _p, _p, _i64, _i64, _i, _i, _p]),
    "alloyb_linear": (_i, [_p, _i, _i, _i, C.POINTER(Weight), _i, _p, _p]),
    "alloyb_q4k_mm": (_i, [_p, _p, _p, _i, _i, _i, _i, _p]),
    "alloyb_q6k_mm": (_i, [_p, _p, _p, _i, _i, _i, _i, _p]),
    "alloyb_q8_0_mm": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "alloyb_gated_linear": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "alloyb_linear_normed": (_i, [_p, _p, _f, _p, _i, _i, _i, C.POINTER(Weight), _i, _p]),
    "alloyb_gated_linear_normed": (_i, [_p, _p, _f, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "alloyb_rope_kv_append": (_i, [_i, _p, _p, _p, _i64, _i64, _p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _i, _i, _i64,
                                   _p, _p]),
    "alloyb_tp_buffer_bytes": (_sz, [_i]),
    "alloyb_tp_alloc": (_i, [_sz, C.POINTER(_p)]),
    "alloyb_tp_free": (_i, [_p]),
    "alloyb_tp_ipc_export": (_i, [_p, _p]),
    "alloyb_tp_ipc_import": (_i, [_p, C.POINTER(_p)]),
    "alloyb_tp_ipc_close": (_i, [_p]),
    "alloyb_linear_allreduce": (_i, [_p, _i, _i, _i, C.POINTER(Weight), _p, C.POINTER(TP), _p]),
    "alloyb_kv_quantize_q8": (_i, [_p, _i64, _i64, _i64, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "alloyb_kv_dequant_q8": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "alloyb_kv_append_q8_paged": (_i, [_p, _p, _i64, _i64, _p, _p, _i, _i64, _p, _i, _i, _i, _p, _p]),
    "alloyb_attn_workspace_bytes": (_sz, [_i, _i, _i]),
    "alloyb_attn_workspace_init": (_i, [_p, _sz, _i, _i, _p]),
    "alloyb_attn_workspace_status": (_i, [_p, C.POINTER(C.c_int32), _p]),
    "alloyb_attn_decode": (_i, [_i, _p, _i64, _i64, _i, _p, _p, _p, _p, _p, _p, _i64, _i64, _p, _i,
                                _p, _i, _i, _i, _i, _i, _i64, _f, _i, _p, _sz, _p]),
    "alloyb_attn_decode_rope": (_i, [_i, _p, _i64, _i64, _p, _p, _p, _p, _p, _p, _i64, _i64, _p, _i, _p,
                                     _p, _i, _i, _i, _i, _i, _i64, _f, _p, _sz, _p]),
    "alloyb_attn_decode_static": (_i, [_i, _p, _i64, _i64, _i, _p, _p, _p, _p, _p, _p, _i64, _i64, _p, _i,
                                       _p, _i, _i, _i, _i, _i, _i64, _f, _i, _p]),
    "alloyb_attn_static_status": (_i, [C.POINTER(C.c_int32), _p]),
    "alloyb_dequant_q5_0": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i, _i, _p]),
    "alloyb_q5_0_mm": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "alloyb_kv_write": (_i, [_i, _p, _p, _i64, _i64, _i64, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i64, _i, _p, _p]),
    "alloyb_attn_chunk": (_i, [_i, _p, _i64, _i64, _i64, _i, _p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _i, _i, _i,
                               _i64, _f, _p, _p]),
    "alloyb_moe_workspace_bytes": (_sz, [_i, _i, _i]),
    "alloyb_moe_routed": (_i, [_p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _sz, _p]),
    "alloyb_decoder_create": (_i, [C.POINTER(DecoderDesc), C.POINTER(_p)]),
    "alloyb_decoder_step": (_i, [_p, _p]),
    "alloyb_decoder_phases": (_i, [_p]),
    "alloyb_decoder_status": (_i, [_p, C.POINTER(C.c_int32), _p]),
    "alloyb_decoder_trace": (_i, [_p, _i]),
    "alloyb_decoder_trace_read": (_i, [_p, C.POINTER(C.c_uint64), _i]),
    "alloyb_decoder_destroy": (_i, [_p]),
    "alloyb_rms_norm": (_i, [_p, _p, _p, _i, _i, _f, _i, _p]),
    "alloyb_rope_inplace": (_i, [_p, _p, _p, _i, _p, _i, _i, _i, _i, _i, _p]),
    "alloyb_silu_mul": (_i, [_p, _p, _p, _i64, _i, _p]),
    "alloyb_argmax": (_i, [_p, _p, _i, _i, _i, _p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once and attach argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise AlloyB200Error(
            f"{LIB_PATH} is missing: build it with `python -m alloy_b200.build` "
            "(there is no CPU or eager fallback for these ops)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    """Raise on a negative status, naming the call."""
    if code == 0:
        return
    lib = load()
    msg = lib.alloyb_error_string(code).decode()
    extra = ""
    if code == -5:
        extra = f" (cudaError {lib.alloyb_last_cuda_error()})"
    raise AlloyB200Error(f"{what}: {msg}{extra}")

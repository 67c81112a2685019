"""alloy_b200 — B200-native (sm_100a) drop-in for the quantised-LLM hot path of
rayanht/alloy: GGUF Q4_K/Q6_K/Q8_0 dequant-fused linears and decode attention
over a q8_0 KV cache, behind the ``torch.ops.alloy.*`` operator surface.

Importing the package registers the ops.  The kernels live in
``liballoy_b200.so`` (built in-tree by ``python -m alloy_b200.build``); without
it every op raises — there is no CPU or eager fallback.
"""

from . import ops  # noqa: F401
from .kv import KV_FORMATS, Q8_0, KVFormat, PagedKVPool, alloc_quantized_kv, resolve_kv_format
from .quant import (QUANT_FORMATS, GGUFQ4_KEmbedding, GGUFQ4_KLinear, GGUFQ5_0Embedding, GGUFQ5_0Linear,
                    GGUFQ6_KEmbedding, GGUFQ6_KLinear, GGUFQ8_0Embedding, GGUFQ8_0Linear, GGUFQuantEmbedding,
                    GGUFQuantLinear, QuantFormat, split_q5_0_weight, split_q8_0_weight, validate_quant_buffers)

__all__ = [
    "ops", "KVFormat", "Q8_0", "KV_FORMATS", "resolve_kv_format", "alloc_quantized_kv", "PagedKVPool",
    "QuantFormat", "QUANT_FORMATS", "validate_quant_buffers", "GGUFQuantLinear", "GGUFQuantEmbedding",
    "GGUFQ4_KLinear", "GGUFQ6_KLinear", "GGUFQ8_0Linear", "GGUFQ4_KEmbedding", "GGUFQ6_KEmbedding",
    "GGUFQ8_0Embedding", "GGUFQ5_0Linear", "GGUFQ5_0Embedding", "split_q8_0_weight", "split_q5_0_weight",
]

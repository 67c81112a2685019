"""KV-cache formats and stores.

``KVFormat`` / ``Q8_0`` / ``KV_FORMATS`` / ``resolve_kv_format`` are adapted from the reference's
``packages/alloy-server/src/alloy_server/kv_format.py:14-63`` (a format descriptor whose field
names, values and error text are the contract its callers rely on); ``alloc_quantized_kv``
allocates the split codes+scales tensors of
``packages/alloy-server/src/alloy_server/cache.py:36-60``.

``PagedKVPool`` is new: the reference's "paged" store hands out virtually
contiguous slices of one VM reservation
(``packages/alloy-server/src/alloy_server/generation/kv.py:298-575``), which has
no CUDA counterpart, so here a page table maps each sequence's 16-token pages
into one pool of 34-byte q8_0 blocks and the attention kernel follows it.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

BLOCK_ELEMS_Q8_0 = 32
PAGE_TOKENS = 16
KV_BLOCK_BYTES = 34


@dataclass(frozen=True)
class KVFormat:
    name: str
    bits_per_elem_k: float
    bits_per_elem_v: float
    block_elems: int
    group_tokens: int

    def code_bytes_per_row(self, head_dim: int) -> int:
        assert head_dim % self.block_elems == 0, (head_dim, self.block_elems)
        return head_dim

    def scale_count_per_row(self, head_dim: int) -> int:
        return head_dim // self.block_elems


Q8_0 = KVFormat(name="q8_0", bits_per_elem_k=8.5, bits_per_elem_v=8.5,
                block_elems=BLOCK_ELEMS_Q8_0, group_tokens=1)
KV_FORMATS: dict[str, KVFormat] = {Q8_0.name: Q8_0}


def resolve_kv_format(name: str | None) -> KVFormat | None:
    """``None``/"none" -> fp16 cache; unknown names raise (never a silent fp16 fallback)."""
    if name is None:
        name = os.environ.get("ALLOY_KV_QUANT")
    if name is None or name == "none":
        return None
    try:
        return KV_FORMATS[name]
    except KeyError:
        raise ValueError(
            f"unknown KV format {name!r}; available: none, {', '.join(sorted(KV_FORMATS))}") from None


def alloc_quantized_kv(max_batch_size: int, num_kv_heads: int, phys_len: int, head_dim: int,
                       device, kv_format: KVFormat = Q8_0):
    """(k_codes, k_scales, v_codes, v_scales): int8 (B,KV_H,S,D) + fp16 (B,KV_H,S,D/32)."""
    assert head_dim % kv_format.block_elems == 0, (head_dim, kv_format.block_elems)
    cs = (max_batch_size, num_kv_heads, phys_len, head_dim)
    ss = (max_batch_size, num_kv_heads, phys_len, head_dim // kv_format.block_elems)
    return (torch.zeros(cs, dtype=torch.int8, device=device),
            torch.zeros(ss, dtype=torch.float16, device=device),
            torch.zeros(cs, dtype=torch.int8, device=device),
            torch.zeros(ss, dtype=torch.float16, device=device))


class PagedKVPool:
    """One layer's pool of 16-token q8_0 pages plus the per-sequence page table.

    ``pool``: uint8 (num_pages, 2, KV_H, 16, D/32*34) — K then V slab per page,
    each token row D/32 blocks of (fp16 scale, 32 int8 codes).
    ``page_table``: int32 (max_batch, max_pages_per_seq), -1 = unmapped.
    Pages are handed out from a free list (host side); sequences never share a
    page.  ``page_table`` may be shared between the layers of a model (same
    mapping in every layer's pool) by passing it in.
    """

    def __init__(self, num_pages: int, num_kv_heads: int, head_dim: int, max_batch: int,
                 max_pages_per_seq: int, device, page_table: torch.Tensor | None = None,
                 free_order: list[int] | None = None) -> None:
        if head_dim % BLOCK_ELEMS_Q8_0:
            raise ValueError(f"head_dim {head_dim} not divisible by {BLOCK_ELEMS_Q8_0}")
        self.num_pages = int(num_pages)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.row_bytes = head_dim // BLOCK_ELEMS_Q8_0 * KV_BLOCK_BYTES
        self.pool = torch.zeros((num_pages, 2, num_kv_heads, PAGE_TOKENS, self.row_bytes),
                                dtype=torch.uint8, device=device)
        self.page_table = page_table if page_table is not None else torch.full(
            (max_batch, max_pages_per_seq), -1, dtype=torch.int32, device=device)
        self._host_table = [[] for _ in range(self.page_table.shape[0])]
        order = list(range(num_pages)) if free_order is None else list(free_order)
        self._free = order[::-1]

    @property
    def max_pages_per_seq(self) -> int:
        return self.page_table.shape[1]

    def bytes_per_token(self) -> int:
        return 2 * self.num_kv_heads * self.row_bytes

    def reserve(self, seq: int, n_tokens: int) -> None:
        """Make sure sequence ``seq`` has pages for positions [0, n_tokens)."""
        need = (n_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS
        have = self._host_table[seq]
        if need > self.max_pages_per_seq:
            raise ValueError(f"{n_tokens} tokens need {need} pages > {self.max_pages_per_seq}")
        if need > len(have):
            if need - len(have) > len(self._free):
                raise MemoryError("KV page pool exhausted")
            new = [self._free.pop() for _ in range(need - len(have))]
            start = len(have)
            have.extend(new)
            self.page_table[seq, start:need] = torch.tensor(new, dtype=torch.int32,
                                                            device=self.page_table.device)

    def release(self, seq: int) -> None:
        pages = self._host_table[seq]
        self._free.extend(reversed(pages))
        self._host_table[seq] = []
        self.page_table[seq].fill_(-1)

    def pages_of(self, seq: int) -> list[int]:
        return list(self._host_table[seq])

"""Tensor-parallel sharding of the quantised linears (new; the reference is single-GPU).

Column-parallel matrices (q, k, v, gate, up, output head) keep a contiguous range of OUTPUT
rows of the packed weight; row-parallel matrices (o_proj, down) keep a contiguous range of
super-blocks of EVERY row, i.e. a K-slice on 256-element boundaries, and their partial
outputs are summed over the ranks with one all-reduce (NCCL over NVLink on GPUs; any
``torch.distributed`` backend works, which is how the logic is tested on CPU with gloo).
"""

from __future__ import annotations

from collections.abc import Callable

import torch
import torch.distributed as dist

BLOCK_BYTES = {"q4_k": 144, "q6_k": 210}


def shard_rows(weight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Column-parallel shard: output rows [rank*N/world, (rank+1)*N/world)."""
    n = weight.shape[0]
    if n % world:
        raise ValueError(f"{n} output rows do not split {world} ways")
    per = n // world
    return weight[rank * per:(rank + 1) * per].contiguous()


def shard_cols(blocks: torch.Tensor, fmt: str, rank: int, world: int) -> torch.Tensor:
    """Row-parallel shard: super-blocks [rank*nb/world, (rank+1)*nb/world) of every row."""
    bb = BLOCK_BYTES[fmt]
    n = blocks.shape[0]
    if blocks.shape[1] % bb:
        raise ValueError(f"row of {blocks.shape[1]} bytes is not whole {bb}-byte blocks")
    nb = blocks.shape[1] // bb
    if nb % world:
        raise ValueError(f"{nb} super-blocks per row do not split {world} ways")
    per = nb // world
    return blocks.view(n, nb, bb)[:, rank * per:(rank + 1) * per].reshape(n, per * bb).contiguous()


def k_slice(k: int, rank: int, world: int) -> slice:
    """The activation columns that go with ``shard_cols``."""
    if k % (256 * world):
        raise ValueError(f"K={k} does not split {world} ways on super-block boundaries")
    per = k // world
    return slice(rank * per, (rank + 1) * per)


def row_parallel(x_shard: torch.Tensor, mm: Callable[[torch.Tensor], torch.Tensor],
                 group=None) -> torch.Tensor:
    """``mm`` applied to this rank's K-slice, then summed over the group (in place)."""
    y = mm(x_shard)
    if group is not None or (dist.is_initialized() and dist.get_world_size() > 1):
        dist.all_reduce(y, group=group)
    return y


def gather_columns(y_shard: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate column-parallel outputs (M, N/world) of all ranks into (M, N)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y_shard
    parts = [torch.empty_like(y_shard) for _ in range(world)]
    dist.all_gather(parts, y_shard.contiguous(), group=group)
    return torch.cat(parts, dim=1)

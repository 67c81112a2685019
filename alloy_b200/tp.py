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
    shard = blocks.view(n, nb, bb)[:, rank * per:(rank + 1) * per].reshape(n, per * bb)
    if (per * bb) % 16 == 0:
        return shard.contiguous()
    # keep a 16-byte row pitch (bulk / TMA copies need it): a strided view of a padded buffer
    pitch = (per * bb + 15) // 16 * 16
    buf = torch.zeros((n, pitch), dtype=blocks.dtype, device=blocks.device)
    buf[:, :per * bb] = shard
    return buf[:, :per * bb]


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


class PeerExchange:
    """This rank's exchange buffer plus the mapped buffers of the other ranks of ``group``.

    Set-up for ``ops.linear_allreduce`` (the row-parallel linear whose all-reduce runs inside
    the GEMV launch over NVLink peer memory).  Every rank allocates one buffer through the C
    library, the 64-byte CUDA IPC handles travel through one ``all_gather`` of the group, and
    each rank maps the others' buffers.  ``world == 1`` needs no group.
    """

    def __init__(self, max_n: int, rank: int = 0, world: int = 1, group=None, device=None) -> None:
        import ctypes as C

        from . import _lib

        if not 1 <= world <= 8:
            raise ValueError("1..8 ranks")
        self.rank, self.world, self.max_n = rank, world, int(max_n)
        self._L = L = _lib.load()
        self._own = C.c_void_p()
        _lib.check(L.alloyb_tp_alloc(L.alloyb_tp_buffer_bytes(self.max_n), C.byref(self._own)), "alloyb_tp_alloc")
        self._imported: list = []
        ptrs = [None] * world
        ptrs[rank] = self._own.value
        if world > 1:
            handle = (C.c_ubyte * 64)()
            _lib.check(L.alloyb_tp_ipc_export(self._own, handle), "alloyb_tp_ipc_export")
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=device)
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine, group=group)
            for r in range(world):
                if r == rank:
                    continue
                raw = (C.c_ubyte * 64)(*parts[r].cpu().tolist())
                p = C.c_void_p()
                _lib.check(L.alloyb_tp_ipc_import(raw, C.byref(p)), "alloyb_tp_ipc_import")
                self._imported.append(p)
                ptrs[r] = p.value
        self.desc = _lib.TP(world, rank, self.max_n, 0, (C.c_void_p * 8)(*ptrs, *([None] * (8 - world))))

    def close(self) -> None:
        for p in self._imported:
            self._L.alloyb_tp_ipc_close(p)
        self._imported = []
        if self._own:
            self._L.alloyb_tp_free(self._own)
            self._own = None


def agree(local_ok: bool, group=None, device=None) -> bool:
    """True only if EVERY rank of the group passes True (one MIN all-reduce).  The ranks of a
    tensor-parallel step must all run the same kernels: whenever one of them cannot take the
    peer-memory path (mapping failed, a bounded wait on a peer ran out), all of them leave it."""
    if not (dist.is_initialized() and dist.get_world_size(group) > 1):
        return bool(local_ok)
    flag = torch.tensor([1 if local_ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(int(flag.item()) == 1)


def rel_errors(got: torch.Tensor, ref: torch.Tensor) -> tuple[float, float]:
    """(max, mean) element-wise relative error of ``got`` against ``ref``, |ref| floored at 1 % of
    rms(ref): the tolerance metric of the parity tests (max <= 1e-2, mean <= 1e-3)."""
    g, r = got.double().flatten(), ref.double().flatten()
    rms = float(r.pow(2).mean().sqrt()) or 1.0
    err = (g - r).abs() / r.abs().clamp_min(1e-2 * rms)
    return float(err.max()), float(err.mean())


ROW_PARALLEL_CHECK_SHAPES = (("q4_k", 8192, 8192), ("q6_k", 8192, 28672))   # 70B o_proj and down


def check_row_parallel(exchange, rank: int, world: int, group, device, shapes=ROW_PARALLEL_CHECK_SHAPES,
                       epochs: int = 3, seed: int = 1234) -> dict:
    """Per-op parity of the tensor-parallel row-parallel linear on the live ranks.

    For each (format, N, K): every rank draws the same full matrix, token and residual, computes
    the unsharded result with the single-GPU kernel on its own GPU (the oracle of tensor
    parallelism: the same op at TP = 1), then its K shard goes through (a) the linear whose
    all-reduce runs inside the launch over peer memory (``exchange``; skipped when None) and
    (b) the plain linear + ``all_reduce`` of fp16 partials.  Returns the worst (max, mean)
    relative errors over shapes, epochs and ranks and ``pass`` for the fused path
    (max <= 1e-2 and mean <= 1e-3).
    """
    from . import ops, synth

    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    worst = {"fused": [0.0, 0.0], "nccl": [0.0, 0.0]}
    fused_calls = 0
    for fmt, n, k in shapes:
        make = synth.q4k_blocks_device if fmt == "q4_k" else synth.q6k_blocks_device
        w = make(n, k, gen, device, 0.1)
        shard = shard_cols(w, fmt, rank, world)
        mm = torch.ops.alloy.gguf_q4_k_mm if fmt == "q4_k" else torch.ops.alloy.gguf_q6_k_mm
        for _ in range(epochs):
            x = torch.randn((1, k), device=device, generator=gen).to(torch.float16)
            r = torch.randn((1, n), device=device, generator=gen).to(torch.float16)
            ref = torch.ops.alloy.linear_residual(x, w, None, r, fmt)
            xs = x[:, k_slice(k, rank, world)].contiguous()
            if exchange is not None:
                y = ops.linear_allreduce(xs, fmt, shard, r, exchange)
                if y is not None:
                    fused_calls += 1
                    mx, mean = rel_errors(y, ref)
                    worst["fused"] = [max(worst["fused"][0], mx), max(worst["fused"][1], mean)]
            part = mm(xs, shard)
            if world > 1:
                dist.all_reduce(part, group=group)
            mx, mean = rel_errors(r + part, ref)
            worst["nccl"] = [max(worst["nccl"][0], mx), max(worst["nccl"][1], mean)]
        del w, shard
    t = torch.tensor(worst["fused"] + worst["nccl"] + [float(-fused_calls)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    v = t.tolist()
    calls = int(-v[4])                                   # the fewest fused calls any rank made
    expected = len(shapes) * epochs if exchange is not None else 0
    return {"shapes": [list(s) for s in shapes], "epochs": epochs,
            "fused": {"max_rel": v[0], "mean_rel": v[1], "calls": calls},
            "nccl_fp16_partials": {"max_rel": v[2], "mean_rel": v[3]},
            "reference": "the same linear on the unsharded matrix, single-GPU kernel, on each rank's GPU",
            "pass": bool(exchange is None or (calls == expected and v[0] <= 1e-2 and v[1] <= 1e-3))}

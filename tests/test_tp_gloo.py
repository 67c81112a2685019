"""World-size-2 gloo test of the tensor-parallel sharding logic on CPU.

The CUDA ops have no CPU kernel, so each rank runs the oracle's dequant + matmul on ITS shard;
what is under test is the host logic: which rows / super-blocks a rank keeps, which activation
columns go with them, and that all-reduce / all-gather put the pieces back together.
"""

import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from alloy_b200 import synth, tp
from oracle import blocks as O


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)                 # same seed on every rank: same full matrices
        m, k, n = 3, 1024, 96
        x = torch.from_numpy(synth.activations(rng, m, k, np.float32))
        w4 = torch.from_numpy(synth.q4k_blocks(rng, n, k))
        w6 = torch.from_numpy(synth.q6k_blocks(rng, n, k))
        full4 = x.numpy() @ O.dequant_q4_k(w4.numpy()).T
        full6 = x.numpy() @ O.dequant_q6_k(w6.numpy()).T

        # row-parallel (o_proj / down): K-slice of every row + all-reduce
        for w, fmt, deq, full in ((w4, "q4_k", O.dequant_q4_k, full4), (w6, "q6_k", O.dequant_q6_k, full6)):
            shard = tp.shard_cols(w, fmt, rank, world)
            assert shard.shape == (n, w.shape[1] // world)
            xs = x[:, tp.k_slice(k, rank, world)]
            y = tp.row_parallel(xs, lambda t: torch.from_numpy(t.numpy() @ deq(shard.numpy()).T))
            np.testing.assert_allclose(y.numpy(), full, rtol=2e-5, atol=2e-4)

        # column-parallel (q/k/v/gate/up/head): row range + all-gather
        shard = tp.shard_rows(w4, rank, world)
        ys = torch.from_numpy(x.numpy() @ O.dequant_q4_k(shard.numpy()).T)
        y = tp.gather_columns(ys)
        np.testing.assert_allclose(y.numpy(), full4, rtol=1e-6, atol=1e-6)

        # shapes that do not shard are refused before any collective
        with pytest.raises(ValueError):
            tp.shard_cols(torch.zeros((4, 3 * 144), dtype=torch.uint8), "q4_k", rank, world)
        with pytest.raises(ValueError):
            tp.k_slice(768, rank, world)
        q.put((rank, "ok"))
    except Exception as e:                              # surface the failure in the parent
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_tp_sharding_world2_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def _agree_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 1 reports a failed peer set-up / a wait that ran out: BOTH ranks must leave the peer path
        got = [tp.agree(True), tp.agree(rank != 1), tp.agree(rank != 0), tp.agree(False)]
        q.put((rank, got))
    except Exception as e:
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_fallback_decision_is_collective_world2_gloo():
    """The choice between the fused peer-memory exchange and NCCL is one MIN all-reduce: a failure
    seen by one rank only (its IPC mapping failed, its wait on a peer ran out) moves every rank."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_agree_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results == {0: [True, False, False, False], 1: [True, False, False, False]}, results
    assert tp.agree(True) and not tp.agree(False)          # no process group: the local answer


def test_shard_helpers_single_process():
    w = torch.arange(4 * 2 * 144, dtype=torch.int64).remainder(251).to(torch.uint8).reshape(4, 288)
    a, b = tp.shard_cols(w, "q4_k", 0, 2), tp.shard_cols(w, "q4_k", 1, 2)
    assert torch.equal(torch.cat([a, b], dim=1), w)
    assert torch.equal(torch.cat([tp.shard_rows(w, r, 2) for r in range(2)]), w)
    assert tp.k_slice(1024, 1, 2) == slice(512, 1024)

"""Time ONE hot-path op in isolation on the current GPU (event-timed, cold L2).

The counterpart of the reference's ``alloy microbench``
(``packages/alloy-cli/src/alloy_cli/commands/microbench.py:31-113``: warm-ups, then the
median of repeated GPU-timestamp runs of one production dispatch).  Small matrices fit
in the B200's 126 MB L2, so each op runs over a RING of distinct weight replicas whose
total size exceeds ``--ring-mb`` and the launches of one sweep are captured in one CUDA
graph; the figure printed is the mean device time per launch and the algorithmic bytes
(weights + activations + outputs) per launch over it.

    python -m alloy_b200.microbench --op q4k_mm --n 4096 --k 4096 --m 1
    python -m alloy_b200.microbench --op gated  --n 14336 --k 4096 --m 1
    python -m alloy_b200.microbench --op q6k_mm --n 4096 --k 14336 --m 4
    python -m alloy_b200.microbench --op attn_paged --batch 64 --ctx-lo 4096 --ctx-hi 32768
    python -m alloy_b200.microbench --op gemm_q4k --m 4096 --n 14336 --k 4096 --dtype bf16
    python -m alloy_b200.microbench --op q8_mm --n 4096 --k 4096 --m 1
"""

from __future__ import annotations

import argparse
import json
import statistics

import torch

from . import ops, synth


def _time_graph(fn, sweeps: int, warm: int = 3) -> list[float]:
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(warm):
        g.replay()
    out = []
    for _ in range(sweeps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return out


def bench_linear(op: str, n: int, k: int, m: int, ring_mb: int, sweeps: int, dtype) -> dict:
    gen = torch.Generator(device="cuda").manual_seed(0)
    if op == "q6k_mm":
        per = n * (k // 256) * 210
        make = lambda: (synth.q6k_blocks_device(n, k, gen),)
        call = lambda x, w: torch.ops.alloy.gguf_q6_k_mm(x, w[0])
    elif op == "q4k_mm":
        per = n * (k // 256) * 144
        make = lambda: (synth.q4k_blocks_device(n, k, gen),)
        call = lambda x, w: torch.ops.alloy.gguf_q4_k_mm(x, w[0])
    elif op == "q8_mm":
        per = n * k + n * (k // 32) * 2
        make = lambda: synth.q8_0_weight_device(n, k, gen)
        call = lambda x, w: torch.ops.alloy.gguf_q8_0_mm(x, w[0], w[1])
    elif op == "gated":
        per = 2 * n * (k // 256) * 144
        make = lambda: (synth.q4k_blocks_device(n, k, gen), synth.q4k_blocks_device(n, k, gen))
        call = lambda x, w: torch.ops.alloy.gguf_q4_k_silu(x, w[0], w[1])
    else:
        raise ValueError(op)
    replicas = max(2, -(-ring_mb * 1024 * 1024 // per))
    ws = [make() for _ in range(replicas)]
    x = torch.randn((m, k), device="cuda").to(dtype)

    def sweep():
        for w in ws:
            call(x, w)

    ms = _time_graph(sweep, sweeps)
    alg = per + m * k * 2 + m * n * 2
    us = [t * 1e3 / replicas for t in ms]
    med = statistics.median(us)
    return {"op": op, "n": n, "k": k, "m": m, "replicas": replicas, "bytes_per_launch": alg,
            "us_per_launch_median": med, "us_per_launch_min": min(us),
            "gbs_median": alg / med / 1e3, "gbs_best": alg / min(us) / 1e3}


def bench_gemm(fmt: str, m: int, n: int, k: int, sweeps: int, dtype) -> dict:
    """Prefill dequant-GEMM (tcgen05 path): M tokens against one packed matrix."""
    gen = torch.Generator(device="cuda").manual_seed(0)
    if fmt == "q8":
        qw, qs = synth.q8_0_weight_device(n, k, gen)
        blk = qw
        op = lambda x, w: torch.ops.alloy.gguf_q8_0_mm(x, w, qs)
        wbytes = n * k + n * (k // 32) * 2
    elif fmt == "q6k":
        blk = synth.q6k_blocks_device(n, k, gen)
        op = torch.ops.alloy.gguf_q6_k_mm
        wbytes = n * (k // 256) * 210
    else:
        blk = synth.q4k_blocks_device(n, k, gen)
        op = torch.ops.alloy.gguf_q4_k_mm
        wbytes = n * (k // 256) * 144
    x = torch.randn((m, k), device="cuda").to(dtype)
    ms = _time_graph(lambda: op(x, blk), sweeps)
    med = statistics.median(ms)
    flop = 2.0 * m * n * k
    return {"op": f"gemm_{fmt}", "m": m, "n": n, "k": k, "flop": flop, "bytes": wbytes + 2 * m * k + 2 * m * n,
            "ms_median": med, "ms_min": min(ms), "tflops_median": flop / med / 1e9,
            "tflops_best": flop / min(ms) / 1e9}


def bench_attn_paged(batch: int, lo: int, hi: int, sweeps: int, kv_heads: int = 8, group: int = 4,
                     d: int = 128) -> dict:
    from .kv import PagedKVPool

    gen = torch.Generator(device="cuda").manual_seed(0)
    cpu = torch.Generator().manual_seed(0)
    lens = torch.randint(lo, hi + 1, (batch,), generator=cpu)
    pages_per = [(int(n) + 16) // 16 for n in lens]
    total = sum(pages_per)
    order = torch.randperm(total, generator=cpu).tolist()
    store = PagedKVPool(total, kv_heads, d, batch, max(pages_per), "cuda", free_order=order)
    for i in range(batch):
        store.reserve(i, int(lens[i]) + 1)
    store.pool.copy_(torch.randint(0, 256, store.pool.shape, dtype=torch.uint8, device="cuda",
                                   generator=gen))
    blocks = store.pool.view(-1, 34)
    sc = torch.empty(blocks.shape[0], device="cuda").uniform_(0.015, 0.03, generator=gen).half()
    blocks[:, 0:2] = sc.view(torch.uint8).view(-1, 2)
    h = kv_heads * group
    q = torch.randn((batch, h, 1, d), device="cuda").half()
    nk = torch.randn((batch, kv_heads, 1, d), device="cuda").half()
    nv = torch.randn((batch, kv_heads, 1, d), device="cuda").half()
    pos = lens.to(torch.int32).cuda()

    def run():
        torch.ops.alloy.attention_cache_q8_paged(q, nk, nv, pos, store.page_table, store.pool)

    ms = _time_graph(run, sweeps)
    alg = int((lens + 1).sum()) * store.bytes_per_token()
    med = statistics.median(ms)
    return {"op": "attn_paged", "batch": batch, "ctx": [lo, hi], "tokens": int((lens + 1).sum()),
            "bytes_per_launch": alg, "us_median": med * 1e3, "us_min": min(ms) * 1e3,
            "gbs_median": alg / med / 1e6, "gbs_best": alg / min(ms) / 1e6}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True,
                    choices=["q4k_mm", "q6k_mm", "q8_mm", "gated", "attn_paged", "gemm_q4k", "gemm_q6k", "gemm_q8"])
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"])
    ap.add_argument("--ring-mb", type=int, default=512)
    ap.add_argument("--sweeps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx-lo", type=int, default=4096)
    ap.add_argument("--ctx-hi", type=int, default=32768)
    a = ap.parse_args()
    dt = torch.float16 if a.dtype == "f16" else torch.bfloat16
    if a.op == "attn_paged":
        res = bench_attn_paged(a.batch, a.ctx_lo, a.ctx_hi, a.sweeps)
    elif a.op.startswith("gemm_"):
        res = bench_gemm(a.op[5:], a.m, a.n, a.k, a.sweeps, dt)
    else:
        res = bench_linear(a.op, a.n, a.k, a.m, a.ring_mb, a.sweeps,
                           torch.float16 if a.dtype == "f16" else torch.bfloat16)
    print(json.dumps(res))


if __name__ == "__main__":
    main()

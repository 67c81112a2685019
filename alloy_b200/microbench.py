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
    python -m alloy_b200.microbench --op layer_ops --batch 1            # the 8B decode step's five launches per layer
    python -m alloy_b200.microbench --op layer_ops --model 70b --tp-dry 8
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


def bench_layer_ops(model: str, batch: int, tp_dry: int, sweeps: int) -> dict:
    """The decode step's per-layer launches, each kind timed on its own: one CUDA graph runs the op of all
    layers back to back (every layer's own weights and cache, so nothing comes from L2), and the figure is the
    mean device time per launch.  The sum over the kinds is what a step would take if its launches followed
    each other as smoothly as launches of one kind do; the step itself is timed beside it."""
    from . import llama

    shape = llama.LLAMA3_70B if model == "70b" else llama.LLAMA3_8B
    context, kv = (4096, "q8_paged") if model == "70b" else (2048, "f16")
    extra = dict(tp_rank=0, tp_size=tp_dry, tp_dry=True) if tp_dry > 1 else {}
    d = llama.QuantLlamaDecoder(shape, batch, context, seed=0, d_scale=0.1, centered=True, kv=kv, **extra)
    d.capture()
    s, n_layers = d.shape, len(d.layers)
    gen = torch.Generator(device="cuda").manual_seed(1)
    rnd = lambda *sh: (torch.randn(sh, device="cuda", generator=gen) * 0.1).half()
    h, a2, act = rnd(batch, s.hidden), rnd(batch, d.heads_l * s.head_dim), rnd(batch, d.ffn_l)
    q3, k3, v3 = rnd(batch, d.heads_l, s.head_dim), rnd(batch, d.kv_heads_l, s.head_dim), rnd(batch, d.kv_heads_l, s.head_dim)
    scale = 1.0 / s.head_dim ** 0.5

    def qkv():
        for lw in d.layers:
            ops.linear_multi(h, [(lw.fmt["wq"], lw.wq, None), (lw.fmt["wk"], lw.wk, None), (lw.fmt["wv"], lw.wv, None)],
                             norm=(lw.norm_in, s.eps))

    def attn():
        for li in range(n_layers):
            if kv == "f16":
                ops.rope_attention_decode(q3, k3, v3, d.pos, d.inv_freq, scale=scale, k_cache=d.k_cache[li],
                                          v_cache=d.v_cache[li])
            else:
                ops.rope_attention_decode(q3, k3, v3, d.seq_pos, d.inv_freq, scale=scale,
                                          paged=(d.pools[li].page_table, d.pools[li].pool))

    def row_parallel(x, name):
        for lw in d.layers:
            w = getattr(lw, name)
            if d.tp_size == 1:
                torch.ops.alloy.linear_residual(x, w, None, h, lw.fmt[name])
            else:
                d._row_parallel(x, lw.fmt[name], w, h)

    def gate_up():
        for lw in d.layers:
            ops.gated_normed(h, lw.norm_post, s.eps, lw.wg, lw.wu)

    kinds = [("qkv", qkv), ("attention", attn), ("o", lambda: row_parallel(a2, "wo")), ("gate_up", gate_up),
             ("down", lambda: row_parallel(act, "wd"))]
    res = {"op": "layer_ops", "model": model, "batch": batch, "tp_dry": tp_dry, "layers": n_layers, "us_per_launch": {}}
    for name, fn in kinds:
        ms = _time_graph(fn, sweeps)
        res["us_per_launch"][name] = statistics.median(ms) * 1e3 / n_layers
    res["sum_us_per_layer"] = sum(res["us_per_launch"].values())
    for _ in range(3):
        d.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(20):
        d.step()
    b.record()
    torch.cuda.synchronize()
    res["step_ms"] = a.elapsed_time(b) / 20
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True,
                    choices=["q4k_mm", "q6k_mm", "q8_mm", "gated", "attn_paged", "gemm_q4k", "gemm_q6k", "gemm_q8",
                             "layer_ops"])
    ap.add_argument("--model", default="8b", choices=["8b", "70b"])
    ap.add_argument("--tp-dry", type=int, default=1, help="layer_ops: one rank's share of an N-way split, nobody to exchange with")
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"])
    ap.add_argument("--ring-mb", type=int, default=512)
    ap.add_argument("--sweeps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=None, help="attn_paged: sequences (default 64); layer_ops: tokens per step (default 1)")
    ap.add_argument("--ctx-lo", type=int, default=4096)
    ap.add_argument("--ctx-hi", type=int, default=32768)
    a = ap.parse_args()
    dt = torch.float16 if a.dtype == "f16" else torch.bfloat16
    if a.op == "layer_ops":
        res = bench_layer_ops(a.model, a.batch or 1, a.tp_dry, min(a.sweeps, 10))
    elif a.op == "attn_paged":
        res = bench_attn_paged(a.batch or 64, a.ctx_lo, a.ctx_hi, a.sweeps)
    elif a.op.startswith("gemm_"):
        res = bench_gemm(a.op[5:], a.m, a.n, a.k, a.sweeps, dt)
    else:
        res = bench_linear(a.op, a.n, a.k, a.m, a.ring_mb, a.sweeps,
                           torch.float16 if a.dtype == "f16" else torch.bfloat16)
    print(json.dumps(res))


if __name__ == "__main__":
    main()

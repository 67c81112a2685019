"""Benchmark of the quantised-LLM decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--workload NAME]
    python bench.py --impl reference ...      # the CPU path of the reference, same metric

One step = one decode step (one new token per sequence) of a random-init Q4_K_M
Llama-shape model under a CUDA graph.  N=1 runs the Llama-3-8B shape with an fp16
KV cache at context 2048; N>1 (under torchrun, one rank per GPU) runs the
Llama-3-70B shape tensor-parallel over N GPUs with NCCL all-reduce on the
row-parallel outputs.  Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

WORKLOADS = {
    "llama3-8b-q4km-decode": dict(shape="LLAMA3_8B", context=2048, kv="f16"),
    "llama3-70b-q4km-decode": dict(shape="LLAMA3_70B", context=4096, kv="q8_paged"),
}
METRIC = "decode_tokens_per_s"
WEIGHT_D_SCALE = 0.1    # multiplier on the synthetic block scales: zero-mean weights of std ~0.02


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _measured_peaks() -> tuple[float, str]:
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def _ncu_traffic(kernel: str):
    """DRAM bytes per launch of the named kernel from the committed ncu summary, if any."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            return json.load(f).get(kernel)
    except (OSError, ValueError):
        return None


def _event_ms(fn, stream=None) -> float:
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b)


# --------------------------------------------------------------------------------- CPU baseline


def cpu_layer_sample(shape, batch: int, seed: int = 0, row_div: int = 1) -> dict:
    """Time the reference's CPU-side path (NumPy block dequantiser -> torch CPU fp32 matmul)
    on 1/row_div of the rows of ONE transformer layer's seven matrices plus 1/(16*row_div)
    of the output head, and extrapolate to a full decode step.  Attention and norms are
    left out (negligible on the CPU path)."""
    import numpy as np

    from alloy_b200 import synth
    from oracle import blocks as O

    torch.set_num_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(seed)
    hd, kvd = shape.heads * shape.head_dim, shape.kv_heads * shape.head_dim
    mats = [("q4", hd, shape.hidden), ("q4", kvd, shape.hidden), ("q6", kvd, shape.hidden),
            ("q4", shape.hidden, hd), ("q4", shape.ffn, shape.hidden), ("q4", shape.ffn, shape.hidden),
            ("q6", shape.hidden, shape.ffn)]
    head_rows = shape.vocab // 16
    t_deq = t_mm = 0.0
    for fmt, n, k in mats + [("q6h", head_rows, shape.hidden)]:
        n = max(16, n // row_div)
        blk = synth.q4k_blocks(rng, n, k) if fmt == "q4" else synth.q6k_blocks(rng, n, k)
        x = torch.from_numpy(synth.activations(rng, batch, k))
        t0 = time.perf_counter()
        w = O.dequant_q4_k(blk) if fmt == "q4" else O.dequant_q6_k(blk)
        t1 = time.perf_counter()
        y = x.float() @ torch.from_numpy(w).T
        y = y.to(torch.float16)
        t2 = time.perf_counter()
        full_n = head_rows * 16 if fmt == "q6h" else None
        scale = (full_n / n) if fmt == "q6h" else float(shape.layers) * row_div
        t_deq += (t1 - t0) * scale
        t_mm += (t2 - t1) * scale
    step_s = t_deq + t_mm
    return {"step_s": step_s, "dequant_s": t_deq, "matmul_s": t_mm,
            "tok_s": batch / step_s, "cores": torch.get_num_threads(),
            "sample": (f"1/{row_div} of the rows of 1 of {shape.layers} layers (7 matrices) + "
                       f"1/{16 * row_div} of the head rows at batch "
                       f"{batch}, NumPy dequant (1 thread) + torch fp32 matmul "
                       f"({torch.get_num_threads()} threads), extrapolated to a full step")}


def run_reference(args, shape, workload: str) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    last = None
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        last = cpu_layer_sample(shape, args.batch, seed=i, row_div=16)
        if i >= args.warmup:
            times.append(last["step_s"])
    step_s = statistics.mean(times)
    val = args.batch / step_s
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "batch": args.batch, "context": WORKLOADS[workload]["context"],
                   "kv": WORKLOADS[workload]["kv"], "parallelism": "host cores (attention and norms left out)"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": last["cores"], "kind": "port",
                         "sample": last["sample"]},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------- GPU arm


def gemv_roofline(dec, reps: int = 8) -> dict:
    """Live event timing of the dominant kernel: the fused Q4_K gate/up dequant-GEMV, one
    launch per layer over that layer's own weights (distinct matrices, 2 GB+ in total, so
    nothing is served from L2)."""
    s = dec.shape
    x = torch.randn((dec.batch, s.hidden), device=dec.device).to(dec.dtype)

    def sweep():
        for lw in dec.layers:
            torch.ops.alloy.gguf_q4_k_silu(x, lw.wg, lw.wu)

    sweep()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sweep()
    g.replay()
    ms = _event_ms(lambda: [g.replay() for _ in range(reps)])
    launches = reps * len(dec.layers)
    n, k = dec.layers[0].wg.shape[0], s.hidden
    alg = 2 * n * (k // 256) * 144 + dec.batch * k * 2 + dec.batch * n * 2
    return {"kernel": "q4k gate/up fused dequant-GEMV", "bytes_per_launch": alg,
            "us_per_launch": ms * 1e3 / launches, "gbs": alg / (ms * 1e-3 / launches) / 1e9}


def run_ours(args, shape_name: str, wl: dict, workload: str) -> None:
    import alloy_b200  # noqa: F401
    from alloy_b200 import llama, ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dry = args.tp_dry if world == 1 else 0
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torchrun); WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    pg = None
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
        pg = torch.distributed.group.WORLD
    shape = getattr(llama, shape_name)
    dev = torch.device("cuda", local)

    t_start = time.perf_counter()

    def note(msg):
        if args.verbose:
            print(f"[bench rank {rank} +{time.perf_counter() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    def build(batch):
        note(f"building decoder batch={batch}")
        # zero-mean weights of std ~0.02 (centred Q4_K blocks, block scales at 0.1 of the kernel-test
        # range): the residual stream of 32 to 80 random layers stays inside fp16, the logits finite
        d = llama.QuantLlamaDecoder(shape, batch, wl["context"], device=dev, seed=0, kv=wl["kv"],
                                    tp_rank=rank, tp_size=dry or world, process_group=pg, tp_dry=bool(dry),
                                    d_scale=WEIGHT_D_SCALE, centered=True)
        torch.cuda.synchronize()
        note("weights ready; capturing")
        d.capture()
        torch.cuda.synchronize()
        note("captured")
        return d

    def timed(dec, steps, warmup):
        gen = torch.Generator().manual_seed(1)
        dec.ids.copy_(torch.randint(0, shape.vocab, (dec.batch,), generator=gen))
        for _ in range(warmup):
            dec.step()
        if world > 1:
            torch.distributed.barrier()
        ms = _event_ms(lambda: [dec.step() for _ in range(steps)])
        t = torch.tensor([ms], device=dev)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    def timed_e2e(dec, steps, warmup):
        gen = torch.Generator().manual_seed(2)
        host_ids = torch.randint(0, shape.vocab, (steps + warmup, dec.batch), generator=gen).pin_memory()
        host_out = torch.empty((dec.batch,), dtype=torch.int64).pin_memory()

        def one(i):
            dec.ids.copy_(host_ids[i], non_blocking=True)
            out = dec.step()
            host_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for i in range(warmup):
            one(i)
        if world > 1:
            torch.distributed.barrier()
        ms = _event_ms(lambda: [one(warmup + i) for i in range(steps)])
        t = torch.tensor([ms], device=dev)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item()), dec.batch * 8, dec.batch * 8

    dec = build(args.batch)
    with ClockSampler(local) as clocks:
        ms = timed(dec, args.steps, args.warmup)
        note(f"timed: {ms / args.steps:.3f} ms/step")
        e2e_ms, h2d, d2h = timed_e2e(dec, args.steps, args.warmup)
        note("e2e timed")
        # a short run can end before nvidia-smi has printed once: keep the same step running (untimed,
        # the same count on every rank) until rank 0's sampler holds a reading taken under load
        for _ in range(40):
            done = torch.tensor([1 if (clocks.rows or clocks.proc is None) else 0], device=dev)
            if world > 1:
                torch.distributed.broadcast(done, 0)
            if int(done.item()):
                break
            for _ in range(20):
                dec.step()
            torch.cuda.synchronize()
    value = args.batch * args.steps / (ms * 1e-3)
    e2e_val = args.batch * args.steps / (e2e_ms * 1e-3)
    w_bytes = shape.weight_bytes()
    peak, peak_kind = _measured_peaks()
    roof = gemv_roofline(dec)
    tp_check = None
    if world > 1 and args.check_tp:
        # the same step with the all-reduce inside the GEMV launches (peer memory) and with NCCL
        note("tp check: building the twins")
        # fp16 KV here: its random contents are a slice of the unsharded cache's, so that the same
        # step of the whole model on this one GPU (fp32 sums over the full K) can referee the two
        mk = lambda peer, size=world: llama.QuantLlamaDecoder(
            shape, args.batch, wl["context"], device=dev, seed=0, kv="f16", tp_rank=rank if size > 1 else 0,
            tp_size=size, process_group=pg if size > 1 else None, d_scale=WEIGHT_D_SCALE, centered=True,
            peer_allreduce=peer)
        fused, twin = mk(True), mk(False)
        for d in (fused, twin):
            d.ids.fill_(11)
        a = fused.step_eager_logits().float().clone()
        b = twin.step_eager_logits().float().clone()
        calls = fused.fused_allreduce_calls
        torch.cuda.synchronize()
        del fused, twin
        torch.cuda.empty_cache()
        whole = mk(False, 1)
        whole.ids.fill_(11)
        c = whole.step_eager_logits().float().clone()
        rms = c.pow(2).mean().sqrt()
        both = torch.stack([(a - b).abs().max() / rms, (a - c).abs().max() / rms, (b - c).abs().max() / rms])
        torch.distributed.all_reduce(both, op=torch.distributed.ReduceOp.MAX)
        tp_check = {"max_abs_diff_over_rms": {"fused_vs_nccl": float(both[0].item()),
                                              "fused_vs_one_gpu": float(both[1].item()),
                                              "nccl_vs_one_gpu": float(both[2].item())},
                    "fused_calls_per_step": calls, "finite": bool(torch.isfinite(a).all().item())}
        torch.cuda.synchronize()
        del whole
        torch.cuda.empty_cache()
    launches_step = dec.launches_per_step + shape.layers + 1   # + KV append per layer + id copy
    finite = bool(torch.isfinite(dec.logits.float()).all().item())

    per_batch = {}
    if world == 1 and not args.no_sweep:
        for b in (1, 4, 16, 32):
            if b == args.batch:
                per_batch[str(b)] = {"ms_per_step": ms / args.steps, "tokens_per_s": value}
                continue
            del dec
            torch.cuda.empty_cache()
            dec = build(b)
            bms = timed(dec, args.steps, args.warmup)
            per_batch[str(b)] = {"ms_per_step": bms / args.steps,
                                 "tokens_per_s": b * args.steps / (bms * 1e-3)}
        for b, r in per_batch.items():
            kv_bytes = int(b) * shape.layers * 2 * shape.kv_heads * shape.head_dim * wl["context"] * 2
            r["frac_of_weight_bound"] = (w_bytes / (peak * 1e9)) / (r["ms_per_step"] * 1e-3)
            r["frac_of_weight_plus_kv_bound"] = ((w_bytes + kv_bytes) / (peak * 1e9)) / (r["ms_per_step"] * 1e-3)

    if rank != 0:
        _leave(world)
        return
    cpu = None
    if world == 1 and not args.no_cpu:
        # three independently seeded samples (~10-15 s of host work), averaged
        runs = [cpu_layer_sample(shape, args.batch, seed=i) for i in range(3)]
        cpu = dict(runs[0])
        cpu["step_s"] = statistics.mean(r["step_s"] for r in runs)
        cpu["tok_s"] = args.batch / cpu["step_s"]
        cpu["sample"] = "mean of 3 samples, each: " + runs[0]["sample"]
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": workload, "batch": args.batch, "context": wl["context"], "kv": wl["kv"],
                   "parallelism": f"tp{world}" if not dry else f"rank 0 of tp{dry}, no peers (not a bench value)", "weight_bytes_per_step": w_bytes // world,
                   "l2": "each step streams its weights once (GBs, far above the 126 MB L2)",
                   "logits_finite": finite, "weight_d_scale": WEIGHT_D_SCALE},
        "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_step * args.steps,
        "clocks": clocks.summary(),
        "weight_stream": {"bytes_per_step": w_bytes // world, "achieved_gbs": (w_bytes / world) / (ms / args.steps * 1e-3) / 1e9,
                          "frac_of_peak": (w_bytes / world) / (ms / args.steps * 1e-3) / 1e9 / peak,
                          "peak_gbs": peak, "peak_kind": peak_kind},
    }
    if roof is not None:
        # the committed ncu capture is of the 8B shape's launch: quoted only where this run's launch is that one
        traffic = _ncu_traffic("gated_q4k")
        if traffic is not None and abs(traffic / roof["bytes_per_launch"] - 1.0) > 0.1:
            traffic = None
        line["roofline"] = {"bound": "hbm", "achieved": roof["gbs"], "peak": peak, "unit": "GB/s",
                            "frac": roof["gbs"] / peak, "traffic": traffic,
                            "kernel": roof["kernel"], "bytes_per_launch": roof["bytes_per_launch"],
                            "us_per_launch": roof["us_per_launch"], "peak_kind": peak_kind}
    if tp_check is not None:
        line["config"]["tp_check"] = tp_check
    if world > 1:
        line["config"]["allreduce"] = ("inside the o_proj/down GEMV launches over NVLink peer memory"
                                       if dec.exchange is not None else "NCCL")
    if per_batch:
        line["per_batch"] = per_batch
    if cpu is not None:
        line["cpu_baseline"] = {"value": cpu["tok_s"], "unit": "tokens/s", "cores": cpu["cores"],
                                "kind": "port", "sample": cpu["sample"]}
    print(json.dumps(line), flush=True)
    _leave(world)


def _leave(world: int) -> None:
    """End a multi-rank run.  The process group is NOT destroyed: with NCCL collectives
    captured in a live CUDA graph, ``destroy_process_group`` blocked for minutes on this
    stack, so the ranks meet at a barrier and exit directly."""
    if world > 1:
        torch.cuda.synchronize()
        torch.distributed.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--tp-dry", type=int, default=0,
                    help="1 GPU: time rank 0's share of a TP-N step with nobody to exchange with (profiling aid; "
                         "not a bench value)")
    ap.add_argument("--check-tp", action="store_true",
                    help="N > 1: also run one step with NCCL all-reduces and report the logits difference")
    ap.add_argument("--no-sweep", action="store_true", help="skip the batch 1/4/16/32 sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline")
    ap.add_argument("--verbose", action="store_true", help="progress notes on stderr")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    workload = args.workload or ("llama3-8b-q4km-decode" if args.gpus == 1 else "llama3-70b-q4km-decode")
    wl = WORKLOADS[workload]
    if args.impl == "reference":
        from alloy_b200 import llama
        run_reference(args, getattr(llama, wl["shape"]), workload)
        return
    run_ours(args, wl["shape"], wl, workload)


if __name__ == "__main__":
    sys.exit(main())

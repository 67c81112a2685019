"""Benchmark of the quantised-LLM decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--workload NAME]
    python bench.py --impl reference ...      # the CPU path of the reference, same metric

One step = one decode step (one new token per sequence) of a random-init Q4_K_M
Llama-shape model under a CUDA graph.  N=1 runs the Llama-3-8B shape with an fp16
KV cache at context 2048; N>1 (under torchrun, one rank per GPU) runs the
Llama-3-70B shape tensor-parallel over N GPUs, the row-parallel sums crossing
NVLink inside the o_proj / down GEMV launches.  Prints ONE JSON line on rank 0.

Besides the contract keys the line carries, measured in the same process:
``roofline`` (the dominant kernel, the fused gate/up GEMV, timed live), ``gemv_cfg0``
(the 4096 x 4096 Q4_K GEMV over a ring of replicas larger than L2), ``prefill_gemm``
(the two M = 4096 dequant-GEMMs), ``attn_paged`` (batch-64 paged q8_0 decode attention,
contexts 4096..32768), ``per_batch`` and ``cpu_baseline``; at N > 1 ``config.tp_check``
(per-op parity of the row-parallel linear against the unsharded single-GPU kernel) and
``tp1_equiv`` (the same 70B step timed on ONE GPU by rank 0, the denominator of the
tensor-parallel scaling).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
WORKLOADS = {
    "llama3-8b-q4km-decode": dict(shape="LLAMA3_8B", context=2048, kv="f16"),
    "llama3-70b-q4km-decode": dict(shape="LLAMA3_70B", context=4096, kv="q8_paged"),
}
METRIC = "decode_tokens_per_s"
WEIGHT_D_SCALE = 0.1    # multiplier on the synthetic block scales: zero-mean weights of std ~0.02
CPU_ROW_DIV = 16        # the CPU leg times 1/16 of the rows of one layer (+ 1/256 of the head) per sample


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


def _measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "kind": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


def _source_hash(files) -> str:
    h = hashlib.sha256()
    for rel in files:
        with open(os.path.join(ROOT, rel), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _ncu_traffic(key: str) -> tuple:
    """(DRAM bytes per launch, note) from the committed ncu summary of kernel+shape ``key``; the
    number is quoted only while the kernel sources it was captured from are unchanged."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            entry = json.load(f).get(key)
    except (OSError, ValueError):
        entry = None
    if not entry:
        return None, f"no ncu capture recorded for {key}"
    try:
        now = _source_hash(entry["sources"])
    except OSError:
        return None, "kernel sources not found"
    if now != entry["source_sha256"]:
        return None, f"stale: {', '.join(entry['sources'])} changed since the capture in {entry['capture']}"
    return entry["dram_bytes"], entry["capture"]


def _event_ms(fn) -> float:
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b)


# --------------------------------------------------------------------------------- CPU baseline


def cpu_layer_sample(shape, batch: int, seed: int = 0, row_div: int = CPU_ROW_DIV) -> dict:
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
    t_deq = t_mm = t_wall = 0.0
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
        scale = (head_rows * 16 / n) if fmt == "q6h" else float(shape.layers) * row_div
        t_deq += (t1 - t0) * scale
        t_mm += (t2 - t1) * scale
        t_wall += t2 - t0
    step_s = t_deq + t_mm
    return {"step_s": step_s, "sample_s": t_wall, "dequant_s": t_deq, "matmul_s": t_mm,
            "tok_s": batch / step_s, "cores": torch.get_num_threads(),
            "sample": (f"1/{row_div} of the rows of 1 of {shape.layers} layers (7 matrices) + "
                       f"1/{16 * row_div} of the head rows at batch "
                       f"{batch}, NumPy dequant (1 thread) + torch fp32 matmul "
                       f"({torch.get_num_threads()} threads), extrapolated to a full step")}


def run_reference(args, shape, workload: str) -> None:
    """The reference arm: the reference's CPU path of the linears on this box's host cores.  A step
    is ONE bounded sample (the same sample the GPU arm's ``cpu_baseline`` uses); ``value`` is the
    tokens/s a full step would give, extrapolated from it, and ``ms_per_step`` the wall time of the
    sample actually run."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, walls, last = [], [], None
    for i in range(args.warmup + args.steps):
        last = cpu_layer_sample(shape, args.batch, seed=i)
        if i >= args.warmup:
            steps.append(last["step_s"])
            walls.append(last["sample_s"])
    step_s = statistics.mean(steps)
    val = args.batch / step_s
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.mean(walls) * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "batch": args.batch, "context": WORKLOADS[workload]["context"],
                   "kv": WORKLOADS[workload]["kv"], "parallelism": "host cores (attention and norms left out)",
                   "extrapolated": True, "full_step_ms_extrapolated": step_s * 1e3,
                   "cpu_sample": last["sample"]},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": last["cores"], "kind": "port",
                         "sample": last["sample"], "extrapolated": True},
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
    return {"kernel": "q4k gate/up fused dequant-GEMV", "shape": f"2x{n}x{k}_m{dec.batch}", "bytes_per_launch": alg,
            "us_per_launch": ms * 1e3 / launches, "gbs": alg / (ms * 1e-3 / launches) / 1e9}


def kernel_extras(peaks: dict, note) -> dict:
    """The other configured kernels, each timed alone over inputs larger than L2 (or re-streamed
    from HBM every launch) in this process: config 0, config 2 and config 3."""
    from alloy_b200 import microbench as mb

    out = {}
    try:
        note("gemv cfg0")
        r = mb.bench_linear("q4k_mm", 4096, 4096, 1, 512, 10, torch.float16)       # 57 replicas = 540 MB
        out["gemv_cfg0"] = {"shape": "Q4_K 4096x4096, one fp16 token", "replicas": r["replicas"],
                            "launches_timed": r["replicas"] * 10, "bytes_per_launch": r["bytes_per_launch"],
                            "us_per_launch": r["us_per_launch_median"], "gbs": r["gbs_median"],
                            "frac_of_hbm_peak": r["gbs_median"] / peaks["hbm_gbs"]}
    except Exception as e:  # noqa: BLE001 - an extra must not lose the contract line
        out["gemv_cfg0"] = {"error": repr(e)}
    try:
        note("prefill gemm")
        gemms = {}
        for fmt, n, k in (("q4k", 14336, 4096), ("q6k", 4096, 14336)):
            r = mb.bench_gemm(fmt, 4096, n, k, 8, torch.bfloat16)
            gemms[f"{fmt}_{n}x{k}"] = {"m": 4096, "ms": r["ms_median"], "tflops": r["tflops_median"],
                                       "frac_of_bf16_burst": r["tflops_median"] / peaks["bf16_tflops"],
                                       "frac_of_bf16_sustained": r["tflops_median"] / peaks["bf16_tflops_sustained"]}
        out["prefill_gemm"] = gemms
    except Exception as e:  # noqa: BLE001
        out["prefill_gemm"] = {"error": repr(e)}
    try:
        note("paged attention")
        r = mb.bench_attn_paged(64, 4096, 32768, 8)
        out["attn_paged"] = {"batch": 64, "ctx": [4096, 32768], "layout": "16-token pages of 34-byte q8_0 blocks, shuffled",
                             "tokens": r["tokens"], "bytes_per_launch": r["bytes_per_launch"], "us": r["us_median"],
                             "gbs": r["gbs_median"], "frac_of_hbm_peak": r["gbs_median"] / peaks["hbm_gbs"]}
    except Exception as e:  # noqa: BLE001
        out["attn_paged"] = {"error": repr(e)}
    torch.cuda.empty_cache()
    return out


def run_ours(args, shape_name: str, wl: dict, workload: str) -> None:
    import alloy_b200  # noqa: F401
    from alloy_b200 import llama, tp

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
    peaks = _measured_peaks()
    peak = peaks["hbm_gbs"]
    w_bytes = shape.weight_bytes()
    one_launch = {"auto": False, "one-launch": True, "per-op": False}[args.step]

    t_start = time.perf_counter()

    def note(msg):
        if args.verbose:
            print(f"[bench rank {rank} +{time.perf_counter() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    def build(batch, *, solo=False, fused=None):
        """``solo``: the whole model on this GPU (no tensor parallelism), whatever the world size."""
        note(f"building decoder batch={batch} solo={solo}")
        # zero-mean weights of std ~0.02 (centred Q4_K blocks, block scales at 0.1 of the kernel-test
        # range): the residual stream of 32 to 80 random layers stays inside fp16, the logits finite
        d = llama.QuantLlamaDecoder(shape, batch, wl["context"], device=dev, seed=0, kv=wl["kv"],
                                    tp_rank=0 if solo else rank, tp_size=1 if solo else (dry or world),
                                    process_group=None if solo else pg, tp_dry=bool(dry) and not solo,
                                    d_scale=WEIGHT_D_SCALE, centered=True,
                                    one_launch=one_launch if fused is None else fused,
                                    fused_attention=not args.split_attention)
        torch.cuda.synchronize()
        note("weights ready; capturing")
        d.capture()
        torch.cuda.synchronize()
        note("captured")
        return d

    def timed(dec, steps, warmup, *, collective=True):
        gen = torch.Generator().manual_seed(1)
        dec.ids.copy_(torch.randint(0, shape.vocab, (dec.batch,), generator=gen))
        for _ in range(warmup):
            dec.step()
        if world > 1 and collective:
            torch.distributed.barrier()
        ms = _event_ms(lambda: [dec.step() for _ in range(steps)])
        t = torch.tensor([ms], device=dev)
        if world > 1 and collective:
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

    # ---- tensor parallel: the same step on ONE GPU first (rank 0 alone; 44 GB fits one B200): the
    # denominator of the scaling figure.  The other ranks wait at the barrier below.
    tp1 = None
    if world > 1 and not args.no_tp1:
        if rank == 0:
            try:
                solo = build(args.batch, solo=True)
                solo_ms = timed(solo, args.steps, args.warmup, collective=False) / args.steps
                tp1 = {"ms_per_step": solo_ms, "bytes_per_s": w_bytes / (solo_ms * 1e-3),
                       "frac_of_hbm_peak": w_bytes / (solo_ms * 1e-3) / 1e9 / peak, "device_error": solo.device_error()}
                del solo
            except Exception as e:  # noqa: BLE001
                tp1 = {"error": repr(e)}
            torch.cuda.empty_cache()
        torch.cuda.synchronize()
        torch.distributed.barrier()

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
    # a bounded wait that ran out anywhere in the timed steps voids them
    dev_err = torch.tensor([dec.device_error()], device=dev)
    if world > 1:
        torch.distributed.all_reduce(dev_err, op=torch.distributed.ReduceOp.MAX)
    dev_err = int(dev_err.item())
    value = args.batch * args.steps / (ms * 1e-3)
    e2e_val = args.batch * args.steps / (e2e_ms * 1e-3)
    roof = gemv_roofline(dec)
    launches_step = dec.launches_per_step + 1              # + the copy of the new token ids
    finite = bool(torch.isfinite(dec.logits.float()).all().item())
    step_kind = "one persistent launch" if dec._fused is not None else "op by op"
    allreduce = None
    if world > 1:
        allreduce = ("inside the o_proj/down GEMV launches over NVLink peer memory" if dec.exchange is not None
                     else "NCCL")

    # ---- tensor parallel: per-op parity of the row-parallel linear on the live ranks (every run)
    tp_check = None
    if world > 1:
        note("tp check")
        torch.cuda.synchronize()
        torch.distributed.barrier()
        tp_check = tp.check_row_parallel(dec.exchange, rank, world, pg, dev)
        tp_check["device_error"] = int(dec.device_error())
    step_check = None
    if world > 1 and args.check_tp:
        step_check = whole_step_check(args, shape, wl, rank, world, pg, dev)

    per_batch = {}
    sweep = () if args.no_sweep else ((1, 4, 16, 32) if world == 1 else (1, 64))
    for b in sweep:
        if b == args.batch:
            per_batch[str(b)] = {"ms_per_step": ms / args.steps, "tokens_per_s": value}
            continue
        try:
            del dec
            torch.cuda.empty_cache()
            dec = build(b)
            bms = timed(dec, args.steps, args.warmup)
            per_batch[str(b)] = {"ms_per_step": bms / args.steps, "tokens_per_s": b * args.steps / (bms * 1e-3)}
        except Exception as e:  # noqa: BLE001 - a sweep point must not lose the contract line
            per_batch[str(b)] = {"error": repr(e)}
            break
    kv_row = 2 * shape.kv_heads * shape.head_dim * (2 if wl["kv"] == "f16" else 34 / 32)
    for b, r in per_batch.items():
        if "ms_per_step" not in r:
            continue
        kv_bytes = int(b) * shape.layers * kv_row * wl["context"]
        r["frac_of_weight_bound"] = (w_bytes / world / (peak * 1e9)) / (r["ms_per_step"] * 1e-3)
        r["frac_of_weight_plus_kv_bound"] = ((w_bytes + kv_bytes) / world / (peak * 1e9)) / (r["ms_per_step"] * 1e-3)

    extras, one_launch_cmp = {}, None
    if world == 1 and not dry and not args.no_extras:
        dec = None
        torch.cuda.empty_cache()
        extras = kernel_extras(peaks, note)
        if args.batch == 1 and args.step == "auto":
            # the same step as ONE persistent launch (opt-in; the op-by-op step is the default)
            try:
                alt = build(1, fused=True)
                ams = timed(alt, args.steps, args.warmup) / args.steps
                one_launch_cmp = {"ms_per_step": ams, "tokens_per_s": 1e3 / ams, "phases": alt._fused.phases,
                                  "device_error": alt.device_error()}
                del alt
            except Exception as e:  # noqa: BLE001
                one_launch_cmp = {"error": repr(e)}
            torch.cuda.empty_cache()
        # the prompt side of the same model: one chunk of `context` tokens through prefill() (tensor-core
        # GEMMs, causal chunk attention, K/V written to the cache), eager, timed with CUDA events
        try:
            pre = llama.QuantLlamaDecoder(shape, 1, wl["context"], device=dev, seed=0, kv=wl["kv"],
                                          d_scale=WEIGHT_D_SCALE, centered=True)
            gen = torch.Generator().manual_seed(2)
            prompt = torch.randint(0, shape.vocab, (1, wl["context"]), generator=gen)
            pre.prefill(prompt)                                    # warm-up
            torch.cuda.synchronize()
            pms = min(_event_ms(lambda: pre.prefill(prompt)) for _ in range(3))
            flop = 2.0 * shape.layer_weight_elems() * wl["context"]          # the layers' linears only
            extras["prefill"] = {"tokens": wl["context"], "ms": pms, "tokens_per_s": wl["context"] / (pms * 1e-3),
                                 "logits_finite": bool(torch.isfinite(pre.logits.float()).all().item()),
                                 "device_error": pre.device_error()}
            if flop:
                extras["prefill"]["linear_tflops"] = flop / pms / 1e9
                extras["prefill"]["frac_of_bf16_burst"] = flop / pms / 1e9 / peaks["bf16_tflops"]
            del pre
        except Exception as e:  # noqa: BLE001
            extras["prefill"] = {"error": repr(e)}
        torch.cuda.empty_cache()

    if rank != 0:
        _leave(world)
        return
    cpu = None
    if not args.no_cpu:
        # three independently seeded samples (a few seconds of host work each), averaged; the SAME
        # sample the reference arm times
        runs = [cpu_layer_sample(shape, args.batch, seed=i) for i in range(3)]
        cpu = dict(runs[0])
        cpu["step_s"] = statistics.mean(r["step_s"] for r in runs)
        cpu["tok_s"] = args.batch / cpu["step_s"]
        cpu["sample"] = "mean of 3 samples, each: " + runs[0]["sample"]
    ws_gbs = (w_bytes / world) / (ms / args.steps * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": workload, "batch": args.batch, "context": wl["context"], "kv": wl["kv"],
                   "parallelism": f"tp{world}" if not dry else f"rank 0 of tp{dry}, no peers (not a bench value)",
                   "step": step_kind, "weight_bytes_per_step": w_bytes // world,
                   "l2": "each step streams its weights once (GBs, far above the 126 MB L2)",
                   "logits_finite": finite, "weight_d_scale": WEIGHT_D_SCALE, "device_error": dev_err},
        "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_step * args.steps,
        "clocks": clocks.summary(),
        "weight_stream": {"bytes_per_step": w_bytes // world, "achieved_gbs": ws_gbs, "frac_of_peak": ws_gbs / peak,
                          "peak_gbs": peak, "peak_kind": peaks["kind"]},
    }
    traffic, traffic_source = _ncu_traffic(f"gemv_stream_gate_up_q4k_{roof['shape']}")
    line["roofline"] = {"bound": "hbm", "achieved": roof["gbs"], "peak": peak, "unit": "GB/s",
                        "frac": roof["gbs"] / peak, "traffic": traffic, "traffic_source": traffic_source,
                        "kernel": roof["kernel"], "shape": roof["shape"], "bytes_per_launch": roof["bytes_per_launch"],
                        "us_per_launch": roof["us_per_launch"], "peak_kind": peaks["kind"]}
    if dev_err:
        line["config"]["invalid"] = "a bounded device-side wait ran out during the timed steps"
    if tp_check is not None:
        line["config"]["tp_check"] = tp_check
    if step_check is not None:
        line["config"]["tp_step_check"] = step_check
    if allreduce is not None:
        line["config"]["allreduce"] = allreduce
    if tp1 is not None:
        line["tp1_equiv"] = dict(tp1)
        if "ms_per_step" in tp1:
            line["tp1_equiv"].update({
                "what": "the same 70B step on one GPU, timed by rank 0 before the tensor-parallel run",
                "scaling_vs_tp1": tp1["ms_per_step"] / (ms / args.steps),
                "tp1_equiv_bytes_per_s": w_bytes / (ms / args.steps * 1e-3),
                "per_rank_hbm_frac": ws_gbs / peak})
    if per_batch:
        line["per_batch"] = per_batch
    if one_launch_cmp is not None:
        line["one_launch_step"] = one_launch_cmp
    line.update(extras)
    if cpu is not None:
        line["cpu_baseline"] = {"value": cpu["tok_s"], "unit": "tokens/s", "cores": cpu["cores"],
                                "kind": "port", "sample": cpu["sample"], "extrapolated": True}
        line["config"]["cpu_sample"] = cpu["sample"]
    print(json.dumps(line), flush=True)
    _leave(world)


def whole_step_check(args, shape, wl, rank, world, pg, dev) -> dict:
    """--check-tp: the whole 80-layer step with the fused exchange, with NCCL all-reduces of fp16
    partials, and on one GPU (fp32 sums over the full K) as referee.  A deep random stack amplifies
    rounding differences, so this is an extra beside the per-op check, with a loose bound."""
    from alloy_b200 import llama

    mk = lambda peer, size=world: llama.QuantLlamaDecoder(
        shape, args.batch, wl["context"], device=dev, seed=0, kv="f16", tp_rank=rank if size > 1 else 0,
        tp_size=size, process_group=pg if size > 1 else None, d_scale=WEIGHT_D_SCALE, centered=True,
        peer_allreduce=peer, one_launch=False)
    fused, twin = mk(True), mk(False)
    for d in (fused, twin):
        d.ids.fill_(11)
    a = fused.step_eager_logits().float().clone()
    b = twin.step_eager_logits().float().clone()
    calls = fused.fused_allreduce_calls
    err = fused.device_error()
    torch.cuda.synchronize()
    del fused, twin
    torch.cuda.empty_cache()
    whole = mk(False, 1)
    whole.ids.fill_(11)
    c = whole.step_eager_logits().float().clone()
    rms = c.pow(2).mean().sqrt()
    both = torch.stack([(a - b).abs().max() / rms, (a - c).abs().max() / rms, (b - c).abs().max() / rms])
    torch.distributed.all_reduce(both, op=torch.distributed.ReduceOp.MAX)
    out = {"max_abs_diff_over_rms": {"fused_vs_nccl": float(both[0].item()), "fused_vs_one_gpu": float(both[1].item()),
                                     "nccl_vs_one_gpu": float(both[2].item())},
           "fused_calls_per_step": calls, "finite": bool(torch.isfinite(a).all().item()), "device_error": int(err),
           "bound": 0.1, "pass": bool(float(both[1].item()) <= 0.1 and err == 0)}
    torch.cuda.synchronize()
    del whole
    torch.cuda.empty_cache()
    return out


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
                    help="N > 1: also run the whole step with NCCL all-reduces and on one GPU and report the logits difference")
    ap.add_argument("--step", default="auto", choices=["auto", "one-launch", "per-op"],
                    help="batch 1: the whole step as one persistent launch, or op by op (auto: op by op, with the "
                         "one-launch step timed beside it at N = 1)")
    ap.add_argument("--split-attention", action="store_true",
                    help="RoPE + KV append as a launch of their own instead of inside the attention kernel")
    ap.add_argument("--no-sweep", action="store_true", help="skip the batch sweep")
    ap.add_argument("--no-extras", action="store_true", help="N = 1: skip the config 0 / 2 / 3 kernel timings")
    ap.add_argument("--no-tp1", action="store_true", help="N > 1: skip the one-GPU run of the same step")
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

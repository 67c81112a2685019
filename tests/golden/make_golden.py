"""Regenerate the golden fixtures in this folder.

Runs only where the reference checkout and the ``gguf`` package (0.19.0, the
version the reference pins) are both present; the fixtures it writes are
committed so that the tests need neither.

    python tests/golden/make_golden.py --reference /path/to/reference

What produces each fixture:

* ``q4k.npz``   weights: the reference's own test decoder (``_dequant`` and
  ``_get_scale_min_k4`` from ``tests/kernels/test_quant_q4k_native.py``, executed
  from the checkout, on blocks drawn by its ``_make_blocks``) AND
  ``gguf.quants.dequantize``; the script asserts they agree bit-for-bit.
* ``q6k.npz``, ``q8_0.npz``   ``gguf.quants.dequantize`` (the reference's tests
  hold no host decoder for these formats).
* ``q5_0.npz``   the reference's ``split_q5_0_weight`` (the three normalised
  buffers, from ``packages/alloy-server/src/alloy_server/gguf/quant.py``) on random
  22-byte wire blocks, and ``gguf.quants.dequantize`` of the same blocks.
* ``attn_chunk.npz``   causal chunk attention over a q8_0 cache: the reference's
  ``_quantize_ref`` + ``_ref_attention`` applied per query row, as its prefill test
  does inline (``tests/kernels/test_kv_quant.py:466-479``).
* ``kv_q8.npz``   the reference's ``_quantize_ref`` from
  ``tests/kernels/test_kv_quant.py`` (codes + scales), its dequantisation, and
  its float64 ``_ref_attention``.

The helper functions are pulled out of the reference's test modules by name
with ``ast`` because those modules import the Metal runtime at the top and
cannot be imported on Linux.
"""

from __future__ import annotations

import argparse
import os
import ast
import pathlib
import sys

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from alloy_b200 import synth  # noqa: E402


def _extract(path: pathlib.Path, names: list[str]) -> dict:
    tree = ast.parse(path.read_text())
    keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in keep}
    if missing:
        raise SystemExit(f"{path}: missing {sorted(missing)}")
    ns: dict = {"np": np}
    exec(compile(ast.Module(body=keep, type_ignores=[]), str(path), "exec"), ns)
    return ns


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ALLOY_REFERENCE"), required="ALLOY_REFERENCE" not in os.environ,
                    help="path of the rayanht/alloy checkout (or set ALLOY_REFERENCE)")
    args = ap.parse_args()
    ref = pathlib.Path(args.reference)

    import gguf
    from gguf import GGMLQuantizationType as T
    from gguf.quants import dequantize

    q4 = _extract(ref / "tests/kernels/test_quant_q4k_native.py",
                  ["_make_blocks", "_get_scale_min_k4", "_dequant"])
    kvt = _extract(ref / "tests/kernels/test_kv_quant.py", ["_quantize_ref", "_ref_attention"])

    # ---- Q4_K: reference-test generator (signed d) and the benchmark generator
    rng = np.random.default_rng(0)
    blk_ref = q4["_make_blocks"](6, 3, rng)
    w_ref = q4["_dequant"](blk_ref, 6, 3)
    w_gguf = dequantize(blk_ref.reshape(-1, 144), T.Q4_K).reshape(6, 3 * 256)
    assert w_ref.dtype == np.float32 and np.array_equal(w_ref.view(np.uint32), w_gguf.view(np.uint32))
    blk_b = synth.q4k_blocks(np.random.default_rng(1), 8, 512)
    w_b_ref = q4["_dequant"](blk_b, 8, 2)
    w_b = dequantize(blk_b.reshape(-1, 144), T.Q4_K).reshape(8, 512)
    assert np.array_equal(w_b_ref.view(np.uint32), w_b.view(np.uint32))
    x = synth.activations(np.random.default_rng(2), 3, 512, np.float16)
    np.savez_compressed(HERE / "q4k.npz", blocks_signed=blk_ref, w_signed=w_ref,
                        blocks=blk_b, w=w_b, x=x,
                        y=(x.astype(np.float32) @ w_b.T).astype(np.float32))

    # ---- Q6_K
    blk6 = synth.q6k_blocks(np.random.default_rng(3), 8, 512)
    w6 = dequantize(blk6.reshape(-1, 210), T.Q6_K).reshape(8, 512)
    np.savez_compressed(HERE / "q6k.npz", blocks=blk6, w=w6.astype(np.float32))

    # ---- Q8_0 weights (wire blocks)
    wire = synth.q8_0_wire(np.random.default_rng(4), 8, 256)
    w8 = dequantize(wire.reshape(-1, 34), T.Q8_0).reshape(8, 256)
    np.savez_compressed(HERE / "q8_0.npz", wire=wire, w=w8.astype(np.float32))

    # ---- q8_0 KV quantise + attention over the dequantised cache
    rng = np.random.default_rng(5)
    kv_heads, s, d, group, pos = 2, 40, 128, 4, 36
    k = (rng.standard_normal((kv_heads, s, d)) * 3).astype(np.float16)
    v = (rng.standard_normal((kv_heads, s, d)) * 3).astype(np.float16)
    k[0, 0, :32] = 0.0                       # all-zero block: scale 0, codes 0
    k[1, 3, 5] = np.float16(2.5)             # plant exact .5 ties: max=127*... see below
    k[1, 3, 32:64] = 0.0
    k[1, 3, 32] = np.float16(127.0)          # max = 127 -> inv = 1 exactly
    k[1, 3, 33] = np.float16(2.5)            # exact half: rounds away from zero -> 3
    k[1, 3, 34] = np.float16(-0.5)           # -> -1
    kc, ks = kvt["_quantize_ref"](k)
    vc, vs = kvt["_quantize_ref"](v)
    dk = kc.astype(np.float32) * np.repeat(ks.astype(np.float32), 32, axis=-1)
    dv = vc.astype(np.float32) * np.repeat(vs.astype(np.float32), 32, axis=-1)
    q = rng.standard_normal((kv_heads * group, d)).astype(np.float16)
    out = kvt["_ref_attention"](dk, dv, q.astype(np.float32), pos, group)
    np.savez_compressed(HERE / "kv_q8.npz", k=k, v=v, k_codes=kc, k_scales=ks, v_codes=vc,
                        v_scales=vs, q=q, pos=np.int64(pos), group=np.int64(group), attn=out)
    # ---- Q5_0: the reference's own wire -> three-buffer split, gguf's decode of the wire blocks
    import torch

    split_ns: dict = {"np": np, "torch": torch}
    tree = ast.parse((ref / "packages/alloy-server/src/alloy_server/gguf/quant.py").read_text())
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "split_q5_0_weight"]
    exec(compile(ast.Module(body=fn, type_ignores=[]), "quant.py", "exec"), split_ns)
    rng = np.random.default_rng(6)
    n5, k5 = 6, 256
    wire5 = rng.integers(0, 256, size=(n5, k5 // 32, 22), dtype=np.uint8)
    wire5[:, :, 0:2] = rng.uniform(1e-4, 2e-3, size=(n5, k5 // 32)).astype(np.float16).view(np.uint8).reshape(
        n5, k5 // 32, 2)
    wire5 = wire5.reshape(n5, -1)
    qw5, qh5, sc5 = split_ns["split_q5_0_weight"](weights=wire5, in_features=k5, out_features=n5)
    w5 = dequantize(wire5.reshape(-1, 22), T.Q5_0).reshape(n5, k5)
    np.savez_compressed(HERE / "q5_0.npz", wire=wire5, qweight=qw5.numpy(), qhigh=qh5.numpy(), scales=sc5.numpy(),
                        w=w5.astype(np.float32))

    # ---- chunk attention over a q8_0 cache (history + chunk both read back from the codes)
    rng = np.random.default_rng(8)
    kv_heads, group, d, start, chunk = 2, 2, 64, 40, 24
    kf = (rng.standard_normal((kv_heads, start + chunk, d)) * 2).astype(np.float16)
    vf = (rng.standard_normal((kv_heads, start + chunk, d)) * 2).astype(np.float16)
    kc, ks = kvt["_quantize_ref"](kf)
    vc, vs = kvt["_quantize_ref"](vf)
    dk = kc.astype(np.float32) * np.repeat(ks.astype(np.float32), 32, axis=-1)
    dv = vc.astype(np.float32) * np.repeat(vs.astype(np.float32), 32, axis=-1)
    qc = rng.standard_normal((kv_heads * group, chunk, d)).astype(np.float16)
    rows = [kvt["_ref_attention"](dk, dv, qc[:, i].astype(np.float32), start + i, group) for i in range(chunk)]
    np.savez_compressed(HERE / "attn_chunk.npz", k=kf, v=vf, q=qc, start=np.int64(start), group=np.int64(group),
                        attn=np.stack(rows, axis=1))
    print("gguf", getattr(gguf, "__version__", "?"), "fixtures written to", HERE)


if __name__ == "__main__":
    main()

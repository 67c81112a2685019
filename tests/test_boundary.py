"""CPU checks of the drop-in boundary: the shared library loads and exports every
symbol the header declares, the op schemas equal the reference's, and host-side
validation behaves like the reference's."""

import os
import pathlib
import re
import sys

import numpy as np
import pytest
import torch

import alloy_b200
from alloy_b200 import _lib, kv, quant, synth

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "alloy_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(alloyb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/alloy_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)
    assert lib.alloyb_version() >= 1
    assert lib.alloyb_error_string(-2).decode().startswith("pointer")


def test_workspace_size_is_pure_arithmetic():
    lib = _lib.load()
    assert lib.alloyb_attn_workspace_bytes(0, 1, 1) == 0
    a = lib.alloyb_attn_workspace_bytes(2, 32, 128)
    assert a % 256 == 0 and a > 2 * 32 * 128 * 4


HOT_OPS = ["gguf_q4_k_mm", "batched_gguf_q4_k_mm", "gguf_q4_k_silu", "gguf_q4_k_gelu",
           "gguf_q4_k_embedding", "gguf_q6_k_mm", "gguf_q6_k_embedding", "batched_gguf_q6_k_mm",
           "gguf_q8_0_embedding", "gguf_q8_0_mm", "batched_gguf_q8_0_mm", "gguf_q8_0_silu",
           "attention_cache", "attention_cache_q8"]


def test_op_schemas_match_reference_source():
    # the reference checkout: ALLOY_REFERENCE, else a sibling "reference" directory of the repo
    root = os.environ.get("ALLOY_REFERENCE") or str(pathlib.Path(__file__).resolve().parents[2] / "reference")
    src = pathlib.Path(root) / "packages/alloy-torch/src/alloy_torch/custom_ops.py"
    if not src.exists():
        pytest.skip("reference checkout not present")
    text = src.read_text()
    defs = {}
    for m in re.finditer(r"_alloy_lib\.define\(\s*((?:\"[^\"]*\"\s*)+)\)", text):
        schema = "".join(re.findall(r"\"([^\"]*)\"", m.group(1)))
        defs[schema.split("(")[0]] = schema
    for name in HOT_OPS:
        ours = str(getattr(torch.ops.alloy, name).default._schema)
        theirs = torch._C.parse_schema("alloy::" + defs[name])
        assert ours == str(theirs), name


def test_ops_have_no_cpu_kernel():
    x = torch.zeros(1, 256, dtype=torch.float16)
    w = torch.zeros(4, 144, dtype=torch.uint8)
    with pytest.raises(NotImplementedError):
        torch.ops.alloy.gguf_q4_k_mm(x, w)
    assert torch.ops.alloy.gguf_q4_k_mm(x.to("meta"), w.to("meta")).shape == (1, 4)
    ids = torch.zeros((2, 3), dtype=torch.int64, device="meta")
    assert torch.ops.alloy.gguf_q6_k_embedding(ids, torch.zeros(4, 420, dtype=torch.uint8, device="meta")
                                               ).shape == (2, 3, 512)
    q = torch.zeros((2, 8, 1, 64), dtype=torch.float16, device="meta")
    assert torch.ops.alloy.attention_cache_q8(q, q, q, q, q, q, q, q).shape == q.shape


def test_validate_quant_buffers_errors():
    blk = torch.zeros((8, 288), dtype=torch.uint8)
    quant.GGUFQ4_KLinear(in_features=512, out_features=8, blocks=blk)
    with pytest.raises(ValueError, match="multiple of 256"):
        quant.GGUFQ4_KLinear(in_features=500, out_features=8, blocks=blk)
    with pytest.raises(ValueError, match="shape"):
        quant.GGUFQ4_KLinear(in_features=512, out_features=9, blocks=blk)
    with pytest.raises(TypeError):
        quant.GGUFQ6_KLinear(in_features=256, out_features=8, qweight=torch.zeros((8, 210), dtype=torch.int8))
    with pytest.raises(ValueError, match="missing"):
        quant.GGUFQ8_0Linear(in_features=64, out_features=8, qweight=torch.zeros((8, 64), dtype=torch.int8))
    with pytest.raises(ValueError, match="unexpected"):
        quant.GGUFQ4_KLinear(in_features=512, out_features=8, blocks=blk, scales=blk)
    assert quant.QUANT_FORMATS["q5_0"].buffer_names == ("qweight", "qhigh", "scales")
    assert quant.QUANT_FORMATS["q6_k"].shapes(8, 512) == {"qweight": (8, 420)}


def test_split_q8_0_weight_matches_oracle():
    from oracle import blocks as O
    wire = synth.q8_0_wire(np.random.default_rng(0), 6, 96)
    q, s = quant.split_q8_0_weight(weights=wire, in_features=96, out_features=6)
    oc, osc = O.split_q8_0(wire)
    assert np.array_equal(q.numpy(), oc) and np.array_equal(s.numpy().view(np.uint16), osc.view(np.uint16))
    with pytest.raises(ValueError):
        quant.split_q8_0_weight(weights=wire, in_features=64, out_features=6)
    with pytest.raises(TypeError):
        quant.split_q8_0_weight(weights=wire.astype(np.int8), in_features=96, out_features=6)


def test_split_q5_0_weight_matches_reference_fixture(golden):
    """The Q5_0 wire split against the buffers the reference's own split_q5_0_weight produced."""
    from oracle import blocks as O
    g = golden["q5_0"]
    n, k = g["w"].shape
    qw, qh, sc = quant.split_q5_0_weight(weights=g["wire"], in_features=k, out_features=n)
    assert np.array_equal(qw.numpy(), g["qweight"]) and np.array_equal(qh.numpy(), g["qhigh"])
    assert np.array_equal(sc.numpy().view(np.uint16), g["scales"].view(np.uint16))
    oq, oh, os_ = O.split_q5_0(g["wire"])
    assert np.array_equal(oq, g["qweight"]) and np.array_equal(oh, g["qhigh"])
    assert np.array_equal(os_.view(np.uint16), g["scales"].view(np.uint16))
    with pytest.raises(ValueError):
        quant.split_q5_0_weight(weights=g["wire"], in_features=k - 32, out_features=n)


REFERENCE = pathlib.Path(os.environ.get("ALLOY_REFERENCE", "/root/reference"))


@pytest.mark.skipif(not (REFERENCE / "packages/alloy-server/src/alloy_server/gguf/quant.py").exists(),
                    reason="needs the rayanht/alloy checkout")
def test_reference_modules_bind_and_run_on_this_op_library():
    """The reference's OWN ``alloy_server/gguf/quant.py`` and ``kv_format.py``, loaded unchanged from the
    checkout, bind every ``torch.ops.alloy.*`` symbol they name at import time and trace through the
    Meta kernels registered here (the device forward of the same ops is what the GPU tests check)."""
    import importlib.util

    def load(rel, name):
        spec = importlib.util.spec_from_file_location(name, REFERENCE / rel)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod           # dataclasses resolve string annotations through sys.modules
        spec.loader.exec_module(mod)
        return mod

    try:
        rq = load("packages/alloy-server/src/alloy_server/gguf/quant.py", "_ref_alloy_quant")
    except ImportError as e:          # a dependency of the reference module that this image lacks
        pytest.skip(f"reference module dependency missing: {e}")
    rk = load("packages/alloy-server/src/alloy_server/kv_format.py", "_ref_alloy_kv_format")
    assert rq.GGUF_Q5_0_MM is torch.ops.alloy.gguf_q5_0_mm.default
    assert set(rq.QUANT_FORMATS) == set(quant.QUANT_FORMATS)
    for name, fmt in rq.QUANT_FORMATS.items():
        mine = quant.QUANT_FORMATS[name]
        assert fmt.align == mine.align and fmt.buffer_names == mine.buffer_names
        assert fmt.mm_op is mine.mm_op and fmt.embed_op is mine.embed_op
        for a, b in zip(fmt.buffers, mine.buffers):
            assert a.dtype is b.dtype and all(a.cols(k) == b.cols(k) for k in (256, 4096, 14336))
    # the reference's modules, built on meta buffers, run through this library's schemas
    lin4 = rq.GGUFQ4_KLinear(in_features=512, out_features=24,
                             blocks=torch.zeros((24, 288), dtype=torch.uint8, device="meta"))
    lin6 = rq.GGUFQ6_KLinear(in_features=512, out_features=24,
                             qweight=torch.zeros((24, 420), dtype=torch.uint8, device="meta"))
    lin8 = rq.GGUFQ8_0Linear(in_features=64, out_features=8,
                             qweight=torch.zeros((8, 64), dtype=torch.int8, device="meta"),
                             scales=torch.zeros((8, 2), dtype=torch.float16, device="meta"))
    x = torch.zeros((2, 3, 512), dtype=torch.float16, device="meta")
    assert lin4(x).shape == (2, 3, 24) and lin6(x).shape == (2, 3, 24) and lin4(x).dtype == torch.float16
    assert lin8(torch.zeros((5, 64), dtype=torch.bfloat16, device="meta")).shape == (5, 8)
    emb = rq.GGUFQ4_KEmbedding(num_embeddings=24, embedding_dim=512,
                               blocks=torch.zeros((24, 288), dtype=torch.uint8, device="meta"))
    ids = torch.zeros((2, 7), dtype=torch.int64, device="meta")
    assert emb(ids).shape == (2, 7, 512) and emb(ids).dtype == torch.float32
    # identical wire splits
    wire = synth.q8_0_wire(np.random.default_rng(1), 4, 64)
    a, b = rq.split_q8_0_weight(weights=wire, in_features=64, out_features=4)
    c, d = quant.split_q8_0_weight(weights=wire, in_features=64, out_features=4)
    assert torch.equal(a, c) and torch.equal(b.view(torch.int16), d.view(torch.int16))
    assert rk.Q8_0 == rk.KV_FORMATS["q8_0"] and rk.Q8_0.name == kv.Q8_0.name
    assert (rk.Q8_0.block_elems, rk.Q8_0.group_tokens, rk.Q8_0.bits_per_elem_k) == \
        (kv.Q8_0.block_elems, kv.Q8_0.group_tokens, kv.Q8_0.bits_per_elem_k)


def test_kv_format_and_page_pool_host_logic():
    assert kv.resolve_kv_format("none") is None and kv.resolve_kv_format("q8_0") is kv.Q8_0
    with pytest.raises(ValueError):
        kv.resolve_kv_format("q4")
    assert kv.Q8_0.scale_count_per_row(128) == 4 and kv.Q8_0.code_bytes_per_row(128) == 128
    pool = kv.PagedKVPool(6, 2, 128, 2, 3, "cpu", free_order=[4, 1, 5, 0, 2, 3])
    assert pool.pool.shape == (6, 2, 2, 16, 136) and pool.bytes_per_token() == 544
    pool.reserve(0, 17)
    pool.reserve(1, 1)
    assert pool.pages_of(0) == [4, 1] and pool.pages_of(1) == [5]
    assert pool.page_table.tolist() == [[4, 1, -1], [5, -1, -1]]
    pool.reserve(0, 33)
    assert pool.pages_of(0) == [4, 1, 0]
    with pytest.raises(ValueError):
        pool.reserve(0, 49)
    pool.release(0)
    assert pool.page_table[0].tolist() == [-1, -1, -1]
    pool.reserve(1, 48)
    assert pool.pages_of(1) == [5, 4, 1]
    pool.reserve(0, 48)
    assert pool.pages_of(0) == [0, 2, 3]
    small = kv.PagedKVPool(2, 2, 128, 1, 3, "cpu")
    with pytest.raises(MemoryError):
        small.reserve(0, 48)

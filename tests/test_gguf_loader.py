"""GGUF file parser and Llama checkpoint mapping (CPU): checked against ``gguf.GGUFReader``, the
reader the reference loads checkpoints with, on a file written by ``gguf.GGUFWriter``."""

import struct

import numpy as np
import pytest
import torch

from alloy_b200 import gguf_loader as GL
from tests._gguf_fixture import TINY_META, permute_rows, write_tiny_llama


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    path = tmp_path_factory.mktemp("gguf") / "tiny-llama.gguf"
    arrays = write_tiny_llama(path, seed=3, tied_head=False)
    return path, arrays


def test_parser_matches_gguf_reader(tiny):
    import gguf
    path, _ = tiny
    ours = GL.read_gguf(path)
    ref = gguf.GGUFReader(str(path))
    assert ours.version == 3 and ours.alignment == 32
    assert set(ours.tensors) == {t.name for t in ref.tensors}
    for t in ref.tensors:
        o = ours.tensors[t.name]
        assert o.ggml_type == int(t.tensor_type)
        assert tuple(reversed([int(x) for x in t.shape])) == o.shape
        assert o.nbytes == int(t.n_bytes)
        assert np.array_equal(o.data, np.asarray(t.data).reshape(-1).view(np.uint8))
    assert ours.metadata["general.architecture"] == "llama"
    for key, field in ref.fields.items():
        if key.startswith("GGUF."):
            continue
        val = field.contents()
        got = ours.metadata[key]
        if isinstance(val, (list, tuple)):
            assert list(got) == list(val)
        elif isinstance(val, float):
            assert got == pytest.approx(val)
        else:
            assert got == val, key


def test_llama_mapping_unpermutes_qk_and_keeps_bytes(tiny):
    path, arrays = tiny
    f = GL.read_gguf(path)
    shape, w = GL.load_llama_weights(f, device="cpu")
    for k, v in TINY_META.items():
        assert getattr(shape, k) == pytest.approx(v)
    assert not w.tied_head and w.head.fmt == "q6_k" and w.embed.fmt == "q4_k"
    assert np.array_equal(w.embed.tensor.numpy(), arrays["embed"][1])
    assert np.array_equal(w.head.tensor.numpy(), arrays["head"][1])
    for i, lay in enumerate(arrays["layers"]):
        got = w.layers[i]
        for name in ("wq", "wk", "wv", "wo", "wg", "wu", "wd"):
            assert got[name].fmt == lay[name][0], (i, name)
            assert np.array_equal(got[name].tensor.numpy(), lay[name][1]), (i, name)   # q/k back in rotate-half order
        assert np.allclose(got["norm_in"].tensor.float().numpy(), lay["norm_in"], atol=1e-3)
    # the inverse of the checkpoint permutation, on its own
    rows = np.arange(64 * 3, dtype=np.uint8).reshape(64, 3)
    back = GL.unpermute_qk_rows(torch.from_numpy(permute_rows(rows, 4)), 4).numpy()
    assert np.array_equal(back, rows)


def test_tied_head_and_errors(tmp_path):
    path = tmp_path / "tied.gguf"
    write_tiny_llama(path, seed=4, tied_head=True)
    f = GL.read_gguf(path)
    _, w = GL.load_llama_weights(f, device="cpu")
    assert w.tied_head and w.head.tensor is w.embed.tensor
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + bytes(40))
    with pytest.raises(GL.GGUFError):
        GL.read_gguf(bad)
    raw = bytearray(path.read_bytes())
    struct.pack_into("<I", raw, 4, 1)                       # version 1
    old = tmp_path / "v1.gguf"
    old.write_bytes(bytes(raw))
    with pytest.raises(GL.GGUFError):
        GL.read_gguf(old)
    trunc = tmp_path / "trunc.gguf"
    trunc.write_bytes(path.read_bytes()[:-1000])
    with pytest.raises(GL.GGUFError):
        GL.read_gguf(trunc)
    f.metadata["general.architecture"] = "qwen2"
    with pytest.raises(GL.GGUFError):
        GL.llama_shape(f.metadata, f.tensors)

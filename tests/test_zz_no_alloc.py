"""The allocation-free decode-attention entry point against the workspace-taking one.

Hosts that may not allocate device memory on the decode path (a serving loop with a frozen
memory plan, a plugin whose host forbids allocation after start-up) call
``alloyb_attn_decode_static``, which keeps its split-K partials in a fixed device array inside
the library.  It must give what ``alloyb_attn_decode`` gives with a caller workspace -- checked
here through the C ABI on two calls in a row (the array is shared and keeps the first call's
contents), for two shapes, plus the size limit.  Collected last on purpose.
"""

import numpy as np
import pytest
import torch

from alloy_b200 import _lib, synth
from oracle import blocks as O
from tests._util import assert_close, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(seed, b, kv_h, group, d, s_max, pos):
    rng = np.random.default_rng(seed)
    h = kv_h * group
    kc, ks = O.kv_quantize_q8_0(synth.kv_rows(rng, (b, kv_h, s_max, d)))
    vc, vs = O.kv_quantize_q8_0(synth.kv_rows(rng, (b, kv_h, s_max, d)))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return dict(b=b, h=h, kv_h=kv_h, d=d, s_max=s_max,
                q=dev(synth.activations(rng, b * h, d).reshape(b, h, d)),
                nk=dev(synth.kv_rows(rng, (b, kv_h, d))), nv=dev(synth.kv_rows(rng, (b, kv_h, d))),
                pos=torch.tensor([pos], dtype=torch.int32, device=DEV),
                cache=[dev(kc), dev(ks), dev(vc), dev(vs)], host=(kc, ks, vc, vs), pos_i=pos)


def _call(L, c, static, cache, out):
    st = torch.cuda.current_stream().cuda_stream
    head = (_lib.KV_Q8_SPLIT, c["q"].data_ptr(), c["q"].stride(0), c["q"].stride(1), _lib.F16,
            cache[0].data_ptr(), cache[1].data_ptr(), cache[2].data_ptr(), cache[3].data_ptr(),
            c["nk"].data_ptr(), c["nv"].data_ptr(), c["nk"].stride(0), c["nk"].stride(1),
            c["pos"].data_ptr(), 1, out.data_ptr(), c["b"], c["h"], c["kv_h"], c["d"], c["s_max"], 0,
            -1.0, 1)
    if static:
        return L.alloyb_attn_decode_static(*head, st)
    n = L.alloyb_attn_workspace_bytes(c["b"], c["h"], c["d"])
    ws = torch.empty(n, dtype=torch.uint8, device=DEV)
    _lib.check(L.alloyb_attn_workspace_init(ws.data_ptr(), n, c["b"], c["h"], st), "ws init")
    rc = L.alloyb_attn_decode(*head, ws.data_ptr(), n, st)
    torch.cuda.synchronize()
    return rc


def test_static_entry_matches_workspace_entry_twice():
    L = _lib.load()
    cases = [_case(1, 2, 2, 4, 128, 640, 517), _case(2, 3, 8, 4, 128, 256, 199)]
    for rep in range(2):                      # two calls in a row per shape, shapes interleaved
        for c in cases:
            ref_cache = [t.clone() for t in c["cache"]]
            got_cache = [t.clone() for t in c["cache"]]
            ref = torch.zeros((c["b"], c["h"], c["d"]), dtype=torch.float16, device=DEV)
            got = torch.full_like(ref, 7.0)
            _lib.check(_call(L, c, False, ref_cache, ref), "alloyb_attn_decode")
            _lib.check(_call(L, c, True, got_cache, got), "alloyb_attn_decode_static")
            torch.cuda.synchronize()
            assert_close(to_np(got), to_np(ref).astype(np.float64), torch.float16, f"static rep {rep}")
            for a, b_ in zip(got_cache, ref_cache):        # the fused append wrote the same bytes
                assert torch.equal(a, b_)
            # and both agree with the oracle
            kc, ks, vc, vs = (x.cpu().numpy() for x in got_cache)
            dk, dv = O.kv_dequant_q8_0(kc, ks), O.kv_dequant_q8_0(vc, vs)
            q = c["q"].cpu().numpy()
            want = np.stack([O.attention_decode_ref(dk[i], dv[i], q[i], c["pos_i"]) for i in range(c["b"])])
            assert_close(to_np(got), want, torch.float16, "static vs oracle")


def test_static_entry_rejects_oversize():
    L = _lib.load()
    c = _case(3, 1, 1, 1, 128, 128, 5)
    big_b, big_h = 64, 64                     # needs far more than the fixed array holds
    assert L.alloyb_attn_workspace_bytes(big_b, big_h, 128) > 16 * 1024 * 1024
    out = torch.zeros((1, 1, 128), dtype=torch.float16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    rc = L.alloyb_attn_decode_static(
        _lib.KV_Q8_SPLIT, c["q"].data_ptr(), 128, 128, _lib.F16, c["cache"][0].data_ptr(),
        c["cache"][1].data_ptr(), c["cache"][2].data_ptr(), c["cache"][3].data_ptr(),
        c["nk"].data_ptr(), c["nv"].data_ptr(), 128, 128, c["pos"].data_ptr(), 1, out.data_ptr(),
        big_b, big_h, 1, 128, 128, 0, -1.0, 0, st)
    assert rc == -8
    assert b"maximum" in L.alloyb_error_string(rc)

"""Llama-shape quantised decode step on the ``torch.ops.alloy`` surface.

A thin harness, not a model zoo: it strings the hot-path ops together the way
the reference's patched HF Llama forward does
(``packages/alloy-server/src/alloy_server/models/attention.py:845-886`` for the
attention block, ``packages/alloy-server/src/alloy_server/generation/decode.py:22-61``
for the greedy next-token head) with the Q4_K_M tensor-type mix: Q4_K for
q/k/o/gate/up and the token embedding, Q6_K for v/down and the output head.
One decode step can be captured in a CUDA graph and replayed.

Tensor parallelism (``tp_rank``/``tp_size``): q/k/v/gate/up and the head are
split by output rows, o_proj/down by input columns on super-block boundaries;
the row-parallel partial outputs are summed by ``all_reduce`` (NCCL) before the
residual add.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops, synth, tp


@dataclass(frozen=True)
class LlamaShape:
    layers: int
    hidden: int
    ffn: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    rope_theta: float = 500000.0
    eps: float = 1e-5

    def weight_bytes(self) -> int:
        """Packed bytes one decode step streams: every linear once, norms, no embedding table."""
        q4 = lambda n, k: n * (k // 256) * 144
        q6 = lambda n, k: n * (k // 256) * 210
        hd = self.heads * self.head_dim
        kvd = self.kv_heads * self.head_dim
        layer = (q4(hd, self.hidden) + q4(kvd, self.hidden) + q6(kvd, self.hidden) +
                 q4(self.hidden, hd) + 2 * q4(self.ffn, self.hidden) + q6(self.hidden, self.ffn))
        norms = (2 * self.layers + 1) * self.hidden * 2
        return layer * self.layers + q6(self.vocab, self.hidden) + norms

    def layer_weight_elems(self) -> int:
        """Weights of the per-layer linears (what every prompt token is multiplied by in prefill)."""
        hd = self.heads * self.head_dim
        kvd = self.kv_heads * self.head_dim
        return self.layers * (hd * self.hidden + 2 * kvd * self.hidden + self.hidden * hd + 3 * self.ffn * self.hidden)


LLAMA3_8B = LlamaShape(layers=32, hidden=4096, ffn=14336, heads=32, kv_heads=8, head_dim=128,
                       vocab=128256)
LLAMA3_70B = LlamaShape(layers=80, hidden=8192, ffn=28672, heads=64, kv_heads=8, head_dim=128,
                        vocab=128256)


class LayerWeights:
    __slots__ = ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "norm_in", "norm_post", "fmt")

    def __init__(self) -> None:
        # format name of every matrix (Q4_K_M: Q4_K for q/k/o/gate/up, Q6_K for v/down)
        self.fmt = {"wq": "q4_k", "wk": "q4_k", "wv": "q6_k", "wo": "q4_k", "wg": "q4_k", "wu": "q4_k", "wd": "q6_k"}



_FMT_CODE = {"q4_k": 0, "q6_k": 1}


class _FusedStep:
    """The decoder's layers handed to ``alloyb_decoder_create``: one persistent launch per step."""

    def __init__(self, dec: "QuantLlamaDecoder") -> None:
        import ctypes as C

        from . import _lib
        from ._lib import DecoderDesc, DecoderLayer, Matrix

        s = dec.shape
        self._L = L = _lib.load()
        dev = dec.device
        self.hidden = torch.zeros(s.hidden, dtype=torch.float16, device=dev)
        self.logits = torch.zeros(dec.vocab_l, dtype=torch.float16, device=dev)

        def mat(w: torch.Tensor, fmt: str) -> Matrix:
            if fmt not in _FMT_CODE:
                raise ValueError(f"format {fmt} is outside the one-launch step")
            if w.stride(1) != 1:
                raise ValueError("packed rows must have unit inner stride")
            pitch = 0 if w.stride(0) == w.shape[1] else w.stride(0)
            return Matrix(_FMT_CODE[fmt], w.shape[0], w.data_ptr(), pitch)

        layers = (DecoderLayer * len(dec.layers))()
        paged = dec.kv_kind == "q8_paged"
        for li, lw in enumerate(dec.layers):
            if paged:
                pool = dec.pools[li]
                k0, k1, v0, v1 = pool.pool.data_ptr(), pool.page_table.data_ptr(), None, None
            else:
                k0, k1, v0, v1 = dec.k_cache[li].data_ptr(), None, dec.v_cache[li].data_ptr(), None
            layers[li] = DecoderLayer(mat(lw.wq, lw.fmt["wq"]), mat(lw.wk, lw.fmt["wk"]), mat(lw.wv, lw.fmt["wv"]),
                                      mat(lw.wo, lw.fmt["wo"]), mat(lw.wg, lw.fmt["wg"]), mat(lw.wu, lw.fmt["wu"]),
                                      mat(lw.wd, lw.fmt["wd"]), lw.norm_in.data_ptr(), lw.norm_post.data_ptr(),
                                      k0, k1, v0, v1)
        self._layers = layers
        if paged:
            s_max, n_pages = dec.pools[0].page_table.shape[1] * 16, dec.pools[0].pool.shape[0]
        else:
            s_max, n_pages = dec.k_cache[0].shape[2], 0
        ex = dec.exchange
        desc = DecoderDesc(len(dec.layers), s.hidden, dec.ffn_l, dec.heads_l, dec.kv_heads_l, s.head_dim, s.eps,
                           _lib.KV_Q8_PAGED if paged else _lib.KV_F16, s_max, n_pages, layers,
                           dec.norm_final.data_ptr(), mat(dec.head, dec.head_fmt), dec.inv_freq.data_ptr(),
                           dec.pos.data_ptr(), self.hidden.data_ptr(), self.logits.data_ptr(),
                           C.pointer(ex.desc) if ex is not None and ex.world > 1 else None)
        self._handle = C.c_void_p()
        _lib.check(L.alloyb_decoder_create(C.byref(desc), C.byref(self._handle)), "alloyb_decoder_create")
        self.phases = int(L.alloyb_decoder_phases(self._handle))

    def step(self) -> None:
        from . import _lib
        _lib.check(self._L.alloyb_decoder_step(self._handle, ops._stream()), "alloyb_decoder_step")

    def close(self) -> None:
        if self._handle:
            self._L.alloyb_decoder_destroy(self._handle)
            self._handle = None


class QuantLlamaDecoder:
    """Q4_K_M Llama-shape decoder for one decode step per call: random-init (seeded) weights, or
    the tensors of a GGUF checkpoint (``weights``: ``gguf_loader.LlamaWeights``, unsharded)."""

    def __init__(self, shape: LlamaShape, batch: int, context: int, *, device="cuda", seed: int = 0,
                 kv: str = "f16", tp_rank: int = 0, tp_size: int = 1, process_group=None,
                 dtype: torch.dtype = torch.float16, d_scale: float = 1.0, centered: bool = False, peer_allreduce: bool = True,
                 tp_dry: bool = False, weights=None, one_launch: bool | None = None,
                 fused_attention: bool = True) -> None:
        if kv not in ("f16", "q8_paged"):
            raise ValueError(f"kv must be 'f16' or 'q8_paged', got {kv!r}")
        if shape.heads % tp_size or shape.kv_heads % tp_size or shape.ffn % (256 * tp_size) \
                or (shape.heads * shape.head_dim) % (256 * tp_size) or shape.vocab % tp_size:
            raise ValueError(f"shape does not shard {tp_size} ways")
        self.shape, self.batch, self.context = shape, int(batch), int(context)
        self.fused_attention = bool(fused_attention)
        self.device, self.dtype, self.kv_kind = torch.device(device), dtype, kv
        self.tp_rank, self.tp_size, self.pg = tp_rank, tp_size, process_group
        # row-parallel outputs are summed inside the GEMV launch over peer memory (NCCL only sets
        # it up and serves the shapes the fused kernel does not cover)
        # tp_dry: this rank's share of the step with nobody to exchange with (sums are the local
        # partials): what one rank of a TP-N step computes, for profiling under tools that cannot
        # wrap a multi-rank run
        self.exchange = None
        self.exchange_error = None
        self.tp_dry = bool(tp_dry)
        if tp_dry:
            self.exchange = tp.PeerExchange(shape.hidden)
        elif tp_size > 1 and peer_allreduce and self.device.type == "cuda" and dtype == torch.float16:
            # every rank must end up on the same path: if mapping the peers' buffers fails anywhere
            # (no peer access between two of the GPUs, IPC not permitted), all ranks use NCCL
            try:
                ex = tp.PeerExchange(shape.hidden, tp_rank, tp_size, process_group, self.device)
            except Exception as e:  # noqa: BLE001 - any set-up failure means "no peer path"
                ex = None
                self.exchange_error = repr(e)
            if tp.agree(ex is not None, process_group, self.device):
                self.exchange = ex
            elif ex is not None:
                ex.close()
        s = shape
        self.heads_l = s.heads // tp_size
        self.kv_heads_l = s.kv_heads // tp_size
        self.ffn_l = s.ffn // tp_size
        self.vocab_l = s.vocab // tp_size
        hd_l, kvd_l = self.heads_l * s.head_dim, self.kv_heads_l * s.head_dim

        # every rank draws the FULL matrices from the same seed and keeps its shard, so the
        # sharded model equals the unsharded one by construction
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed)
        r, n = tp_rank, tp_size

        def rows(t, per):
            return tp.shard_rows(t, r, n)

        self.embed_fmt, self.head_fmt = "q4_k", "q6_k"
        self.layers: list[LayerWeights] = []
        if weights is not None:
            # checkpoint tensors: same sharding as the synthetic model
            self.embed, self.embed_fmt = weights.embed.tensor, weights.embed.fmt
            for lsrc in weights.layers:
                lw = LayerWeights()
                lw.fmt = {k: lsrc[k].fmt for k in lw.fmt}
                lw.wq, lw.wk, lw.wv = (rows(lsrc[k].tensor, 0) for k in ("wq", "wk", "wv"))
                lw.wg, lw.wu = rows(lsrc["wg"].tensor, 0), rows(lsrc["wu"].tensor, 0)
                lw.wo = tp.shard_cols(lsrc["wo"].tensor, lw.fmt["wo"], r, n)
                lw.wd = tp.shard_cols(lsrc["wd"].tensor, lw.fmt["wd"], r, n)
                lw.norm_in, lw.norm_post = lsrc["norm_in"].tensor, lsrc["norm_post"].tensor
                self.layers.append(lw)
            self.norm_final = weights.norm_final.tensor
            self.head, self.head_fmt = rows(weights.head.tensor, 0), weights.head.fmt
        else:
            ctr = {"centered": centered}   # zero-mean Q4_K weights keep a deep random stack inside fp16
            self.embed = synth.q4k_blocks_device(s.vocab, s.hidden, gen, self.device, d_scale, **ctr)
            for _ in range(s.layers):
                lw = LayerWeights()
                lw.wq = rows(synth.q4k_blocks_device(s.heads * s.head_dim, s.hidden, gen, self.device, d_scale, **ctr), hd_l)
                lw.wk = rows(synth.q4k_blocks_device(s.kv_heads * s.head_dim, s.hidden, gen, self.device, d_scale, **ctr), kvd_l)
                lw.wv = rows(synth.q6k_blocks_device(s.kv_heads * s.head_dim, s.hidden, gen, self.device, d_scale), kvd_l)
                lw.wo = tp.shard_cols(synth.q4k_blocks_device(s.hidden, s.heads * s.head_dim, gen, self.device, d_scale, **ctr), "q4_k", r, n)
                lw.wg = rows(synth.q4k_blocks_device(s.ffn, s.hidden, gen, self.device, d_scale, **ctr), self.ffn_l)
                lw.wu = rows(synth.q4k_blocks_device(s.ffn, s.hidden, gen, self.device, d_scale, **ctr), self.ffn_l)
                lw.wd = tp.shard_cols(synth.q6k_blocks_device(s.hidden, s.ffn, gen, self.device, d_scale), "q6_k", r, n)
                lw.norm_in = self._norm_weight(gen)
                lw.norm_post = self._norm_weight(gen)
                self.layers.append(lw)
            self.norm_final = self._norm_weight(gen)
            self.head = rows(synth.q6k_blocks_device(s.vocab, s.hidden, gen, self.device, d_scale), self.vocab_l)
        # q and k of a layer share a format: their packed rows are kept back to back in ONE buffer (wq and wk are
        # views of it), which lets the library run the two projections of several tokens as a single GEMM
        for lw in self.layers:
            if lw.fmt["wq"] == lw.fmt["wk"] and lw.wq.shape[1:] == lw.wk.shape[1:] and lw.wq.dtype == lw.wk.dtype:
                nq = lw.wq.shape[0]
                qk = torch.cat([lw.wq, lw.wk], 0)
                lw.wq, lw.wk = qk[:nq], qk[nq:]
        self.inv_freq = (1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, dtype=torch.float32) /
                                                 s.head_dim))).to(self.device)
        self._init_kv(gen)
        # static step inputs/outputs (CUDA-graph friendly)
        self.ids = torch.zeros(self.batch, dtype=torch.int64, device=self.device)
        self.pos = torch.full((1,), self.context - 1, dtype=torch.int32, device=self.device)
        self.seq_pos = torch.full((self.batch,), self.context - 1, dtype=torch.int32, device=self.device)
        self.next_ids = torch.zeros(self.batch, dtype=torch.int64, device=self.device)
        self.logits: torch.Tensor | None = None
        self._graph: torch.cuda.CUDAGraph | None = None
        self.launches_per_step = 0
        # One sequence: the whole step runs as one persistent launch (``alloyb_decoder_step``) when the
        # shape is inside what that kernel is built for; ``one_launch=False`` keeps the op-by-op step.
        self._fused = None
        self.one_launch_error = None
        want = bool(one_launch)
        if want and self.batch == 1 and self.device.type == "cuda" and dtype == torch.float16 and \
                (tp_size == 1 or tp_dry or self.exchange is not None):
            try:
                self._fused = _FusedStep(self)
            except Exception as e:  # noqa: BLE001 - outside the kernel's shapes: the op-by-op step serves it
                self.one_launch_error = repr(e)
                if one_launch:
                    raise
        if tp_size > 1 and not tp_dry:
            # every rank runs the same kind of step
            if not tp.agree(self._fused is not None, process_group, self.device) and self._fused is not None:
                self._fused.close()
                self._fused = None

    def _norm_weight(self, gen) -> torch.Tensor:
        w = torch.empty(self.shape.hidden, dtype=torch.float32, device=self.device)
        w.normal_(0.0, 0.02, generator=gen).add_(1.0)
        return w.to(self.dtype)

    def _init_kv(self, gen) -> None:
        s, b, ctx = self.shape, self.batch, self.context
        full = (b, s.kv_heads, ctx, s.head_dim)
        lo, hi = self.tp_rank * self.kv_heads_l, (self.tp_rank + 1) * self.kv_heads_l
        self.k_cache, self.v_cache, self.pools = [], [], []
        if self.kv_kind == "f16":
            for _ in range(s.layers):
                k = torch.empty(full, dtype=torch.float32, device=self.device).normal_(generator=gen)
                v = torch.empty(full, dtype=torch.float32, device=self.device).normal_(generator=gen)
                self.k_cache.append(k[:, lo:hi].to(torch.float16).contiguous())
                self.v_cache.append(v[:, lo:hi].to(torch.float16).contiguous())
                del k, v
        else:
            from .kv import PagedKVPool
            pages_per = (ctx + 15) // 16
            total = b * pages_per
            order = torch.randperm(total, generator=torch.Generator().manual_seed(1234)).tolist()
            table = None
            for _ in range(s.layers):
                pool = PagedKVPool(total, self.kv_heads_l, s.head_dim, b, pages_per, self.device,
                                   page_table=table, free_order=order)
                if table is None:
                    for i in range(b):
                        pool.reserve(i, ctx)
                    table = pool.page_table
                # random codes, scales ~ |N(0,1)| max / 127 magnitude
                pool.pool.copy_(torch.randint(0, 256, pool.pool.shape, dtype=torch.uint8,
                                              device=self.device, generator=gen))
                blocks = pool.pool.view(-1, 34)
                sc = torch.empty(blocks.shape[0], dtype=torch.float32, device=self.device).uniform_(
                    0.015, 0.03, generator=gen).to(torch.float16)
                blocks[:, 0:2] = sc.view(torch.uint8).view(-1, 2)
                self.pools.append(pool)

    def _row_parallel(self, x, fmt, w, h):
        """h + sum over ranks of x_r W_r^T: inside the GEMV launch over peer memory when the
        fused kernel covers the shape, else the plain linear + NCCL all-reduce."""
        if self.exchange is not None:
            y = ops.linear_allreduce(x, fmt, w, h, self.exchange)
            if y is not None:
                self.fused_allreduce_calls += 1
                return y
        mm = torch.ops.alloy.gguf_q4_k_mm if fmt == "q4_k" else torch.ops.alloy.gguf_q6_k_mm
        return h + tp.row_parallel(x, lambda t: mm(t, w), self.pg)

    # ------------------------------------------------------------------ one decode step

    def step_eager_logits(self) -> torch.Tensor:
        """One eager (uncaptured) step; returns the logits."""
        self._enter_together()
        self._step()
        return self.logits

    def _enter_together(self) -> None:
        """Tensor-parallel ranks start an eager step together: a rank still busy elsewhere would let
        its peers' bounded waits in the fused exchange run out."""
        if self.tp_size > 1 and not self.tp_dry:
            torch.cuda.synchronize()
            torch.distributed.barrier(group=self.pg)

    def device_error(self, clear: bool = True) -> int:
        """The library's sticky device error word (non-zero: a bounded wait ran out somewhere since
        it was last cleared, results since then are not to be trusted).  Synchronises the device."""
        from . import _lib
        return int(_lib.load().alloyb_device_error(1 if clear else 0))

    def _step(self) -> None:
        s, b = self.shape, self.batch
        n0 = ops.launch_count()
        self.fused_allreduce_calls = 0
        if self._fused is not None:
            fs = self._fused
            ops._embedding(self.ids, ops._FORMATS[self.embed_fmt], self.embed, None, out=fs.hidden)
            fs.step()
            logits = fs.logits.view(1, -1)
            if self.tp_size > 1 and not self.tp_dry:
                logits = tp.gather_columns(logits, self.pg)
            self.logits = logits
            ops.argmax(logits, out=self.next_ids)
            self.launches_per_step = ops.launch_count() - n0
            return
        h = ops._embedding(self.ids, ops._FORMATS[self.embed_fmt], self.embed, None, out_dtype=self.dtype)
        scale = 1.0 / (s.head_dim ** 0.5)
        for li, lw in enumerate(self.layers):
            # q/k (Q4_K) and v (Q6_K) of one token run as ONE streaming launch that also applies the input
            # RMSNorm (several tokens: the norm, then the projections)
            q, k, v = ops.linear_multi(h, [(lw.fmt["wq"], lw.wq, None), (lw.fmt["wk"], lw.wk, None),
                                           (lw.fmt["wv"], lw.wv, None)], norm=(lw.norm_in, s.eps))
            q3 = q.view(b, self.heads_l, s.head_dim)
            k3 = k.view(b, self.kv_heads_l, s.head_dim)
            v3 = v.view(b, self.kv_heads_l, s.head_dim)
            # RoPE of q and k, the cache append and the attention in one launch (or, on request, RoPE +
            # append as a launch of their own before an attention that only reads)
            kv_args = (dict(k_cache=self.k_cache[li], v_cache=self.v_cache[li]) if self.kv_kind == "f16"
                       else dict(paged=(self.pools[li].page_table, self.pools[li].pool)))
            p_arg = self.pos if self.kv_kind == "f16" else self.seq_pos
            if self.fused_attention:
                a = ops.rope_attention_decode(q3, k3, v3, p_arg, self.inv_freq, scale=scale, **kv_args)
            else:
                ops.rope_kv_append(q3, k3, v3, p_arg, self.inv_freq, **kv_args)
                q4, k4, v4 = q3.unsqueeze(2), k3.unsqueeze(2), v3.unsqueeze(2)
                if self.kv_kind == "f16":
                    a = torch.ops.alloy.attention_cache(q4, k4, v4, self.pos, self.k_cache[li], self.v_cache[li],
                                                        scale, 0, False)
                else:
                    a = torch.ops.alloy.attention_cache_q8_paged(q4, k4, v4, self.seq_pos, self.pools[li].page_table,
                                                                 self.pools[li].pool, -1.0, False)
                a = a.transpose(1, 2)
            a2 = a.reshape(b, self.heads_l * s.head_dim)
            if self.tp_size == 1:
                h = torch.ops.alloy.linear_residual(a2, lw.wo, None, h, lw.fmt["wo"])
            else:
                h = self._row_parallel(a2, lw.fmt["wo"], lw.wo, h)
            if lw.fmt["wg"] == "q4_k" and lw.fmt["wu"] == "q4_k":
                act = ops.gated_normed(h, lw.norm_post, s.eps, lw.wg, lw.wu)
            else:
                gate, up = ops.linear_multi(h, [(lw.fmt["wg"], lw.wg, None), (lw.fmt["wu"], lw.wu, None)],
                                            norm=(lw.norm_post, s.eps))
                act = ops.silu_mul(gate, up)
            if self.tp_size == 1:
                h = torch.ops.alloy.linear_residual(act, lw.wd, None, h, lw.fmt["wd"])
            else:
                h = self._row_parallel(act, lw.fmt["wd"], lw.wd, h)
        logits = ops.linear_multi(h, [(self.head_fmt, self.head, None)], norm=(self.norm_final, s.eps))[0]
        if self.tp_size > 1 and not self.tp_dry:
            logits = tp.gather_columns(logits, self.pg)
        self.logits = logits
        ops.argmax(logits, out=self.next_ids)
        self.launches_per_step = ops.launch_count() - n0

    # ------------------------------------------------------------------ prefill

    def prefill(self, ids: torch.Tensor, start: int = 0) -> torch.Tensor:
        """Run ``ids`` (B, S) through the model as ONE chunk at positions ``start .. start + S - 1``: the
        linears see B * S tokens at once (tensor-core GEMM from 28 tokens up), every layer writes its S
        new K / V rows per sequence to the cache (quantised for the q8 pool) and attends causally over
        the cache (``attention_cache*`` with ``seq_len > 1``).  Returns the logits of each sequence's
        last token (B, vocab) and leaves ``pos`` at ``start + S``, so ``step()`` continues from there --
        the prefill half of the reference's serving loop (model forward over the prompt chunk,
        ``server/models/attention.py:281-342``)."""
        s, b = self.shape, self.batch
        if ids.ndim != 2 or ids.shape[0] != b:
            raise ValueError(f"ids must be ({b}, S), got {tuple(ids.shape)}")
        n = int(ids.shape[1])
        if n < 1 or start < 0 or start + n > self.context:
            raise ValueError(f"positions {start}..{start + n - 1} do not fit a cache of {self.context}")
        if self._graph is not None:
            raise RuntimeError("prefill runs eagerly: call it before capture()")
        dev = self.device
        m = b * n
        x = ops._embedding(ids.to(dev).reshape(-1), ops._FORMATS[self.embed_fmt], self.embed, None, out_dtype=self.dtype)
        rows_pos = (start + torch.arange(n, dtype=torch.int32, device=dev)).repeat(b)       # position of token row
        start_t = torch.full((b,), start, dtype=torch.int32, device=dev)
        scale = 1.0 / (s.head_dim ** 0.5)
        self._enter_together()
        for li, lw in enumerate(self.layers):
            xn = ops.rms_norm(x, lw.norm_in, s.eps)
            q, k, v = ops.linear_multi(xn, [(lw.fmt["wq"], lw.wq, None), (lw.fmt["wk"], lw.wk, None),
                                            (lw.fmt["wv"], lw.wv, None)])
            q3 = q.view(m, self.heads_l, s.head_dim)
            k3 = k.view(m, self.kv_heads_l, s.head_dim)
            ops.rope_inplace(q3, k3, rows_pos, self.inv_freq)
            q4 = q3.view(b, n, self.heads_l, s.head_dim).transpose(1, 2)
            k4 = k3.view(b, n, self.kv_heads_l, s.head_dim).transpose(1, 2)
            v4 = v.view(b, n, self.kv_heads_l, s.head_dim).transpose(1, 2)
            if self.kv_kind == "f16":
                a = torch.ops.alloy.attention_cache(q4, k4, v4, start_t[:1], self.k_cache[li], self.v_cache[li],
                                                    scale, 0, True)
            else:
                pool = self.pools[li]
                a = torch.ops.alloy.attention_cache_q8_paged(q4, k4, v4, start_t, pool.page_table, pool.pool, -1.0, True)
            a2 = a.transpose(1, 2).reshape(m, self.heads_l * s.head_dim)
            if self.tp_size == 1:
                x = torch.ops.alloy.linear_residual(a2, lw.wo, None, x, lw.fmt["wo"])
            else:
                x = self._row_parallel(a2, lw.fmt["wo"], lw.wo, x)
            xn = ops.rms_norm(x, lw.norm_post, s.eps)
            if lw.fmt["wg"] == "q4_k" and lw.fmt["wu"] == "q4_k":
                act = torch.ops.alloy.gguf_q4_k_silu(xn, lw.wg, lw.wu)
            else:
                gate, up = ops.linear_multi(xn, [(lw.fmt["wg"], lw.wg, None), (lw.fmt["wu"], lw.wu, None)])
                act = ops.silu_mul(gate, up)
            if self.tp_size == 1:
                x = torch.ops.alloy.linear_residual(act, lw.wd, None, x, lw.fmt["wd"])
            else:
                x = self._row_parallel(act, lw.fmt["wd"], lw.wd, x)
        last = x.view(b, n, s.hidden)[:, -1].contiguous()
        logits = ops.linear_multi(last, [(self.head_fmt, self.head, None)], norm=(self.norm_final, s.eps))[0]
        if self.tp_size > 1 and not self.tp_dry:
            logits = tp.gather_columns(logits, self.pg)
        self.logits = logits
        ops.argmax(logits, out=self.next_ids)
        self.pos.fill_(start + n)
        if hasattr(self, "seq_pos"):
            self.seq_pos.fill_(start + n)
        return logits

    def capture(self) -> None:
        """Warm up once eagerly, then record the step into a CUDA graph."""
        # the ranks enter their first exchange together (a rank still building its weights
        # would let the others' bounded waits run out)
        self._enter_together()
        self._step()
        torch.cuda.synchronize()
        if self.tp_size > 1 and not self.tp_dry and self.exchange is not None:
            # did any rank's wait on a peer run out?  Then nobody uses the peer path.
            if not tp.agree(self.device_error() == 0, self.pg, self.device):
                self.exchange_error = "a bounded wait on a peer ran out in the first step; using NCCL all-reduces"
                self.exchange.close()
                self.exchange = None
                self._enter_together()
                self._step()
                torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._step()
        self._graph = g

    def step(self) -> torch.Tensor:
        """Run one decode step on ``self.ids`` at ``self.pos``; returns ``self.next_ids``."""
        if self._graph is not None:
            self._graph.replay()
        else:
            self._step()
        return self.next_ids

"""Causal grouped-query attention over the paged cache, as a mixer part.

One fused q/k/v projection (the three matrices are stacked at load time into one
``[(H + 2K) * head_dim, hidden]`` matrix), then bias, per-head RMSNorm of q and k, rotation and the
cache write in one kernel, then attention over the cache, then the output projection added into
the residual stream. Formulas and their order: sleuth/forge/model/attention.py:101-157 (projections
:106-108, QK-norm before RoPE :121-126, cache update :129-130, scale 1/sqrt(head_dim) :84, GQA
head mapping :197-199, window mask :160-169, output projection without bias :155-157).

With ``reads_shared_kv`` the part has no k/v projections and reads the cache entry another layer
application wrote.

Options that another design may set (``AttentionSpec``): values of another width than the keys (``value_dim``), one
RMSNorm over the whole q projection and one over the whole k projection instead of one per head
(``qk_norm_span="projection"``), rotation of neighbouring channels (the position's ``pairing``), and a learned sink per
head in the softmax denominator (``sinks``). Any of the first three sends a step through the *wide* form: the stacked
projection with a float32 result, ``qkv_post_span`` (norms, rotation, cache write) and the attention kernel.
"""

from __future__ import annotations

import math
import os

import torch

from ..cache.paged import KVRequest
from ..kernels import ops
from .base import BuildContext, ParamDecl, Part, build_position, register_mixer
from .base import Normed
from .linear import Linear, use_tc
from .spec import AttentionSpec


# Which kernel serves a step that brings several tokens per sequence: "auto" takes the tcgen05 kernel once a
# sequence fills at least one of its 128-row tiles, "mma" always the mma.sync kernel, "tc" the tcgen05 kernel
# whenever it takes the shape.
ATTENTION_CHOICE = os.environ.get("SLEUTH_B200_ATTENTION", "auto")


def use_tc_attention(heads: int, kv_heads: int, head_dim: int, dtype, max_count: int, scale: float = 1.0) -> bool:
    if ATTENTION_CHOICE == "mma" or scale <= 0 or not ops.attention_tc_supported(heads, kv_heads, head_dim, dtype):
        return False
    return ATTENTION_CHOICE == "tc" or max_count * (heads // kv_heads) >= 128


class GQAAttention(Part):
    accepts_normed = True

    def __init__(self, spec: AttentionSpec, ctx: BuildContext):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads ({spec.heads}) must be a multiple of kv_heads ({spec.kv_heads})")
        if spec.head_dim % 2 or spec.head_dim > 256:
            raise ValueError(f"head_dim {spec.head_dim} is not supported: it must be even and at most 256")
        if spec.qk_norm_span not in ("head", "projection"):
            raise ValueError(f"qk_norm_span {spec.qk_norm_span!r} is not 'head' or 'projection'")
        self.spec = spec
        self.ctx = ctx
        self.position = build_position(spec.position, ctx)
        self.scale = spec.scale or 1.0 / math.sqrt(spec.head_dim)
        self.qkv = self.o = None
        self.bias = self.q_gain = self.k_gain = self.sinks = None
        self.value_dim = spec.value_dim or spec.head_dim
        if self.value_dim > 256:
            raise ValueError(f"value_dim {self.value_dim} is not supported: at most 256")
        self.whole_norm = spec.qk_norm and spec.qk_norm_span == "projection"
        # the wide form: what the per-head kernels (equal widths, per-head norms, halves turned together) do not take
        self.wide = (self.value_dim != spec.head_dim or self.whole_norm or getattr(self.position, "neighbours", False))
        # The tensor-core attention kernels take keys and values of one width, 64 or 128. A bfloat16 run of the wide form
        # with other widths up to 128 gives every head zero channels at its end until it has such a width (zero rows in
        # the projections, zero columns in the output matrix): scores and outputs are the same numbers, the cache rows are
        # wider, and prompts and single tokens run on the tensor cores instead of the general kernel.
        self.key_run, self.value_run = spec.head_dim, self.value_dim
        if self.wide and ctx.dtype == torch.bfloat16 and max(spec.head_dim, self.value_dim) <= 128:
            self.key_run = self.value_run = 64 if max(spec.head_dim, self.value_dim) <= 64 else 128
        if self.wide and (spec.qkv_bias or spec.reads_shared_kv):
            raise ValueError("attention: biases and a borrowed cache entry are not built for values of another width, "
                             "whole-projection norms or neighbour pairing")

    # ---- weights ----
    def declare(self):
        s = self.spec
        d = {"q_proj.weight": ParamDecl((s.heads * s.head_dim, s.hidden)),
             "o_proj.weight": ParamDecl((s.hidden, s.heads * self.value_dim))}
        if not s.reads_shared_kv:
            d["k_proj.weight"] = ParamDecl((s.kv_heads * s.head_dim, s.hidden))
            d["v_proj.weight"] = ParamDecl((s.kv_heads * self.value_dim, s.hidden))
        if s.qkv_bias:
            d["q_proj.bias"] = ParamDecl((s.heads * s.head_dim,), "vector")
            if not s.reads_shared_kv:
                d["k_proj.bias"] = ParamDecl((s.kv_heads * s.head_dim,), "vector")
                d["v_proj.bias"] = ParamDecl((s.kv_heads * s.head_dim,), "vector")
        if s.qk_norm:
            d["q_norm.weight"] = ParamDecl(((s.heads if self.whole_norm else 1) * s.head_dim,), "vector", init="gain")
            if not s.reads_shared_kv:
                d["k_norm.weight"] = ParamDecl(((s.kv_heads if self.whole_norm else 1) * s.head_dim,), "vector", init="gain")
        if s.sinks:
            d["sinks"] = ParamDecl((s.heads,), "vector")
        return d

    def bind(self, t):
        s = self.spec
        names = ["q_proj"] if s.reads_shared_kv else ["q_proj", "k_proj", "v_proj"]
        if (self.key_run, self.value_run) != (s.head_dim, self.value_dim):
            self._bind_padded(t)
            return
        self.qkv = Linear(torch.cat([t[n + ".weight"] for n in names], dim=0), self.ctx.dtype)
        self.o = Linear(t["o_proj.weight"], self.ctx.dtype)
        if s.qkv_bias:
            self.bias = torch.cat([t[n + ".bias"] for n in names]).contiguous()
        if s.qk_norm:
            self.q_gain = t["q_norm.weight"]
            self.k_gain = t["q_norm.weight"] if s.reads_shared_kv else t["k_norm.weight"]
        if s.sinks:
            self.sinks = t["sinks"].to(torch.float32).contiguous()

    def _bind_padded(self, t):
        """The wide form's tensors with every head widened by zero channels to ``key_run`` / ``value_run``."""
        s, dt = self.spec, self.ctx.dtype

        def heads_padded(w, n, width, run):          # [n * width, ...] -> [n * run, ...], zeros behind each head
            rest = w.shape[1:]
            out = torch.zeros((n, run, *rest), dtype=w.dtype, device=w.device)
            out[:, :width] = w.reshape(n, width, *rest)
            return out.reshape(n * run, *rest)

        q = heads_padded(t["q_proj.weight"], s.heads, s.head_dim, self.key_run)
        k = heads_padded(t["k_proj.weight"], s.kv_heads, s.head_dim, self.key_run)
        v = heads_padded(t["v_proj.weight"], s.kv_heads, self.value_dim, self.value_run)
        self.qkv = Linear(torch.cat([q, k, v], dim=0), dt)
        o = t["o_proj.weight"]                        # [hidden, heads * value_dim]: zero columns behind each head
        self.o = Linear(heads_padded(o.t().contiguous(), s.heads, self.value_dim, self.value_run).t().contiguous(), dt)
        if s.qk_norm:
            if self.whole_norm:
                self.q_gain = heads_padded(t["q_norm.weight"], s.heads, s.head_dim, self.key_run).contiguous()
                self.k_gain = heads_padded(t["k_norm.weight"], s.kv_heads, s.head_dim, self.key_run).contiguous()
            else:
                self.q_gain = heads_padded(t["q_norm.weight"], 1, s.head_dim, self.key_run).contiguous()
                self.k_gain = heads_padded(t["k_norm.weight"], 1, s.head_dim, self.key_run).contiguous()
        if s.sinks:
            self.sinks = t["sinks"].to(torch.float32).contiguous()

    def cache_request(self):
        s = self.spec
        return KVRequest(s.kv_heads, self.key_run, s.window, 0 if self.value_run == self.key_run else self.value_run)

    # ---- one step ----
    def _attend(self, q, y, b, view, table, ws):
        """Attention of the step's (post-processed) queries over the cache into ``y``; the kernel by dtype and step shape."""
        s = self.spec
        hd, vd = self.key_run, self.value_run
        flash = ops.flash_supported(hd, self.ctx.dtype) and vd == hd
        if not flash:
            ops.attention(q, view.k_pool, view.v_pool, y, b.tok_seq, b.tok_pos, table, s.heads, s.kv_heads,
                          hd, view.window, self.scale, b.stream, sinks=self.sinks, value_dim=vd)
        elif b.max_count == 1:
            splits = ops.decode_splits(b.n, s.kv_heads, s.heads // s.kv_heads, table.shape[1])
            floats = ops.decode_scratch_floats(b.n, s.heads, hd, splits)
            scratch = ws.take((floats,), torch.float32) if floats else None
            ops.attention_decode(q, view.k_pool, view.v_pool, y, b.seq_start, b.past, table, s.heads, s.kv_heads,
                                 hd, view.window, self.scale, splits, scratch, b.stream, sinks=self.sinks,
                                 next_read=self.o.weight)
        elif use_tc_attention(s.heads, s.kv_heads, hd, self.ctx.dtype, b.max_count, self.scale):
            ops.attention_tc(q, view.k_pool, view.v_pool, y, b.seq_start, b.past, b.counts, table, b.max_count,
                             s.heads, s.kv_heads, hd, view.window, self.scale, b.stream, max_keys=b.max_len,
                             sinks=self.sinks)
        else:
            ops.attention_prefill(q, view.k_pool, view.v_pool, y, b.seq_start, b.past, b.counts, table, b.max_count,
                                  s.heads, s.kv_heads, hd, view.window, self.scale, b.stream, sinks=self.sinks)

    def lead_weight(self):
        return self.qkv.weight if self.qkv is not None else None

    def fused_decode(self):
        s = self.spec
        rot = self.position.rot_dim
        if (self.wide or self.sinks is not None or self.ctx.dtype != torch.bfloat16 or self.qkv is None or s.reads_shared_kv or s.head_dim not in (64, 128)
                or rot not in (0, s.head_dim) or s.heads // s.kv_heads > 8 or s.hidden % 128
                or (s.qk_norm and (self.q_gain is None or self.k_gain is None))):
            return None
        tables = self.position.tables() if rot else None
        return {"w_qkv": self.qkv.weight, "w_o": self.o.weight, "bias": self.bias, "q_gain": self.q_gain if s.qk_norm else None,
                "k_gain": self.k_gain if s.qk_norm else None, "cos": tables[0] if tables else None,
                "sin": tables[1] if tables else None, "heads": s.heads, "kv_heads": s.kv_heads, "head_dim": s.head_dim,
                "window": s.window, "qk_eps": s.qk_norm_eps, "scale": self.scale, "hidden": s.hidden}

    def forward(self, h, x, b, view, ws):
        s = self.spec
        T = h.shape[0]
        writes = view.writes and not s.reads_shared_kv
        kvh = 0 if s.reads_shared_kv else s.kv_heads
        table = b.tables[view.group]
        mark = ws.mark()
        tables = self.position.tables()
        cos, sin = tables if tables is not None else (None, None)
        rot = self.position.rot_dim
        if self.wide:
            self._forward_wide(h, x, b, view, table, cos, sin, rot, ws)
            ws.release(mark)
            return
        flash = ops.flash_supported(s.head_dim, self.ctx.dtype)
        fused_post = (flash and rot in (0, s.head_dim) and b.max_count > 1 and (writes or s.reads_shared_kv)
                      and use_tc(T, self.qkv.out_features, self.qkv.in_features))
        if fused_post:
            # many tokens: the projection's epilogue post-processes q/k/v on its float32 accumulators
            q = ws.take((T, s.heads, s.head_dim), self.ctx.dtype)
            hh = h.tensor() if isinstance(h, Normed) else h
            ops.gemm_tc_qkv(hh, self.qkv.weight, s.heads, kvh, s.head_dim, self.bias, self.q_gain, self.k_gain,
                            cos if rot else None, sin if rot else None, s.qk_norm_eps, q,
                            view.k_pool if kvh else None, view.v_pool if kvh else None, b.tok_seq, b.tok_pos, table,
                            b.stream)
            y = ws.take((T, s.heads * s.head_dim), self.ctx.dtype)
            self._attend(q, y, b, view, table, ws)
            self.o.forward(y, into=x, ws=ws, stream=b.stream)
            ws.release(mark)
            return
        single = flash and b.max_count == 1 and rot in (0, s.head_dim) and (writes or s.reads_shared_kv)
        pages = None
        if single:
            splits = ops.decode_splits(b.n, s.kv_heads, s.heads // s.kv_heads, table.shape[1])
            # the attention kernel gets onto the SMs too late to fetch ahead: the projection asks L2 for its first pages
            pages = ops.next_pages(view.k_pool, view.v_pool, table, b.past, splits, view.window)
        qkv = self.qkv.forward(h, ws=ws, stream=b.stream, next_pages=pages)
        y = ws.take((T, s.heads * s.head_dim), self.ctx.dtype)
        if single:
            # one token per sequence: the attention kernel post-processes q/k/v itself and appends to the cache
            floats = ops.decode_scratch_floats(b.n, s.heads, s.head_dim, splits)
            scratch = ws.take((floats,), torch.float32) if floats else None
            ops.attention_decode(None, view.k_pool, view.v_pool, y, b.seq_start, b.past, table, s.heads, s.kv_heads,
                                 s.head_dim, view.window, self.scale, splits, scratch, b.stream, qkv=qkv,
                                 qkv_kv_heads=kvh, bias=self.bias, q_gain=self.q_gain, k_gain=self.k_gain,
                                 cos=cos if rot else None, sin=sin if rot else None, eps=s.qk_norm_eps,
                                 next_read=self.o.weight, sinks=self.sinks)
            self.o.forward(y, into=x, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None))
            ws.release(mark)
            return
        q = ws.take((T, s.heads, s.head_dim), self.ctx.dtype)
        ops.qkv_post(qkv, self.bias, self.q_gain, self.k_gain, cos, sin, q,
                     view.k_pool if writes else None, view.v_pool if writes else None,
                     b.tok_seq, b.tok_pos, table, s.heads, kvh, s.head_dim, rot, s.qk_norm_eps, b.stream)
        self._attend(q, y, b, view, table, ws)
        self.o.forward(y, into=x, ws=ws, stream=b.stream)
        ws.release(mark)


    def _forward_wide(self, h, x, b, view, table, cos, sin, rot, ws):
        """The wide form: the stacked projection's float32 rows, then norms, rotation and the cache write in one kernel
        on those rows (one rounding, at the store), then attention over the cache and the output projection."""
        s = self.spec
        T = h.shape[0]
        qkv = self.qkv.forward(h, ws=ws, stream=b.stream, out_dtype=torch.float32)
        q = ws.take((T, s.heads, self.key_run), self.ctx.dtype)
        writes = view.writes
        ops.qkv_post_span(qkv, self.q_gain, self.k_gain, cos if rot else None, sin if rot else None, q,
                          view.k_pool if writes else None, view.v_pool if writes else None, b.tok_seq, b.tok_pos, table,
                          s.heads, s.kv_heads, self.key_run, self.value_run, rot, self.position.neighbours, self.whole_norm,
                          s.qk_norm_eps, b.stream, norm_dim=s.head_dim)
        y = ws.take((T, s.heads * self.value_run), self.ctx.dtype)
        self._attend(q, y, b, view, table, ws)
        self.o.forward(y, into=x, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None))


register_mixer("gqa_attention", GQAAttention)

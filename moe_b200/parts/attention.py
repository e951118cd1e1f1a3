"""Grouped-query attention with optional q/k/v bias, a position encoding of its own
kind and an optional sliding window (src/model.rs:689-834, Gqa at :42-50).

  q = Wq n + bq, k = Wk n + bk, v = Wv n + bv   (bias by tensor, :707-713)
  rotate q and k heads at the token's position (:729-731); cache k (rotated) and v (:733-734)
  scores over [lo, p], lo = max(0, p + 1 - window) with a window else 0 (:803-808)
  kv head of query head h is h / (heads / kv_heads) (:809); delta = Wo ctx, no bias (:829-833)

A layer with ``own_kv = False`` projects queries only and attends over the cache
entry another layer wrote.
"""
from __future__ import annotations

import math

import torch

from ..cache.kv import KVRequest
from ..config.spec import PartSpec
from ..ops import core
from ..ops.linear import linear
from .base import Part, TensorSpec, make_part, register_part


class GQAttention(Part):
    category, kind = "mixer", "gqa_attention"
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.bias = bool(p.get("qkv_bias", False))
        self.window = p.get("window")
        self.own_kv = bool(p.get("own_kv", True))
        pos = dict(p.get("position") or {"kind": "none"})
        self.position = make_part("position", PartSpec(pos.pop("kind"), pos, spec.prefix))
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            raise ValueError(f"head_dim {self.hd}: the attention kernels take multiples of 16 from 16 to 256")
        if self.window is not None and self.window <= 0:
            raise ValueError("window must be positive")

    def tensors(self):
        t = {
            "q_proj.weight": TensorSpec((self.nh * self.hd, self.hidden)),
            "o_proj.weight": TensorSpec((self.hidden, self.nh * self.hd)),
        }
        if self.own_kv:
            t["k_proj.weight"] = TensorSpec((self.nkv * self.hd, self.hidden))
            t["v_proj.weight"] = TensorSpec((self.nkv * self.hd, self.hidden))
        if self.bias:
            t["q_proj.bias"] = TensorSpec((self.nh * self.hd,), vector=True)
            if self.own_kv:
                t["k_proj.bias"] = TensorSpec((self.nkv * self.hd,), vector=True)
                t["v_proj.bias"] = TensorSpec((self.nkv * self.hd,), vector=True)
        t.update(self.position.tensors())
        return t

    def kv_request(self):
        return KVRequest(self.nkv, self.hd, self.window)

    def describe(self):
        d = f"GQA({self.nh} q / {self.nkv} kv heads, head_dim={self.hd}{', bias' if self.bias else ''})"
        d += f", {self.position.describe()}"
        if self.window:
            d += f", window {self.window}"
        if not self.own_kv:
            d += ", reads another layer's cache"
        return d

    def state_request(self):
        return None

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        names = ["q_proj", "k_proj", "v_proj"] if self.own_kv else ["q_proj"]
        ws = [tensors[n + ".weight"] for n in names]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.wqkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.bqkv = None
        if self.bias:
            self.bqkv = torch.cat([tensors[n + ".bias"].to(torch.float32) for n in names]).contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()
        self.position.bind(tensors, rt)
        self.scale = self.position.attention_scale() / math.sqrt(self.hd)

    def forward(self, rt, h, batch, cache_view, state=None):
        T = batch.num_tokens
        nkv = self.nkv if self.own_kv else 0
        qkv = linear(rt, h.act, self.wqkv, bias=self.bqkv)
        table, rot = self.position.rotary_table()
        if table is None and hasattr(self.position, "apply"):
            self.position.apply(rt, qkv, self.nh, nkv, self.hd, batch.pos)
        ctx = rt.empty((T, self.nh * self.hd))
        if getattr(batch, "has_padding", False) and not batch.all_decode:
            ctx.zero_()      # rows of no sequence are written by no attention kernel
        if batch.all_decode and self.own_kv:
            # one token per sequence: rotation, append, attention split along the keys and the
            # merge in ONE launch where the head size allows it
            if core.attention_decode_fused(qkv, table, rot, cache_view, batch, ctx, nh=self.nh, window=self.window,
                                           scale=self.scale, status=rt.status):
                return linear(rt, ctx, self.wo)
            # else: rotate and append in one launch, then attend over the cache alone
            q = rt.empty((T, self.nh, self.hd))
            core.rope_commit(qkv, batch.pos, table, self.nh, nkv, self.hd, rot, q, cache_view, batch, rt.status)
            core.attention_decode(q, cache_view, batch, ctx, nh=self.nh, window=self.window, scale=self.scale,
                                  status=rt.status)
            return linear(rt, ctx, self.wo)
        q = rt.empty((T, self.nh, self.hd))
        k_new = rt.empty((T, max(nkv, 1), self.hd))
        v_new = rt.empty((T, max(nkv, 1), self.hd))
        # whole prompts read nothing from the cache, so their keys and values may go there at once
        early = batch.all_fresh and self.own_kv and not batch.all_decode
        committed = early and core.rope_split(qkv, batch.pos, table, self.nh, nkv, self.hd, rot, q, k_new, v_new,
                                              commit=(cache_view, batch), status=rt.status)
        if not committed:
            core.rope_split(qkv, batch.pos, table, self.nh, nkv, self.hd, rot, q, k_new, v_new)
        if batch.all_decode:
            # a layer that reads another layer's cache: queries only
            core.attention_decode(q, cache_view, batch, ctx, nh=self.nh, window=self.window, scale=self.scale,
                                  status=rt.status)
        else:
            done = False
            if batch.all_fresh and self.own_kv and rt.is_bf16:
                # whole prompts: nothing is read from the cache; tensor-core kernel
                from ..ops import tc

                done = tc.attention_prefill(q, k_new, v_new, batch, ctx, nh=self.nh, nkv=self.nkv, hd=self.hd,
                                            window=self.window, scale=self.scale, status=rt.status)
            elif self.own_kv and rt.is_bf16:
                # keys of earlier steps from the pages of the cache, keys of this step from its own
                # buffers; the same tensor-core kernel
                from ..ops import tc

                done = tc.attention_cached(q, k_new, v_new, cache_view, batch, ctx, nh=self.nh, window=self.window,
                                           scale=self.scale, status=rt.status)
            if not done:
                # the same on the CUDA cores in 32-bit arithmetic, 64 queries to a block (the plain
                # kernel where that one declines)
                kw = dict(nh=self.nh, window=self.window, scale=self.scale, use_local=self.own_kv, status=rt.status)
                if not core.attention_tiled(q, k_new, v_new, cache_view, batch, ctx, **kw):
                    core.attention_generic(q, k_new, v_new, cache_view, batch, ctx, **kw)
            if self.own_kv and not committed:
                core.kv_commit(k_new, v_new, cache_view, batch, rt.status)
        return linear(rt, ctx, self.wo)


register_part("mixer", "gqa_attention", GQAttention)

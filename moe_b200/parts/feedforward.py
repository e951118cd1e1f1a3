"""Feed-forward parts: a dense SwiGLU MLP and routed SwiGLU experts with an
optional sigmoid-gated shared expert.

SwiGLU (src/model.rs:26-35):   y = Wd (silu(Wg n) * (Wu n))
Routing (src/model.rs:844-897): softmax over all experts, top k, optional
  renormalisation, scaling factor.
Experts (src/model.rs:902-942): out_i = sum_e w_ie * y_e(n_i).
Shared expert (src/model.rs:956-970): out += sigmoid(Wsg n) * y_s(n).
"""
from __future__ import annotations

import os

import torch

from ..ops import core
from ..ops.linear import grouped_linear, grouped_swiglu_linear, linear, swiglu_linear
from .base import Activations, LazyDelta, Part, TensorSpec, register_part


def _fuse_rows(tensors):
    dt = tensors[0].dtype if all(t.dtype == tensors[0].dtype for t in tensors) else torch.float32
    return torch.cat([t.to(dt) for t in tensors], dim=0).contiguous()


class DenseSwiGLU(Part):
    category, kind = "ffn", "dense_swiglu"
    graph_safe = True
    wants32 = False

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.size = int(self.params["size"])

    def tensors(self):
        return {
            "gate_proj.weight": TensorSpec((self.size, self.hidden)),
            "up_proj.weight": TensorSpec((self.size, self.hidden)),
            "down_proj.weight": TensorSpec((self.hidden, self.size)),
        }

    def describe(self):
        return f"dense SwiGLU {self.size}"

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_gu = _fuse_rows([tensors["gate_proj.weight"], tensors["up_proj.weight"]])
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, rt, h, batch):
        return linear(rt, swiglu_linear(rt, h.act, self.w_gu), self.w_down)


class CombineDelta(LazyDelta):
    """The routed experts' outputs before the combine: delta[t] = sum_j w[t, j] * y[pos[t, j]] +
    gate[t] * shared[t].  An RMS norm forms it inside its own kernel."""

    kind = "expert_combine"

    def __init__(self, y, pos_of_pair, topk_w, top_k, shared, shared_gate, tokens, hidden):
        self.y, self.pos_of_pair, self.topk_w, self.top_k = y, pos_of_pair, topk_w, top_k
        self.shared, self.shared_gate, self.tokens, self.hidden = shared, shared_gate, tokens, hidden

    def materialize(self, rt):
        out = rt.empty((self.tokens, self.hidden), torch.float32)
        core.moe_combine(self.y, self.pos_of_pair, self.topk_w, self.top_k, out, shared=self.shared,
                         shared_gate=self.shared_gate)
        return out


class RoutedExperts(Part):
    category, kind = "ffn", "routed_experts"
    graph_safe = True
    wants32 = True   # router logits are computed from the 32-bit normed state

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.E = int(p["num_experts"])
        self.k = int(p["top_k"])
        self.size = int(p["expert_size"])
        self.norm_topk = bool(p.get("norm_topk_prob", False))
        self.scale = float(p.get("routed_scaling_factor", 1.0))
        self.shared_size = int(p.get("shared_size", 0) or 0)
        self.shared_gate = bool(p.get("shared_gate", False)) and self.shared_size > 0
        if not 0 < self.k <= self.E:
            raise ValueError("top_k must lie in 1..num_experts")
        # Set to a list to record every routing decision as (expert ids [T, k], weights [T, k]);
        # the reference's State::trace does the same per token and layer (src/model.rs:157, 943-950).
        self.trace = None
        # measured on a B200: the fused norm + router + dispatch launch wins up to 8 tokens and loses
        # from 16 on, where its single gathering block is the bottleneck
        self.fused_norm_tokens = int(os.environ.get("MOE_B200_NORM_ROUTE_MAX", "8"))
        self.shared_beside = os.environ.get("MOE_B200_SHARED_BESIDE", "1") != "0"
        # up to this many tokens one block picks, inverts and gathers (one launch after the logits);
        # beyond, a warp per token picks and the inversion and the gather are launches of their own
        # (measured on a B200, ms a decode step at 16 / 32 / 64 tokens: 4.65 / 5.89 / 7.38 with one
        # block up to 64 tokens, 4.48 / 5.75 / 7.07 with one block up to 8)
        self.route_dispatch_tokens = int(os.environ.get("MOE_B200_ROUTE_DISPATCH_MAX", "8"))
        # from this many tokens on (a prompt) the router's logits are a tensor-core product of the
        # 32-bit activations split into three bfloat16 terms (35 -> about 15 us at 2,048 tokens)
        self.tc_router_tokens = int(os.environ.get("MOE_B200_TC_ROUTER_MIN", "257"))

    def tensors(self):
        t = {"gate.weight": TensorSpec((self.E, self.hidden))}
        for e in range(self.E):
            t[f"experts.{e}.gate_proj.weight"] = TensorSpec((self.size, self.hidden), sparse=True)
            t[f"experts.{e}.up_proj.weight"] = TensorSpec((self.size, self.hidden), sparse=True)
            t[f"experts.{e}.down_proj.weight"] = TensorSpec((self.hidden, self.size), sparse=True)
        return self._common(t)

    def _common(self, t):
        if self.shared_size:
            t["shared_expert.gate_proj.weight"] = TensorSpec((self.shared_size, self.hidden))
            t["shared_expert.up_proj.weight"] = TensorSpec((self.shared_size, self.hidden))
            t["shared_expert.down_proj.weight"] = TensorSpec((self.hidden, self.shared_size))
        if self.shared_gate:
            t["shared_expert_gate.weight"] = TensorSpec((1, self.hidden))
        return t

    def tensors_in(self, has):
        """Three checkpoint layouts of the experts, as the reference reads them (src/model.rs:396-420):
        fused ``experts.gate_up_proj`` [E, 2 size, hidden] (rows [0, size) gate, then up) with
        ``experts.down_proj`` [E, hidden, size]; stacked ``experts.{gate,up,down}_proj`` of three
        dimensions; else one tensor per expert and projection."""
        E, n, H = self.E, self.size, self.hidden
        if has("experts.gate_up_proj"):
            t = {"gate.weight": TensorSpec((E, H)), "experts.gate_up_proj": TensorSpec((E, 2 * n, H), sparse=True),
                 "experts.down_proj": TensorSpec((E, H, n), sparse=True)}
            return self._common(t)
        if has("experts.gate_proj") and has("experts.up_proj"):
            t = {"gate.weight": TensorSpec((E, H)), "experts.gate_proj": TensorSpec((E, n, H), sparse=True),
                 "experts.up_proj": TensorSpec((E, n, H), sparse=True),
                 "experts.down_proj": TensorSpec((E, H, n), sparse=True)}
            return self._common(t)
        return self.tensors()

    def describe(self):
        return (f"{self.E} experts of {self.size}, top-{self.k}, softmax gate"
                + (", renormalised" if self.norm_topk else "")
                + (f", scaled by {self.scale:g}" if self.scale != 1.0 else "")
                + (f", shared expert {self.shared_size}" + (" (gated)" if self.shared_gate else "")
                   if self.shared_size else ""))

    def step_elements(self, num_tokens):
        """The router, the shared expert, and the experts that ``num_tokens`` tokens are expected to
        touch if each picks ``top_k`` of them evenly: E (1 - (1 - k/E)^tokens)."""
        dense = sparse = 0
        for ts in self.tensors().values():
            n = 1
            for d in ts.shape:
                n *= d
            if ts.sparse:
                sparse += n
            else:
                dense += n
        touched = 1.0 - (1.0 - self.k / self.E) ** max(num_tokens, 0)
        return dense + sparse * touched

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_router = tensors["gate.weight"].contiguous()
        dev = self.w_router.device
        # The device layout is [E, 2 * size, hidden] (rows [0, size) gate, [size, 2 size) up) and
        # [E, hidden, size], whatever the checkpoint's; tensors are fetched one at a time.
        if "experts.gate_up_proj" in tensors:
            self.w_gu = tensors["experts.gate_up_proj"].contiguous()
            self.w_down = tensors["experts.down_proj"].contiguous()
            if self.w_gu.dtype != self.w_down.dtype:
                self.w_gu, self.w_down = self.w_gu.float(), self.w_down.float()
        elif "experts.gate_proj" in tensors:
            g, u, self.w_down = tensors["experts.gate_proj"], tensors["experts.up_proj"], tensors["experts.down_proj"]
            dt = g.dtype if g.dtype == u.dtype == self.w_down.dtype else torch.float32
            self.w_gu = torch.cat([g.to(dt), u.to(dt)], dim=1).contiguous()
            self.w_down = self.w_down.to(dt).contiguous()
        else:
            first = tensors["experts.0.gate_proj.weight"]
            dt = first.dtype
            self.w_gu = torch.empty((self.E, 2 * self.size, self.hidden), dtype=dt, device=dev)
            self.w_down = torch.empty((self.E, self.hidden, self.size), dtype=dt, device=dev)
            for e in range(self.E):
                for name, dst in ((f"experts.{e}.gate_proj.weight", self.w_gu[e, : self.size]),
                                  (f"experts.{e}.up_proj.weight", self.w_gu[e, self.size:]),
                                  (f"experts.{e}.down_proj.weight", self.w_down[e])):
                    t = tensors[name]
                    if t.dtype != dt:                  # a checkpoint of mixed dtypes: everything in 32-bit
                        self.w_gu, self.w_down, dt = self.w_gu.float(), self.w_down.float(), torch.float32
                        dst = {"gate": self.w_gu[e, : self.size], "up": self.w_gu[e, self.size:],
                               "down": self.w_down[e]}[name.split(".")[2].split("_")[0]]
                    dst.copy_(t)
        self.ws_gu = self.ws_down = self.w_sgate = None
        if self.shared_size:
            self.ws_gu = _fuse_rows([tensors["shared_expert.gate_proj.weight"], tensors["shared_expert.up_proj.weight"]])
            self.ws_down = tensors["shared_expert.down_proj.weight"].contiguous()
        if self.shared_gate:
            self.w_sgate = tensors["shared_expert_gate.weight"].reshape(-1).to(self.w_router.dtype).contiguous()
        # For prompts the router's logits come from the tensor cores: the 32-bit activations as three
        # bfloat16 terms against the (bfloat16, hence exact) router rows, three times side by side.
        self.w_router3 = None
        if rt.is_bf16 and self.w_router.dtype == torch.bfloat16 and self.hidden % 8 == 0:
            rows = [self.w_router] + ([self.w_sgate.reshape(1, -1)] if self.w_sgate is not None else [])
            one = torch.cat(rows, dim=0)
            self.w_router3 = torch.cat([one, one, one], dim=1).contiguous()

    def route(self, rt, h, batch, after_logits=None):
        """-> (topk_idx [T, k] int32, topk_w [T, k] float32, shared_gate [T] float32 or None)
        ``after_logits``: called once the logits' product is launched (or, where logits and picks are one
        launch, after that)."""
        T = h.f32.shape[0]
        topk_idx = rt.empty((T, self.k), torch.int32)
        topk_w = rt.empty((T, self.k), torch.float32)
        sg = rt.empty((T,), torch.float32) if self.w_sgate is not None else None
        if self.w_router3 is not None and T >= self.tc_router_tokens:
            from ..ops import tc

            logits = rt.empty((T, self.w_router3.shape[0]), torch.float32)
            if tc.gemm_tc(core.split3(h.f32), self.w_router3, logits, bn=64, splits=8, status=rt.status):
                if after_logits is not None:
                    after_logits()
                core.router_topk(logits, self.k, self.norm_topk, self.scale, topk_idx, topk_w, num_experts=self.E,
                                 shared_gate=sg, seq_of_token=getattr(batch, "seq_of_token", None))
                return topk_idx, topk_w, sg
        core.router(h.f32, self.w_router, self.k, self.norm_topk, self.scale, topk_idx, topk_w,
                    shared_gate_w=self.w_sgate, shared_gate=sg, seq_of_token=getattr(batch, "seq_of_token", None))
        if after_logits is not None:
            after_logits()
        return topk_idx, topk_w, sg

    def _shared(self, rt, h):
        return linear(rt, swiglu_linear(rt, h.act, self.ws_gu), self.ws_down)

    def forward(self, rt, h, batch):
        return self._run(rt, h, batch, None).materialize(rt)

    def forward_lazy(self, rt, h, batch):
        """The same, the combine left to whoever adds the delta (see ``CombineDelta``)."""
        return self._run(rt, h, batch, None)

    def forward_prenorm(self, rt, x, delta, norm, batch):
        """The block's offer to take the norm before this feed-forward along: for a step of few
        tokens, norm, router and dispatch are one launch.  None if the sizes or the kind of norm do
        not allow it (the block then runs the norm itself and calls ``forward``)."""
        rms = getattr(norm, "rms_params", None)          # the norm says whether it can be run by a neighbour
        if rms is None or x.shape[0] > self.fused_norm_tokens or self.E > 256:
            return None
        norm_w, norm_eps = rms()
        routed = core.norm_route(x, delta, norm_w, norm_eps, self.w_router, self.k, self.norm_topk, self.scale,
                                 bf16=rt.is_bf16, shared_gate_w=self.w_sgate,
                                 seq_of_token=getattr(batch, "seq_of_token", None), status=rt.status)
        if routed is None:
            return None
        out32, out16 = routed[:2]
        h = Activations(act=out16 if rt.is_bf16 else out32, f32=out32)
        return self._run(rt, h, batch, routed[2:])

    def _run(self, rt, h, batch, routed):
        T = h.act.shape[0]
        P = T * self.k
        few = T <= 64 and self.E <= 256
        ys = side = None
        if self.ws_gu is not None and few:
            # few tokens: neither branch fills the GPU, so the shared expert runs beside the routed
            # ones on a second stream (inside a captured graph this becomes a fork and a join)
            main = torch.cuda.current_stream()
            side = rt.side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                ys = self._shared(rt, h)
        if routed is not None:
            topk_idx, topk_w, sg, offsets, sorted_token, pos_of_pair, xs = routed
        elif few and T <= self.route_dispatch_tokens:
            # pick, table inversion and gather in one launch after the logits
            topk_idx, topk_w, sg, offsets, sorted_token, pos_of_pair, xs = core.route_dispatch(
                h.f32, self.w_router, self.k, self.norm_topk, self.scale, shared_gate_w=self.w_sgate,
                seq_of_token=getattr(batch, "seq_of_token", None),
                gather=h.act if h.act.dtype == torch.bfloat16 and T <= 16 else None, status=rt.status)
            # (more tokens: the gather by that one block would take longer than a launch of its own)
        else:
            def shared_beside():
                # Many tokens: pick, table inversion and gather are small launches that leave the GPU
                # idle (37 us of a layer at 2,048 tokens), so the shared expert starts beside them on
                # a second stream.  (Not before the logits' product: the shared expert's CTAs fill every
                # SM's shared memory, and that product would wait for them to end.)
                nonlocal ys, side
                main = torch.cuda.current_stream()
                side = rt.side_stream()
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    ys = self._shared(rt, h)

            topk_idx, topk_w, sg = self.route(rt, h, batch,
                                              after_logits=shared_beside if self.ws_gu is not None and side is None and self.shared_beside else None)
            offsets = rt.empty((self.E + 1,), torch.int32)
            sorted_token = rt.empty((P,), torch.int32)
            pos_of_pair = rt.empty((P,), torch.int32)
            core.moe_align(topk_idx, T, self.k, self.E, offsets, sorted_token, pos_of_pair, rt.status)
            xs = None
        if self.trace is not None:
            self.trace.append((topk_idx.clone(), topk_w.clone()))
        act = grouped_swiglu_linear(rt, h.act, self.w_gu, offsets, sorted_token, P, gathered=xs)
        # (the offsets were written before the product above: the second product may start on its weights early)
        y = grouped_linear(rt, act, self.w_down, offsets, P, early_offsets=True)
        if self.ws_gu is not None and side is None:
            ys = self._shared(rt, h)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
            ys.record_stream(torch.cuda.current_stream())
        return CombineDelta(y, pos_of_pair, topk_w, self.k, ys, sg, T, self.hidden)


register_part("ffn", "dense_swiglu", DenseSwiGLU)
register_part("ffn", "routed_experts", RoutedExperts)

"""RMSNorm: s = 1/sqrt(mean(x^2) + eps), out = x * s * w (src/model.rs:211-216)."""
from __future__ import annotations

import torch

from ..ops import core
from .base import Activations, LazyDelta, Part, TensorSpec, register_part


class RMSNorm(Part):
    category, kind = "norm", "rmsnorm"
    graph_safe = True
    lazy_kinds = ("expert_combine",)      # deltas this norm forms inside its own kernel

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])
        self.eps = float(self.params["eps"])

    def tensors(self):
        return {"weight": TensorSpec((self.size,), init="ones", vector=True)}

    def describe(self):
        return f"RMSNorm eps {self.eps:g}"

    def rms_params(self):
        """(weight, eps): what a neighbour needs to run this norm inside a kernel of its own (a
        feed-forward that fuses the norm before it with its first step asks for this; a norm
        that is no plain RMS norm simply has no such method)."""
        return self.weight, self.eps

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def forward(self, rt, x, delta=None, rows=None, want32=False, write_back=True) -> Activations:
        """Normalise ``x (+ delta)``; with ``delta`` the sum is written back into ``x``
        (unless ``rows`` selects a subset, which leaves ``x`` alone)."""
        n = x.shape[0] if rows is None else rows.numel()
        out32 = out16 = None
        if rt.is_bf16:
            out16 = rt.empty((n, self.size), torch.bfloat16)
            if want32:
                out32 = rt.empty((n, self.size), torch.float32)
        else:
            out32 = rt.empty((n, self.size), torch.float32)
        if isinstance(delta, LazyDelta):
            if delta.kind != "expert_combine" or not core.rmsnorm_combine(
                    x, delta, self.weight, self.eps, rows=rows, out32=out32, out16=out16, write_back=write_back,
                    status=rt.status):
                delta = delta.materialize(rt)
            else:
                return Activations(act=out16 if rt.is_bf16 else out32, f32=out32)
        core.rmsnorm(x, self.weight, self.eps, delta=delta, rows=rows, out32=out32, out16=out16,
                     write_back=write_back, status=rt.status)
        return Activations(act=out16 if rt.is_bf16 else out32, f32=out32)


register_part("norm", "rmsnorm", RMSNorm)

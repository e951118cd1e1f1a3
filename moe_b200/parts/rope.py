"""Rotary position encoding.

inv_freq[i] = theta^(-2 i / dim) for i < dim/2, computed in float32 as the
reference does (src/spec.rs:89-96); the angle of position p is float32(p) *
inv_freq[i] (src/model.rs:326-328).  Pairs are half-split: (i, i + dim/2).
"""
from __future__ import annotations

import torch

from .base import Part, register_part


def rotary_inv_freq(theta: float, dim: int) -> torch.Tensor:
    # float32 exponent as in the reference, the power itself correctly rounded to float32
    i = torch.arange(dim // 2, dtype=torch.float32)
    expo = ((-2.0 * i) / torch.tensor(float(dim), dtype=torch.float32)).to(torch.float64)
    theta32 = torch.tensor(float(theta), dtype=torch.float32).to(torch.float64)
    return torch.pow(theta32, expo).to(torch.float32)


class RotaryEncoding(Part):
    category, kind = "position", "rotary"

    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(self.params["theta"])
        self.rotary_dim = int(self.params["rotary_dim"])
        if self.rotary_dim % 2:
            raise ValueError("rotary_dim must be even")

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.inv_freq = rotary_inv_freq(self.theta, self.rotary_dim).to(rt.device)

    def describe(self):
        return f"rope theta {self.theta:.0f}" + (f" on {self.rotary_dim} dims" if self.params.get("partial") else "")

    def rotary_table(self):
        """(inv_freq, rotary_dim): lets the mixer rotate inside its own kernel."""
        return self.inv_freq, self.rotary_dim

    def attention_scale(self) -> float:
        """Extra factor on 1/sqrt(head_dim); 1 without context extension (src/spec.rs:148-151)."""
        return 1.0


class NoPositionEncoding(Part):
    category, kind = "position", "none"

    def describe(self):
        return "no position encoding"

    def rotary_table(self):
        return None, 0

    def attention_scale(self) -> float:
        return 1.0


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)

"""How a mixer, a feed-forward and their norms are arranged in a layer.

Pre-norm with two residual sums (src/model.rs:669-684):
    n = norm1(x); x += mixer(n); n = norm2(x); x += ffn(n)
The residual stream ``x`` is float32.  The last sum of a block is left pending
and folded into the next norm (of the next block, or the final one), which
reads and writes the stream once instead of twice.
"""
from __future__ import annotations

from ..config.spec import LayerSpec
from .base import delta_for, make_part


class PreNormBlock:
    category, kind = "block", "prenorm"

    def __init__(self, layer: LayerSpec):
        self.layer = layer
        self.norm1 = make_part("norm", layer.norm1)
        self.mixer = make_part("mixer", layer.mixer)
        self.norm2 = make_part("norm", layer.norm2)
        self.ffn = make_part("ffn", layer.ffn)

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def forward(self, rt, x, pending, batch, cache_view, state):
        """x: [T, hidden] float32 stream; pending: a delta not yet added (or None).
        Returns (x, pending)."""
        h = self.norm1.forward(rt, x, delta=delta_for(self.norm1, pending, rt),
                               want32=getattr(self.mixer, "wants32", False))
        delta = self.mixer.forward(rt, h, batch, cache_view, state)
        # a feed-forward may offer to run the norm before it itself (fused with its first
        # kernels); it returns None where it cannot, and nothing has happened then
        prenorm = getattr(self.ffn, "forward_prenorm", None)
        if prenorm is not None:
            out = prenorm(rt, x, delta, self.norm2, batch)
            if out is not None:
                return x, out
        h = self.norm2.forward(rt, x, delta=delta, want32=getattr(self.ffn, "wants32", False))
        # (its delta may come back uncombined, for the next norm to finish: base.LazyDelta)
        return x, getattr(self.ffn, "forward_lazy", self.ffn.forward)(rt, h, batch)


_BLOCKS = {"prenorm": PreNormBlock}


def register_block(kind: str, cls) -> None:
    _BLOCKS[kind] = cls


def make_block(layer: LayerSpec):
    if layer.block not in _BLOCKS:
        raise KeyError(f"no block arrangement '{layer.block}'; registered: {', '.join(sorted(_BLOCKS))}")
    return _BLOCKS[layer.block](layer)

"""What every part of a layer looks like to the rest of the library.

A part is built from a ``PartSpec`` (its kind, its constants, a tensor-name
prefix), says which tensors it needs, is bound to those tensors, and is then
called once per step.  A part knows its own sizes and nothing about the model
it sits in.  New kinds are added with ``register_part``; the model builder picks
them by the ``kind`` string of the spec.

Interfaces by category
  norm      forward(rt, x, delta=None, rows=None, want32=False, write_back=True) -> Activations
  position  rotary_table() -> (inv_freq, rotary_dim) or None;  apply(rt, qkv32, layout, positions)
  mixer     forward(rt, h: Activations, batch, cache_view, state) -> delta [T, hidden] float32
            kv_request() -> KVRequest | None;  state_request() -> StateRequest | None
  ffn       forward(rt, h: Activations, batch) -> delta [T, hidden] float32;  wants32: bool
            optional: forward_lazy(rt, h, batch) -> delta or LazyDelta;
                      forward_prenorm(rt, x, delta, norm, batch) -> delta, LazyDelta, or None (not taken)
  block     forward(rt, x, pending, batch, cache_view, state) -> (x, pending)
A pending delta may be a ``LazyDelta``; ``delta_for(norm, delta, rt)`` gives what a norm can take.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch

from ..config.spec import PartSpec


class LazyDelta:
    """A residual delta that is not computed yet.  A feed-forward may hand one to its block
    (``forward_lazy`` / ``forward_prenorm``) instead of a tensor; the norm that adds it next either
    knows its ``kind`` and forms it inside its own kernel (it then declares ``lazy_kinds``), or
    gets the tensor from ``materialize``."""

    kind = ""

    def materialize(self, rt) -> torch.Tensor:
        raise NotImplementedError


def delta_for(norm, delta, rt):
    """What ``norm`` can be given for ``delta``: the lazy form if the norm takes that kind, else the tensor."""
    if isinstance(delta, LazyDelta) and delta.kind not in getattr(norm, "lazy_kinds", ()):
        return delta.materialize(rt)
    return delta


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    init: str = "normal"        # "normal" | "ones" | "zeros" for the random-weights mode
    vector: bool = False        # small vectors are widened to float32 when bound (exact)
    sparse: bool = False        # read only for the tokens that are routed to it (an expert's weights)


class Runtime:
    """Device, compute dtype and the device status word shared by all parts of a model."""

    def __init__(self, device, compute_dtype: torch.dtype):
        if compute_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("compute dtype must be float32 or bfloat16")
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        self.status = None
        if self.device.type == "cuda":
            from ..ops import core

            self.status = core.new_status(self.device)

    @property
    def is_bf16(self) -> bool:
        return self.compute_dtype == torch.bfloat16

    def side_stream(self) -> "torch.cuda.Stream":
        """A second stream of this runtime, for a branch that may run beside the main one."""
        if getattr(self, "_side", None) is None:
            from ..ops import tc

            # (default priority: a higher one was measured slower, the side branch then crowds out
            # the routed experts' first product)
            self._side = torch.cuda.Stream(device=self.device)
            tc.register_side_stream(self._side)     # its products get a split-K workspace of their own
        return self._side

    def empty(self, shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.compute_dtype, device=self.device)

    def check(self) -> None:
        from ..ops import core

        core.check_status(self.status)


@dataclass
class Activations:
    """A normed hidden state: in the compute dtype for matrix products (``act``),
    and in float32 (``f32``) for parts that ask for it (routing)."""

    act: torch.Tensor
    f32: Optional[torch.Tensor] = None


class Part:
    category = ""
    kind = ""
    # True if forward() only launches kernels on the current stream (no host synchronisation, no
    # data-dependent host control flow), so that a decode step may be captured in a CUDA graph.
    graph_safe = False
    # A part may record what it decided in a call (a router's picks, say): when ``trace`` is a list,
    # forward() appends one tuple of tensors per call; None switches it off.  A graph-safe part makes
    # those tensors with device copies only (``clone``), so that a captured step fills them again.
    # A graph-safe part must also leave rows of no sequence (``batch.seq_of_token < 0``) without
    # effect on any sequence's cache or state: captured steps are padded with such rows, and a new
    # shape of step is first run with nothing but such rows.
    trace = None

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.params = dict(spec.params)

    def tensors(self) -> Dict[str, TensorSpec]:
        """Local tensor name -> shape; the checkpoint name is spec.prefix + local name."""
        return {}

    def tensors_in(self, has: Callable[[str], bool]) -> Dict[str, TensorSpec]:
        """The tensors to read from a checkpoint in which ``has(local name)`` says what exists.  By
        default ``tensors()``; a part that takes several checkpoint layouts picks one here, and
        ``bind`` is then given those names."""
        return self.tensors()

    def describe(self) -> str:
        """One line for a summary of the model: the part's kind and the constants a reader wants."""
        return self.kind

    def step_elements(self, num_tokens: int) -> float:
        """Weight elements that a step of ``num_tokens`` tokens has to read from this part: by
        default every tensor once.  A part that reads only what its tokens pick says so here."""
        n = 0
        for ts in self.tensors().values():
            k = 1
            for d in ts.shape:
                k *= d
            n += k
        return float(n)

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        """Take ownership of the loaded tensors (re-laying them out is allowed)."""
        self.rt = rt


_REGISTRY: Dict[Tuple[str, str], Callable[[PartSpec], Part]] = {}


def register_part(category: str, kind: str, factory: Callable[[PartSpec], Part]) -> None:
    _REGISTRY[(category, kind)] = factory


def make_part(category: str, spec: PartSpec) -> Part:
    key = (category, spec.kind)
    if key not in _REGISTRY:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise KeyError(f"no {category} part of kind '{spec.kind}'; registered: {', '.join(known) or '(none)'}")
    return _REGISTRY[key](spec)


def registered_parts(category: str):
    return sorted(k for c, k in _REGISTRY if c == category)

"""Projections: choosing a kernel for y = x W^T (+ b) and for the SwiGLU pair.

The bfloat16 path uses the tcgen05 kernel (``tc.gemm_tc``) wherever activations and
weight are both bfloat16 and the shape qualifies, and the plain kernel otherwise (a
weight stored in 32-bit, a width that is no multiple of 8).  The float32 path always
uses the plain kernel, which is true 32-bit arithmetic.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import core


def _use_tc(rt, a: torch.Tensor, w: torch.Tensor) -> bool:
    return rt.is_bf16 and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16


def linear(rt, a: torch.Tensor, w: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
           out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """a: [M, K]; w: [N, K]; returns [M, N] in ``out_dtype``."""
    out = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=a.device)
    if _use_tc(rt, a, w):
        from . import tc

        if tc.gemm_tc(a, w, out, bias=bias, status=rt.status):
            return out
    core.gemm_generic(a, w, out, bias=bias, status=rt.status)
    return out


def swiglu_linear(rt, a: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(a Wg^T) * (a Wu^T) with w_gate_up = [Wg; Wu] of shape [2 I, K]; returns [M, I] in the
    compute dtype."""
    M, inter = a.shape[0], w_gate_up.shape[0] // 2
    act = torch.empty((M, inter), dtype=rt.compute_dtype, device=a.device)
    if _use_tc(rt, a, w_gate_up):
        from . import tc

        if tc.gemm_tc(a, w_gate_up, act, swiglu=True, status=rt.status):
            return act
    gu = torch.empty((M, 2 * inter), dtype=torch.float32, device=a.device)
    core.gemm_generic(a, w_gate_up, gu, status=rt.status)
    core.swiglu(gu, act)
    return act


def grouped_swiglu_linear(rt, a: torch.Tensor, w_gate_up: torch.Tensor, group_offsets: torch.Tensor,
                          rows: torch.Tensor, num_rows: int, gathered: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row i of the result is the SwiGLU of a[rows[i]] under the weights of i's group
    (w_gate_up: [G, 2 I, K]); returns [num_rows, I] in the compute dtype.  ``gathered`` may bring
    a[rows] already gathered."""
    inter = w_gate_up.shape[1] // 2
    act = torch.empty((num_rows, inter), dtype=rt.compute_dtype, device=a.device)
    if _use_tc(rt, a, w_gate_up) and a.shape[1] % 8 == 0:
        from . import tc

        xs = gathered if gathered is not None else tc.gather_rows(a, rows, num_rows, rt.status)
        if tc.gemm_tc(xs, w_gate_up, act, swiglu=True, group_offsets=group_offsets, status=rt.status):
            return act
    gu = torch.empty((num_rows, 2 * inter), dtype=torch.float32, device=a.device)
    core.gemm_generic(a, w_gate_up, gu, a_rows=rows, group_offsets=group_offsets, status=rt.status)
    core.swiglu(gu, act)
    return act


def grouped_linear(rt, a: torch.Tensor, w: torch.Tensor, group_offsets: torch.Tensor, num_rows: int,
                   early_offsets: bool = False) -> torch.Tensor:
    """Rows [offsets[g], offsets[g+1]) of a use w[g] ([G, N, K]); returns float32 [num_rows, N].
    ``early_offsets``: see ``tc.gemm_tc``."""
    out = torch.empty((num_rows, w.shape[1]), dtype=torch.float32, device=a.device)
    if _use_tc(rt, a, w):
        from . import tc

        if tc.gemm_tc(a, w, out, group_offsets=group_offsets, status=rt.status, early_offsets=early_offsets):
            return out
    core.gemm_generic(a, w, out, group_offsets=group_offsets, status=rt.status)
    return out

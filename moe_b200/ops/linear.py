"""y = x W^T (+ b): choosing a kernel for a projection.

The bfloat16 path uses the tensor-core kernels where a shape qualifies and the
plain kernel otherwise; the float32 path always uses the plain kernel, which is
true 32-bit arithmetic.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import core


def linear(rt, a: torch.Tensor, w: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
           out_dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a: [M, K] (float32 or bfloat16); w: [N, K]; returns [M, N] in ``out_dtype``."""
    M = a.shape[0]
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    core.gemm_generic(a, w, out, bias=bias, status=rt.status)
    return out


def grouped_linear(rt, a: torch.Tensor, w: torch.Tensor, group_offsets: torch.Tensor, num_rows: int, *,
                   a_rows: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Rows [offsets[g], offsets[g+1]) of the output use w[g]; row i reads a[a_rows[i]]."""
    N = w.shape[1]
    out = torch.empty((num_rows, N), dtype=out_dtype, device=a.device)
    core.gemm_generic(a, w, out, a_rows=a_rows, group_offsets=group_offsets, status=rt.status)
    return out

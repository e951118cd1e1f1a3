"""Python face of the kernel library ``tc``: the tcgen05 / TMA matrix product of the
bfloat16 path (``csrc/gemm_tc.cu``).

``gemm_tc`` returns False when the kernel refuses a shape (K or a row pitch that is
no multiple of 8 elements, an unaligned pointer); the caller then uses the plain kernel.
"""
from __future__ import annotations

import os
from ctypes import byref, c_int, c_void_p
from typing import Optional

import torch

from . import build, core

_lib = None
_NUM_SMS = None


def lib():
    global _lib
    if _lib is None:
        L = build.load("tc")
        P, I = c_void_p, c_int
        L.moe_gemm_tc.argtypes = [P, I, P, I, I, I, I, P, I, I, P, P, I, I, I, P, P, P, I, P]
        L.moe_gemm_tc.restype = c_int
        L.moe_gemm_tc_plan.argtypes = [I, I, I, I, I, I, P]
        L.moe_gemm_tc_plan.restype = c_int
        L.moe_gather_rows_bf16.argtypes = [P, P, P, I, I, I, P, P]
        L.moe_gather_rows_bf16.restype = c_int
        from ctypes import c_float

        L.moe_attention_prefill_bf16.argtypes = [P, P, P, P, P, I, I, I, I, I, I, c_float, P]
        L.moe_attention_prefill_bf16.restype = c_int
        L.moe_attention_prefill_tc.argtypes = [P, P, P, P, P, I, I, I, I, I, I, c_float, P, P]
        L.moe_attention_prefill_tc.restype = c_int
        L.moe_attention_cached_tc.argtypes = [P] * 10 + [I] * 10 + [c_float, P, P]
        L.moe_attention_cached_tc.restype = c_int
        L.moe_tc_set_pdl.argtypes = [c_int]
        L.moe_tc_set_pdl.restype = None
        import os

        if os.environ.get("MOE_B200_PDL", "1") == "0":      # programmatic dependent launch off
            L.moe_tc_set_pdl(0)
        L.moe_tc_set_persistent.argtypes = [c_int]
        L.moe_tc_set_persistent.restype = None
        if os.environ.get("MOE_B200_PERSISTENT", "1") == "0":   # one CTA per tile also for many tokens
            L.moe_tc_set_persistent(0)
        L.moe_tc_set_swiglu_interleaved.argtypes = [c_int]
        L.moe_tc_set_swiglu_interleaved.restype = None
        if os.environ.get("MOE_B200_SWIGLU_IL", "1") == "0":    # many tokens: SwiGLU with two accumulators
            L.moe_tc_set_swiglu_interleaved(0)
        L.moe_tc_set_pair.argtypes = [c_int]
        L.moe_tc_set_pair.restype = None
        if os.environ.get("MOE_B200_PAIR", "0") == "1":         # pairs of CTAs (cta_group::2) for many tokens
            L.moe_tc_set_pair(1)
        _lib = L
    return _lib


_SPLIT_TARGET = int(os.environ.get("MOE_B200_SPLIT_TARGET", "0"))      # read once: the environment is slow to ask
_ATTN_TC = os.environ.get("MOE_B200_ATTN_TC", "1") != "0"


def num_sms(device) -> int:
    global _NUM_SMS
    if _NUM_SMS is None:
        _NUM_SMS = torch.cuda.get_device_properties(device).multi_processor_count
    return _NUM_SMS


class Workspace:
    """Scratch of the split-K reduction: float32 partial sums (grown on demand) and the
    tile tickets, which every launch leaves at zero."""

    TICKETS = 1 << 16

    def __init__(self, device):
        self.device = device
        self.partials = torch.empty(1 << 24, dtype=torch.float32, device=device)   # 64 MB
        self.tickets = torch.zeros(self.TICKETS, dtype=torch.int32, device=device)

    def partials_for(self, n: int) -> torch.Tensor:
        if self.partials.numel() < n:
            if torch.cuda.is_current_stream_capturing():
                raise core.KernelError("the split-K workspace must be sized before a CUDA graph is captured")
            self.partials = torch.empty(max(n, 2 * self.partials.numel()), dtype=torch.float32, device=self.device)
        return self.partials


_workspaces = {}


def workspace(device) -> Workspace:
    """The scratch of the calling stream: products on the side stream (``Runtime.side_stream``)
    have a workspace of their own, since they may run beside products on the main stream."""
    side = core._stream() in _side_handles
    key = (device.index or 0 if isinstance(device, torch.device) else torch.device(device).index or 0, side)
    if key not in _workspaces:
        _workspaces[key] = Workspace(device)
    return _workspaces[key]


_side_streams = set()
_side_handles = set()       # their raw handles: asking torch for the current Stream object is slow


def register_side_stream(stream) -> None:
    _side_streams.add(stream)
    _side_handles.add(stream.cuda_stream)


def token_tile(rows_per_group: float, grouped: bool = False) -> int:
    """Smallest token tile (the MMA's N) that holds the expected rows of a group.  Grouped products
    of more than 16 rows a group take a tile of at least 128, i.e. the persistent form (measured at
    60 groups of 2048 x 1408: equal at 17 rows a group, 12 % faster at 34)."""
    if grouped and rows_per_group > 16:
        return 128 if rows_per_group <= 128 else 256
    for bn in (16, 32, 64, 128, 256):
        if rows_per_group <= bn:
            return bn
    return 256


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, swiglu: bool = False,
            bias: Optional[torch.Tensor] = None, group_offsets: Optional[torch.Tensor] = None,
            bn: Optional[int] = None, splits: Optional[int] = None, status=None, early_offsets: bool = False) -> bool:
    """out = x @ w[g].T (PLAIN) or silu(x @ gate.T) * (x @ up.T) (SwiGLU, w rows = gate then up).

    x: [M, K] bf16 (row pitch a multiple of 8); w: [N', K] or [G, N', K] bf16 contiguous;
    out: [M, N] float32 or bfloat16 with N = N' (PLAIN) or N' / 2 (SwiGLU).
    ``early_offsets``: the caller vouches that ``group_offsets`` were written at least two kernels
    before this one on the stream (not by its direct predecessor); the kernel then starts loading
    weights while the predecessor still runs."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_cuda:
        return False
    G = w.shape[0] if w.dim() == 3 else 1
    w_rows, K = w.shape[-2], w.shape[-1]
    N = w_rows // 2 if swiglu else w_rows
    M = x.shape[0]
    if x.shape[1] != K or out.shape[1] != N or out.shape[0] < M or x.stride(1) != 1 or not w.is_contiguous():
        raise core.KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if (G > 1 or group_offsets is not None) and (group_offsets is None or group_offsets.numel() != G + 1):
        raise core.KernelError("gemm_tc: group_offsets must have G + 1 entries")
    grouped = group_offsets is not None
    if bn is None:
        bn = token_tile(M / max(G, 1), True) if grouped else token_tile(min(M, 256))
    L = lib()
    n_tiles = -(-N // 128)
    gy = c_int(0)
    if splits is None:
        if bn > 64:
            # many tokens: the product is bound by the tensor cores and by L2, and the split-K
            # merge (one CTA re-reading every partial tile) costs more than it gains
            splits = 1
        else:
            # few tokens: the weight stream bounds the time; enough CTAs to keep every SM loading
            tiles = n_tiles * (max(1, -(-M // bn)) if not grouped else max(1, min(G, M)))
            # (up to 8 splits add up through the shared memory of a cluster; more would go through
            # partial sums in global memory)
            # (measured: about 1.5 CTAs per SM is best up to 32 tokens, where all clusters of a
            # launch then find room at once; 2 per SM at 64 tokens)
            # (a single sequence, i.e. one row, or up to four rows of routed experts: one CTA per SM;
            # 1.76 -> 1.70 ms a step at batch 1, while two sequences and more lose by it)
            one = M == 1 if not grouped else M <= 4
            target = num_sms(x.device) if one else 3 * num_sms(x.device) // 2 if bn <= 32 else 2 * num_sms(x.device)
            if _SPLIT_TARGET:                              # for measurements
                target = _SPLIT_TARGET
            splits = max(1, min(8, target // max(tiles, 1), -(-K // 64) // 4))
    splits = L.moe_gemm_tc_plan(K, int(splits), M, bn, G, 1 if grouped else 0, byref(gy))
    partials = tickets = None
    if splits > 1:
        ws = workspace(x.device)
        if gy.value * n_tiles > ws.TICKETS:
            splits = 1
        else:
            partials = ws.partials_for(splits * M * (2 * N if swiglu else N))
            tickets = ws.tickets
    code = L.moe_gemm_tc(x.data_ptr(), x.stride(0), w.data_ptr(), G, N, K, 1 if swiglu else 0, out.data_ptr(),
                         1 if out.dtype == torch.bfloat16 else 0, out.stride(0),
                         None if bias is None else bias.data_ptr(),
                         None if group_offsets is None else group_offsets.data_ptr(), M, bn, splits,
                         None if partials is None else partials.data_ptr(),
                         None if tickets is None else tickets.data_ptr(),
                         None if status is None else status.data_ptr(), 1 if early_offsets else 0, core._stream())
    if code == -1:
        return False
    core._ok(code, "gemm_tc")
    return True


def attention_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, batch, out: torch.Tensor, *, nh: int, nkv: int,
                      hd: int, window, scale: float, status=None) -> bool:
    """Causal (optionally windowed) attention of whole prompts on the tensor cores; every
    sequence of ``batch`` must start at position 0.  False if the head size is not taken.
    Head sizes 64 and 128 run on tcgen05 (``attention_prefill_tc.cu``), 16 and 32 on mma.sync."""
    if q.dtype != torch.bfloat16 or hd not in (16, 32, 64, 128):
        return False
    if hd in (64, 128) and status is not None and _ATTN_TC:
        code = lib().moe_attention_prefill_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                              batch.cu_seqlens.data_ptr(), batch.num_seqs, batch.num_tokens, nh, nkv,
                                              hd, int(window or 0), float(scale), status.data_ptr(), core._stream())
        if code != -1:
            core._ok(code, "attention_prefill_tc")
            return True
    code = lib().moe_attention_prefill_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                            batch.cu_seqlens.data_ptr(), batch.num_seqs, batch.num_tokens, nh, nkv,
                                            hd, int(window or 0), float(scale), core._stream())
    if code == -1:
        return False
    core._ok(code, "attention_prefill")
    return True


def attention_cached(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, view, batch, out: torch.Tensor, *,
                     nh: int, window, scale: float, status) -> bool:
    """Causal (optionally windowed) attention of a step whose sequences go on from the cache, on
    tcgen05: the keys before the step from the pages of ``view`` (one layer's cache), the step's own
    from ``k_new`` / ``v_new``.  False, with nothing launched, for what the kernel does not take
    (head sizes other than 64 and 128, another dtype or page size)."""
    g = view.group
    hd = g.head_dim
    if q.dtype != torch.bfloat16 or g.dtype != torch.bfloat16 or hd not in (64, 128) or not _ATTN_TC:
        return False
    code = lib().moe_attention_cached_tc(q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), view.k.data_ptr(),
                                         view.v.data_ptr(), out.data_ptr(), batch.cu_seqlens.data_ptr(),
                                         batch.seq_start.data_ptr(), batch.slots.data_ptr(), g.table.data_ptr(),
                                         g.table.stride(0), g.ring, g.page_size, g.num_pages, batch.num_seqs,
                                         batch.num_tokens, nh, g.num_kv_heads, hd, int(window or 0), float(scale),
                                         status.data_ptr(), core._stream())
    if code == -1:
        return False
    core._ok(code, "attention_cached_tc")
    return True


def gather_rows(src: torch.Tensor, rows: torch.Tensor, n: int, status) -> torch.Tensor:
    """dst[i] = src[rows[i]] for bf16 rows (expert dispatch)."""
    if src.dtype != torch.bfloat16 or src.shape[1] % 8:
        raise core.KernelError("gather_rows: bfloat16 rows of a multiple of 8 elements")
    dst = torch.empty((n, src.shape[1]), dtype=torch.bfloat16, device=src.device)
    core._ok(lib().moe_gather_rows_bf16(src.data_ptr(), rows.data_ptr(), dst.data_ptr(), n, src.shape[1],
                                        src.shape[0], status.data_ptr(), core._stream()), "gather_rows")
    return dst

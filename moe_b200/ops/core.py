"""Python face of the kernel library ``core``: argument checks, then one C call.

Every function launches on the current CUDA stream and returns at once.  There
is no fallback: a tensor on the CPU, a dtype the kernels do not take or a
library that cannot be built raises.
"""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build

DT_F32, DT_BF16 = 0, 1


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = build.load("core")
        P, I, F, LL = c_void_p, c_int, c_float, c_longlong
        sig = {
            "moe_embed": [P, I, P, P, I, I, I, P, P, P, P, P],
            "moe_rmsnorm": [P, P, P, P, P, P, I, I, I, F, I, P, P],
            "moe_rmsnorm_combine": [P, P, P, P, I, P, P, P, P, P, P, I, I, I, F, I, P, P],
            "moe_add_inplace": [P, P, LL, P],
            "moe_gemm_generic": [P, I, I, P, I, P, I, LL, P, I, I, P, P, I, I, I, I, P, P],
            "moe_rope_split": [P, P, P, I, I, I, I, I, P, P, P, I, P, P, P, P, P, P, I, I, I, I, P, P],
            "moe_kv_commit": [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, P, P],
            "moe_attention_generic": [P, P, P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P],
            "moe_router": [P, P, P, I, P, I, I, I, I, I, F, P, P, P, P, P, LL, P],
            "moe_router_logits": [P, P, P, I, I, I, I, P, P, LL, P],
            "moe_router_topk": [P, P, I, I, I, I, I, F, P, P, P, P],
            "moe_split3": [P, P, LL, I, P],
            "moe_route_dispatch": [P, P, I, I, I, I, I, F, P, P, P, P, P, P, P, P, I, P, P],
            "moe_rope_commit": [P, P, P, I, I, I, I, I, P, P, P, I, P, P, P, I, I, I, I, P, P],
            "moe_attention_decode": [P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P],
            "moe_attention_tiled": [P, P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P],
            "moe_attention_decode_fused": [P, P, I, P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P],
            "moe_norm_route": [P, P, P, F, I, I, P, P, P, P, I, I, I, I, F, P, P, P, P, P, P, P, P, P, P, P],
            "moe_align": [P, I, I, I, P, P, P, P, P],
            "moe_swiglu": [P, P, I, LL, I, P],
            "moe_combine": [P, P, P, I, P, P, P, I, I, P],
            "moe_sample": [P, I, I, P, P, P, I, F, I, F, F, P, P, P, LL, I, P],
            "moe_logprobs": [P, I, I, P, I, P, P, P, P],
            "moe_seed_rng": [P, P, P, I, P],
            "moe_table_update": [P, I, P, I, P],
        }
        for name, argtypes in sig.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        L.moe_router_scratch_floats.argtypes = [I, I, I, I]
        L.moe_router_scratch_floats.restype = LL
        L.moe_set_pdl.argtypes = [c_int]
        L.moe_set_pdl.restype = None
        if os.environ.get("MOE_B200_PDL", "1") == "0":      # programmatic dependent launch off
            L.moe_set_pdl(0)
        L.moe_set_norm_route_cluster.argtypes = [c_int]
        L.moe_set_norm_route_cluster.restype = None
        if os.environ.get("MOE_B200_NORM_ROUTE_CLUSTER", "1") == "0":   # ticket form also for few tokens
            L.moe_set_norm_route_cluster(0)
        _lib = L
    return _lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle.  (``torch.cuda.current_stream()`` builds a Python object on
    every call, which with hundreds of launches a step is milliseconds of host time.)"""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return DT_F32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _chk(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name}: expected {dims} dimensions, got {tuple(t.shape)}")
    return t


launches = 0   # kernels launched through this module since import (benchmarks read the difference)


def _ok(code: int, what: str):
    global launches
    launches += 1
    if code != 0:
        try:
            msg = torch.cuda.cudart().cudaGetErrorString(code)
        except Exception:
            msg = "?"
        raise KernelError(f"{what}: CUDA error {code} ({msg})")


# --------------------------------------------------------------------------- status word
STATUS_BITS = {
    1: "a token id lies outside the vocabulary",
    2: "a page table entry lies outside the page pool",
    4: "routing produced an expert id outside the expert range",
    8: "a bounded wait inside a kernel ran out",
    16: "a gather index lies outside its tensor",
}


# Where a bounded wait ran out (status[1]; the first one of a step): kernel and role, barrier.
WAIT_SITES = {
    0x10: "tensor-core product, one CTA a tile", 0x20: "tensor-core product, persistent",
    0x30: "tensor-core product, pairs of CTAs", 0x40: "tensor-core prompt attention",
}
WAIT_ROLES = {
    0x1: "producer: a free stage", 0x2: "producer: its own copies in flight", 0x3: "MMA issuer: a free accumulator",
    0x4: "MMA issuer: a loaded stage", 0x5: "epilogue: a finished accumulator",
}
WAIT_ROLES_ATTENTION = {
    0x1: "producer: a free key stage", 0x2: "producer: a free value stage", 0x3: "producer: its own copies in flight",
    0x4: "MMA issuer: the queries", 0x5: "MMA issuer: a key tile",
    0x7: "MMA issuer: a value tile", 0x8: "MMA issuer: P", 0x9: "softmax: the scores", 0xa: "softmax: its partner's maximum",
    0xb: "softmax: the last P V product", 0xc: "softmax: its partner's sum", 0xd: "softmax: the final P V product",
}


def wait_site(code: int) -> str:
    kernel, role = code & 0xf0, code & 0xf
    roles = WAIT_ROLES_ATTENTION if kernel == 0x40 else WAIT_ROLES
    return f"{WAIT_SITES.get(kernel, 'kernel ?')}, {roles.get(role, 'wait ?')} (site 0x{code:02x})"


def new_status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor):
    """Read the status word (synchronises) and raise if a kernel flagged a fault."""
    v, site = (int(x) for x in status[:2].tolist())
    if v:
        status.zero_()
        msg = "; ".join(m for b, m in STATUS_BITS.items() if v & b) or f"status {v}"
        if v & 8 and site:
            msg += f" [{wait_site(site)}]"
        raise KernelError(msg)


# --------------------------------------------------------------------------- kernels
def embed(table, token_ids, out, status, last_token=None, seq_of_token=None, slots=None):
    """out[t] = table[token_ids[t]]; with ``last_token`` (a per-slot table the sampler fills) a token
    id of -1 stands for the token sampled last for the row's sequence."""
    _chk(table, "table", dims=2), _chk(token_ids, "token_ids", torch.int32, 1), _chk(out, "out", torch.float32, 2)
    T, H = out.shape
    if token_ids.numel() < T or table.shape[1] != H:
        raise KernelError("embed: shape mismatch")
    if last_token is not None:
        _chk(last_token, "last_token", torch.int32, 1), _chk(seq_of_token, "seq_of_token", torch.int32, 1)
        _chk(slots, "slots", torch.int32, 1)
    _ok(lib().moe_embed(_p(table), _dt(table), _p(token_ids), _p(out), T, H, table.shape[0], _p(status),
                        _p(last_token), _p(seq_of_token), _p(slots), _stream()), "embed")


def rmsnorm(x, weight, eps, *, delta=None, rows=None, out32=None, out16=None, write_back=True, status=None):
    """y = rmsnorm(x[r] (+ delta[r])) for r in rows (or every row).

    With ``delta`` and ``write_back`` the sum is stored back into ``x`` (the
    32-bit residual stream).  ``out32`` / ``out16`` receive y in float32 /
    bfloat16; either may be None."""
    _chk(x, "x", torch.float32, 2), _chk(weight, "weight", torch.float32, 1)
    S, H = x.shape
    n_out = S if rows is None else rows.numel()
    if weight.numel() != H:
        raise KernelError("rmsnorm: weight size")
    if delta is not None:
        _chk(delta, "delta", torch.float32, 2)
        if delta.shape != x.shape:
            raise KernelError("rmsnorm: delta shape")
    if rows is not None:
        _chk(rows, "rows", torch.int32, 1)
    for o, dt in ((out32, torch.float32), (out16, torch.bfloat16)):
        if o is not None:
            _chk(o, "out", dt, 2)
            if o.shape[0] < n_out or o.shape[1] != H:
                raise KernelError("rmsnorm: output shape")
    _ok(lib().moe_rmsnorm(_p(x), _p(delta), _p(weight), _p(rows), _p(out32), _p(out16), n_out, S, H, float(eps),
                          1 if (write_back and rows is None) else 0, _p(status), _stream()), "rmsnorm")


def rmsnorm_combine(x, cd, weight, eps, *, rows=None, out32=None, out16=None, write_back=True, status=None) -> bool:
    """``rmsnorm`` whose delta is still the uncombined output of routed experts (``cd``: y,
    pos_of_pair, topk_w, top_k, shared, shared_gate): combined inside the norm's kernel.  False,
    with nothing launched, if the rows are not whole 16-byte units."""
    _chk(x, "x", torch.float32, 2), _chk(weight, "weight", torch.float32, 1), _chk(cd.y, "y", torch.float32, 2)
    S, H = x.shape
    n_out = S if rows is None else rows.numel()
    if weight.numel() != H or cd.y.shape[1] != H or cd.pos_of_pair.numel() < S * cd.top_k:
        raise KernelError("rmsnorm_combine: shapes")
    code = lib().moe_rmsnorm_combine(_p(x), _p(cd.y), _p(cd.pos_of_pair), _p(cd.topk_w), cd.top_k, _p(cd.shared),
                                     _p(cd.shared_gate), _p(weight), _p(rows), _p(out32), _p(out16), n_out, S, H,
                                     float(eps), 1 if (write_back and rows is None) else 0, _p(status), _stream())
    if code == -1:
        return False
    _ok(code, "rmsnorm_combine")
    return True


def add_inplace(a, b):
    _chk(a, "a", torch.float32), _chk(b, "b", torch.float32)
    if a.numel() != b.numel():
        raise KernelError("add_inplace: sizes differ")
    _ok(lib().moe_add_inplace(_p(a), _p(b), a.numel(), _stream()), "add_inplace")


def gemm_generic(a, w, out, *, bias=None, a_rows=None, group_offsets=None, status=None, m=None):
    """out[i, :] = a[row(i), :] @ w[g(i)].T (+ bias); the plain kernel, any sizes.

    a: [S, K]; w: [N, K] or [G, N, K]; out: [M, N].  ``a_rows`` int32[M] gathers
    rows of a; ``group_offsets`` int32[G+1] splits the M rows into groups."""
    _chk(a, "a", dims=2), _chk(out, "out", dims=2)
    if not w.is_cuda or not w.is_contiguous():
        raise KernelError("gemm: weight must be a contiguous CUDA tensor")
    if w.dim() == 2:
        G, (N, K) = 1, w.shape
    elif w.dim() == 3:
        G, N, K = w.shape
    else:
        raise KernelError("gemm: weight must be [N, K] or [G, N, K]")
    M = out.shape[0] if m is None else m
    if a.shape[1] != K or out.shape[1] != N or M > out.shape[0]:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if a_rows is None and a.shape[0] < M:
        raise KernelError("gemm: a has fewer rows than out")
    if a_rows is not None:
        _chk(a_rows, "a_rows", torch.int32, 1)
        if a_rows.numel() < M:
            raise KernelError("gemm: a_rows too short")
    if group_offsets is not None:
        _chk(group_offsets, "group_offsets", torch.int32, 1)
        if group_offsets.numel() != G + 1:
            raise KernelError("gemm: group_offsets must have G + 1 entries")
    elif G != 1:
        raise KernelError("gemm: a stacked weight needs group_offsets")
    if bias is not None:
        _chk(bias, "bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError("gemm: bias size")
    _ok(lib().moe_gemm_generic(_p(a), _dt(a), a.stride(0), _p(a_rows), a.shape[0], _p(w), _dt(w), N * K, _p(out),
                               _dt(out), out.stride(0), _p(bias), _p(group_offsets), G, M, N, K, _p(status),
                               _stream()), "gemm_generic")


def rope_split(qkv, pos, inv_freq, nh, nkv, hd, rot, q, k, v, commit=None, status=None):
    """Rotate and split a step's projections.  ``commit=(view, batch)``: also append the keys and
    values to that cache layer in the same launch (only for a step whose attention reads nothing
    from the cache); returns False if this was asked for and the sizes do not allow it (nothing is
    launched then), else True."""
    _chk(qkv, "qkv", torch.float32, 2), _chk(pos, "pos", torch.int32, 1)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError("rope_split: qkv width")
    for t, n in ((q, nh), (k, nkv), (v, nkv)):
        _chk(t, "q/k/v")
        if t.numel() < T * n * hd or t.dtype != q.dtype:
            raise KernelError("rope_split: output size or dtype")
    if rot:
        _chk(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() < rot // 2:
            raise KernelError("rope_split: inv_freq too short")
    if commit is not None:
        view, batch = commit
        g = view.group
        if k.dtype != g.dtype or g.num_kv_heads != nkv or g.head_dim != hd:
            raise KernelError("rope_split: the cache layer differs from the keys in dtype or shape")
        code = lib().moe_rope_split(_p(qkv), _p(pos), _p(inv_freq) if rot else None, T, nh, nkv, hd, rot, _p(q),
                                    _p(k), _p(v), _dt(q), _p(view.k), _p(view.v), _p(batch.seq_of_token),
                                    _p(batch.seq_end), _p(batch.slots), _p(g.table), g.table.stride(0), g.ring,
                                    g.page_size, g.num_pages, _p(status), _stream())
        if code == -1:
            return False
        _ok(code, "rope_split")
        return True
    _ok(lib().moe_rope_split(_p(qkv), _p(pos), _p(inv_freq) if rot else None, T, nh, nkv, hd, rot, _p(q), _p(k), _p(v),
                             _dt(q), None, None, None, None, None, None, 0, 0, 0, 0, None, _stream()), "rope_split")
    return True


def kv_commit(k_new, v_new, view, batch, status):
    """Append the step's keys and values to the cache layer ``view``."""
    g = view.group
    T = batch.num_tokens
    if k_new.dtype != g.dtype:
        raise KernelError("kv_commit: cache dtype differs from the keys'")
    _ok(lib().moe_kv_commit(_p(k_new), _p(v_new), _p(view.k), _p(view.v), _dt(k_new), _p(batch.seq_of_token),
                            _p(batch.pos), _p(batch.seq_end), _p(batch.slots), _p(g.table), g.table.stride(0),
                            g.ring, g.page_size, g.num_pages, T, g.num_kv_heads, g.head_dim, _p(status), _stream()),
        "kv_commit")


def attention_generic(q, k_new, v_new, view, batch, out, *, nh, window, scale, use_local, status):
    g = view.group
    T = batch.num_tokens
    if q.dtype != g.dtype or out.dtype != q.dtype:
        raise KernelError("attention: dtypes of queries, cache and output must agree")
    _ok(lib().moe_attention_generic(_p(q), _p(k_new), _p(v_new), _p(view.k), _p(view.v), _p(out), _dt(q),
                                    _p(batch.seq_of_token), _p(batch.pos), _p(batch.seq_start), _p(batch.cu_seqlens),
                                    _p(batch.slots), _p(g.table), g.table.stride(0), g.ring, g.page_size,
                                    g.num_pages, T, nh, g.num_kv_heads, g.head_dim, int(window or 0), float(scale),
                                    1 if use_local else 0, _p(status), _stream()), "attention_generic")


def attention_tiled(q, k_new, v_new, view, batch, out, *, nh, window, scale, use_local, status) -> bool:
    """The same as ``attention_generic`` with 64 queries of a (sequence, head) to a block and the
    keys staged through shared memory (32-bit arithmetic on the CUDA cores).  False, with nothing
    launched, for a layout it does not take (a page size other than 64, unaligned rows)."""
    g = view.group
    if q.dtype != g.dtype or out.dtype != q.dtype:
        raise KernelError("attention: dtypes of queries, cache and output must agree")
    code = lib().moe_attention_tiled(_p(q), _p(k_new), _p(v_new), _p(view.k), _p(view.v), _p(out), _dt(q),
                                     _p(batch.cu_seqlens), _p(batch.seq_start), _p(batch.slots), _p(g.table),
                                     g.table.stride(0), g.ring, g.page_size, g.num_pages, batch.num_seqs,
                                     batch.num_tokens, nh, g.num_kv_heads, g.head_dim, int(window or 0), float(scale),
                                     1 if use_local else 0, _p(status), _stream())
    if code == -1:
        return False
    _ok(code, "attention_tiled")
    return True


def router(h32, w_router, top_k, norm_topk, scale, topk_idx, topk_w, *, shared_gate_w=None, shared_gate=None,
           seq_of_token=None):
    _chk(h32, "h", torch.float32, 2), _chk(w_router, "router weight", dims=2)
    T, H = h32.shape
    E = w_router.shape[0]
    if w_router.shape[1] != H:
        raise KernelError("router: weight shape")
    _chk(topk_idx, "topk_idx", torch.int32), _chk(topk_w, "topk_w", torch.float32)
    if topk_idx.numel() < T * top_k or topk_w.numel() < T * top_k:
        raise KernelError("router: output size")
    if shared_gate_w is not None:
        _chk(shared_gate_w, "shared gate weight")
        if shared_gate_w.dtype != w_router.dtype or shared_gate_w.numel() != H:
            raise KernelError("router: the shared gate weight must have the router's dtype and width")
        _chk(shared_gate, "shared_gate", torch.float32)
    logits = torch.empty((T, E + (1 if shared_gate_w is not None else 0)), dtype=torch.float32, device=h32.device)
    need = lib().moe_router_scratch_floats(T, H, E, 1 if shared_gate_w is not None else 0)
    scratch = torch.empty((need,), dtype=torch.float32, device=h32.device) if need else None
    _ok(lib().moe_router(_p(h32), _p(w_router), _p(shared_gate_w), _dt(w_router), _p(seq_of_token), T, H, E, top_k,
                         1 if norm_topk else 0, float(scale), _p(logits), _p(topk_idx), _p(topk_w), _p(shared_gate),
                         _p(scratch), need, _stream()), "router")


def split3(x32: torch.Tensor) -> torch.Tensor:
    """[T, H] float32 -> [T, 3 H] bfloat16 with x = p0 + p1 + p2 exactly (three terms of 8 bits)."""
    _chk(x32, "x", torch.float32, 2)
    T, H = x32.shape
    out = torch.empty((T, 3 * H), dtype=torch.bfloat16, device=x32.device)
    _ok(lib().moe_split3(_p(x32), _p(out), T, H, _stream()), "split3")
    return out


def router_topk(logits, top_k, norm_topk, scale, topk_idx, topk_w, *, num_experts, shared_gate=None, seq_of_token=None):
    """Picks and weights from logits [T, E (+ 1 row for the shared gate)] that are already there."""
    _chk(logits, "logits", torch.float32, 2)
    T = logits.shape[0]
    gate_row = logits.shape[1] == num_experts + 1
    if logits.shape[1] not in (num_experts, num_experts + 1) or (gate_row and shared_gate is None):
        raise KernelError("router_topk: logits must have one column per expert (and one for the shared gate)")
    _ok(lib().moe_router_topk(_p(logits), _p(seq_of_token), T, num_experts, 1 if gate_row else 0, top_k,
                              1 if norm_topk else 0, float(scale), _p(topk_idx), _p(topk_w), _p(shared_gate), _stream()),
        "router_topk")


_SMS = {}


_DECODE_CTAS = None


def decode_splits(device, num_tokens: int, nkv: int, max_end: int = 0) -> int:
    """Key splits of the decode attention: about four small CTAs per SM (each is a chain of
    dependent loads, so many must be in flight), but no more than leave each of a CTA's four warps
    a tile of 32 keys of the longest sequence (``max_end``, 0 if unknown): with a short context and
    one sequence, 32 splits of one tile each cost more in the merge than they gain."""
    idx = torch.device(device).index or 0
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(device).multi_processor_count
    global _DECODE_CTAS
    if _DECODE_CTAS is None:
        _DECODE_CTAS = int(os.environ.get("MOE_B200_DECODE_CTAS", "4"))
    per_sm = _DECODE_CTAS
    n = max(1, min(32, (per_sm * _SMS[idx]) // max(1, num_tokens * nkv)))
    if max_end > 0:
        n = min(n, max(1, -(-max_end // 32) // 4))
    return n


def _head_blocks(nh: int, nkv: int) -> int:
    """Blocks along the heads of the decode attention's grid: a kv head's query heads two at a time."""
    group = max(1, nh // max(nkv, 1))
    return nkv * (1 if group == 1 else -(-group // 2))


def attention_decode(q, view, batch, out, *, nh, window, scale, status):
    """Attention of one new token per sequence over the cache alone (its own key already
    appended); split along the keys and merged."""
    g = view.group
    T = batch.num_tokens
    if q.dtype != g.dtype or out.dtype != q.dtype:
        raise KernelError("attention: dtypes of queries, cache and output must agree")
    nsplit = decode_splits(q.device, T, _head_blocks(nh, g.num_kv_heads), getattr(batch, "max_end", 0))
    partial = torch.empty(T * nh * nsplit * (g.head_dim + 2), dtype=torch.float32, device=q.device)
    _ok(lib().moe_attention_decode(_p(q), _p(view.k), _p(view.v), _p(out), _p(partial), _dt(q),
                                   _p(batch.seq_of_token), _p(batch.pos), _p(batch.slots), _p(g.table),
                                   g.table.stride(0), g.ring, g.page_size, g.num_pages, T, nh, g.num_kv_heads,
                                   g.head_dim, int(window or 0), float(scale), nsplit, _p(status), _stream()),
        "attention_decode")


_TICKETS = {}


def _tickets(device, n: int) -> torch.Tensor:
    """Zeroed counters that kernels with a 'last CTA finishes the job' step use and leave zero."""
    idx = torch.device(device).index or 0
    t = _TICKETS.get(idx)
    if t is None or t.numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the ticket array must be sized before a CUDA graph is captured")
        t = _TICKETS[idx] = torch.zeros(max(n, 1 << 14), dtype=torch.int32, device=device)
    return t


def attention_decode_fused(qkv, inv_freq, rot, view, batch, out, *, nh, window, scale, status) -> bool:
    """One token per sequence, ONE launch: rotate the step's q/k/v rows, append key and value to
    the cache layer ``view``, attend over the cache split along the keys, merge.  False (nothing
    launched) if the head size is not one the fast kernel takes."""
    _chk(qkv, "qkv", torch.float32, 2)
    g = view.group
    T = batch.num_tokens
    if qkv.shape[1] != (nh + 2 * g.num_kv_heads) * g.head_dim or out.dtype != g.dtype:
        raise KernelError("attention_decode_fused: shapes or dtypes do not fit the cache")
    if rot:
        _chk(inv_freq, "inv_freq", torch.float32, 1)
    nsplit = decode_splits(qkv.device, T, _head_blocks(nh, g.num_kv_heads), getattr(batch, "max_end", 0))
    partial = torch.empty(T * nh * nsplit * (g.head_dim + 2), dtype=torch.float32, device=qkv.device)
    tickets = _tickets(qkv.device, T * g.num_kv_heads)
    code = lib().moe_attention_decode_fused(_p(qkv), _p(inv_freq) if rot else None, rot, _p(view.k), _p(view.v),
                                            _p(out), _p(partial), _p(tickets), _dt(out), _p(batch.seq_of_token),
                                            _p(batch.pos), _p(batch.slots), _p(g.table), g.table.stride(0), g.ring,
                                            g.page_size, g.num_pages, T, nh, g.num_kv_heads, g.head_dim,
                                            int(window or 0), float(scale), nsplit, _p(status), _stream())
    if code == -1:
        return False
    _ok(code, "attention_decode_fused")
    return True


def moe_align(topk_idx, num_tokens, top_k, num_experts, offsets, sorted_token, pos_of_pair, status):
    for t in (topk_idx, offsets, sorted_token, pos_of_pair):
        _chk(t, "align", torch.int32)
    if offsets.numel() != num_experts + 1 or sorted_token.numel() < num_tokens * top_k:
        raise KernelError("moe_align: output size")
    _ok(lib().moe_align(_p(topk_idx), num_tokens, top_k, num_experts, _p(offsets), _p(sorted_token), _p(pos_of_pair),
                        _p(status), _stream()), "moe_align")


def swiglu(gu, act):
    _chk(gu, "gu", torch.float32, 2), _chk(act, "act", dims=2)
    rows, two_i = gu.shape
    if two_i % 2 or act.shape != (rows, two_i // 2):
        raise KernelError("swiglu: shapes")
    _ok(lib().moe_swiglu(_p(gu), _p(act), _dt(act), rows, two_i // 2, _stream()), "swiglu")


def moe_combine(y, pos_of_pair, topk_w, top_k, out, *, shared=None, shared_gate=None):
    _chk(y, "y", torch.float32, 2), _chk(out, "out", torch.float32, 2)
    T, H = out.shape
    _ok(lib().moe_combine(_p(y), _p(pos_of_pair), _p(topk_w), top_k, _p(shared), _p(shared_gate), _p(out), T, H,
                          _stream()), "moe_combine")


_sample_ws = {}


def sample(logits, slots, rng_states, out_tokens, *, temp=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, history=None,
           last_token=None, kernel=None):
    """One token per row of ``logits``.  ``kernel="global"`` takes the kernel that works over global
    memory whatever the vocabulary (otherwise only a vocabulary too large for a cluster's shared
    memory does)."""
    _chk(logits, "logits", torch.float32, 2), _chk(out_tokens, "out_tokens", torch.int32, 1)
    R, V = logits.shape
    if temp > 0:
        _chk(slots, "slots", torch.int32, 1), _chk(rng_states, "rng_states", torch.int64, 1)
    if last_token is not None:
        _chk(last_token, "last_token", torch.int32, 1), _chk(slots, "slots", torch.int32, 1)
        if slots.numel() < R:
            raise KernelError("sample: fewer slots than rows")
    hl = 0
    if history is not None:
        _chk(history, "history", torch.int32, 2)
        hl = history.shape[1]
    if out_tokens.numel() < R:
        raise KernelError("sample: fewer places for tokens than rows")
    ws = _sample_ws.get(logits.device)
    if ws is None or ws.numel() < 2 * R:       # zeroed once; the kernels leave it zeroed
        ws = _sample_ws[logits.device] = torch.zeros(max(2 * R, 512), dtype=torch.int64, device=logits.device)
    _ok(lib().moe_sample(_p(logits), R, V, _p(slots), _p(rng_states), _p(history), hl, float(temp), int(top_k),
                         float(top_p), float(repeat_penalty), _p(out_tokens), _p(last_token), _p(ws), ws.numel() * 8,
                         1 if kernel == "global" else 0, _stream()), "sample")


def logprobs(logits, tokens, top: int):
    """What the model thought of the committed ``tokens`` [rows], from the raw ``logits`` [rows, vocab]:
    (logprob [rows] float32, ids [rows, top] int32, logprobs [rows, top] float32), the ``top`` most
    likely tokens strongest first (reference: src/generate.rs:91-105)."""
    _chk(logits, "logits", torch.float32, 2), _chk(tokens, "tokens", torch.int32, 1)
    R, V = logits.shape
    if tokens.numel() < R or not 0 <= top <= 64:
        raise KernelError("logprobs: fewer tokens than rows, or more than 64 alternatives")
    lp = torch.empty(R, dtype=torch.float32, device=logits.device)
    ids = torch.empty((R, top), dtype=torch.int32, device=logits.device)
    lps = torch.empty((R, top), dtype=torch.float32, device=logits.device)
    _ok(lib().moe_logprobs(_p(logits), R, V, _p(tokens), top, _p(lp), _p(ids) if top else None,
                           _p(lps) if top else None, _stream()), "logprobs")
    return lp, ids, lps


def seed_rng(rng_states, slots, seeds):
    _chk(rng_states, "rng_states", torch.int64, 1), _chk(slots, "slots", torch.int32, 1)
    _chk(seeds, "seeds", torch.int64, 1)
    _ok(lib().moe_seed_rng(_p(rng_states), _p(slots), _p(seeds), slots.numel(), _stream()), "seed_rng")


def table_update(table, updates, n):
    """table[slot, index] = page for the first n (slot, index, page) triples of ``updates``."""
    _chk(table, "table", torch.int32, 2), _chk(updates, "updates", torch.int32)
    if updates.numel() < 3 * n:
        raise KernelError("table_update: updates too short")
    _ok(lib().moe_table_update(_p(table), table.stride(0), _p(updates), n, _stream()), "table_update")


def rope_commit(qkv, pos, inv_freq, nh, nkv, hd, rot, q, view, batch, status):
    """Decode step: rotate, write the queries, and append keys and values straight into the
    cache layer ``view`` (one launch instead of rope_split + kv_commit)."""
    _chk(qkv, "qkv", torch.float32, 2), _chk(pos, "pos", torch.int32, 1)
    g = view.group
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd or nkv != g.num_kv_heads or hd != g.head_dim or q.dtype != g.dtype:
        raise KernelError("rope_commit: shapes or dtypes do not fit the cache")
    if rot:
        _chk(inv_freq, "inv_freq", torch.float32, 1)
    _ok(lib().moe_rope_commit(_p(qkv), _p(pos), _p(inv_freq) if rot else None, T, nh, nkv, hd, rot, _p(q), _p(view.k),
                              _p(view.v), _dt(q), _p(batch.seq_of_token), _p(batch.slots), _p(g.table),
                              g.table.stride(0), g.ring, g.page_size, g.num_pages, _p(status), _stream()),
        "rope_commit")


def norm_route(x, delta, norm_w, eps, w_router, top_k, norm_topk, scale, *, bf16, shared_gate_w=None,
               seq_of_token=None, status=None):
    """Few tokens: ``x += delta``, RMS norm, router logits, pick, table inversion and gather of the
    normalised bfloat16 rows in ONE launch.  Returns None (nothing launched) for sizes the kernel
    does not take, else (out32 or None, out16 or None, topk_idx, topk_w, shared_gate, offsets,
    sorted_token, pos_of_pair, gathered or None)."""
    _chk(x, "x", torch.float32, 2), _chk(norm_w, "norm weight", torch.float32, 1), _chk(w_router, "router weight", dims=2)
    T, H = x.shape
    E = w_router.shape[0]
    if T > 64 or E > 256 or T * top_k > 4096 or norm_w.numel() != H or w_router.shape[1] != H:
        return None
    dev = x.device
    out16 = torch.empty((T, H), dtype=torch.bfloat16, device=dev) if bf16 else None
    out32 = None if bf16 else torch.empty((T, H), dtype=torch.float32, device=dev)
    P_ = T * top_k
    topk_idx = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    topk_w = torch.empty((T, top_k), dtype=torch.float32, device=dev)
    sg = torch.empty((T,), dtype=torch.float32, device=dev) if shared_gate_w is not None else None
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    sorted_token = torch.empty((P_,), dtype=torch.int32, device=dev)
    pos_of_pair = torch.empty((P_,), dtype=torch.int32, device=dev)
    xs = torch.empty((P_, H), dtype=torch.bfloat16, device=dev) if bf16 and (H * 2) % 16 == 0 else None
    ticket = _tickets(dev, 1)
    code = lib().moe_norm_route(_p(x), _p(delta), _p(norm_w), float(eps), H, T, _p(out32), _p(out16), _p(w_router),
                                _p(shared_gate_w), _dt(w_router), E, top_k, 1 if norm_topk else 0, float(scale),
                                _p(seq_of_token), _p(topk_idx), _p(topk_w), _p(sg), _p(offsets), _p(sorted_token),
                                _p(pos_of_pair), _p(xs), _p(ticket), _p(status), _stream())
    if code == -1:
        return None
    _ok(code, "norm_route")
    return out32, out16, topk_idx, topk_w, sg, offsets, sorted_token, pos_of_pair, xs


def route_dispatch(h32, w_router, top_k, norm_topk, scale, *, shared_gate_w=None, seq_of_token=None, gather=None,
                   status=None):
    """Few tokens (<= 64) and <= 256 experts: router logits, then pick + table inversion + gather in
    ONE more launch.  Returns (topk_idx, topk_w, shared_gate, offsets, sorted_token, pos_of_pair,
    gathered) where ``gathered[p] = gather[sorted_token[p]]`` (or None)."""
    _chk(h32, "h", torch.float32, 2), _chk(w_router, "router weight", dims=2)
    T, H = h32.shape
    E = w_router.shape[0]
    dev = h32.device
    rows = E + (1 if shared_gate_w is not None else 0)
    logits = torch.empty((T, rows), dtype=torch.float32, device=dev)
    _ok(lib().moe_router_logits(_p(h32), _p(w_router), _p(shared_gate_w), _dt(w_router), T, H, E, _p(logits), None, 0,
                                _stream()), "router_logits")
    P_ = T * top_k
    topk_idx = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    topk_w = torch.empty((T, top_k), dtype=torch.float32, device=dev)
    sg = torch.empty((T,), dtype=torch.float32, device=dev) if shared_gate_w is not None else None
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    sorted_token = torch.empty((P_,), dtype=torch.int32, device=dev)
    pos_of_pair = torch.empty((P_,), dtype=torch.int32, device=dev)
    xs, row_bytes = None, 0
    if gather is not None:
        _chk(gather, "gather", dims=2)
        row_bytes = gather.shape[1] * gather.element_size()
        if row_bytes % 16:
            gather, row_bytes = None, 0
        else:
            xs = torch.empty((P_, gather.shape[1]), dtype=gather.dtype, device=dev)
    _ok(lib().moe_route_dispatch(_p(logits), _p(seq_of_token), T, E, 1 if shared_gate_w is not None else 0, top_k,
                                 1 if norm_topk else 0, float(scale), _p(topk_idx), _p(topk_w), _p(sg), _p(offsets),
                                 _p(sorted_token), _p(pos_of_pair), _p(gather), _p(xs), row_bytes, _p(status),
                                 _stream()), "route_dispatch")
    return topk_idx, topk_w, sg, offsets, sorted_token, pos_of_pair, xs

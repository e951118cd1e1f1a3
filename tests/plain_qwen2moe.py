"""A plain, slow implementation of Qwen2 MoE, written from the reference's formulas.

Whole sequences, no cache, one function per part, float64 arithmetic on the CPU
(except the rotary angle, which the reference forms in float32).  It shares no
code with ``moe_b200``: it reads config.json and model.safetensors itself.

Anchoring: ``tests/golden`` holds logits computed by the reference's own
``scripts/oracle.py`` on a tiny random model; ``test_plain.py`` compares this
file with them.  The oracle cannot express q/k/v bias, the gated shared expert
and ``decoder_sparse_step``; those rest on the formulas cited below.

Every citation is ``file:line`` inside the JGalego/Moe source tree.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch

F64 = torch.float64


# --------------------------------------------------------------------------- files
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """u64 header length, JSON header, payload (src/store.rs:80-119).  Floats -> float64."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    head = json.loads(raw[8:8 + hlen])
    out = {}
    for name, v in head.items():
        if name == "__metadata__":
            continue
        b, e = v["data_offsets"]
        blob = raw[8 + hlen + b:8 + hlen + e]
        if v["dtype"] == "F32":
            a = np.frombuffer(blob, dtype="<f4").astype(np.float64)
        elif v["dtype"] == "BF16":
            # bf16 -> f32 is bits << 16 (src/quant.rs:189-193)
            a = (np.frombuffer(blob, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif v["dtype"] == "F16":
            a = np.frombuffer(blob, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {v['dtype']}")
        out[name] = torch.from_numpy(a.copy()).reshape(v["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    for n in sorted(os.listdir(model_dir)):
        if n.endswith(".safetensors"):
            w.update(read_safetensors(os.path.join(model_dir, n)))
    return cfg, w


# --------------------------------------------------------------------------- config
def layer_windows(cfg: dict) -> List[Optional[int]]:
    """src/spec.rs:422-444: no window -> none; layer_types; use_sliding_window false -> none;
    else layers l >= max_window_layers are windowed."""
    n = cfg["num_hidden_layers"]
    w = cfg.get("sliding_window") or 0
    if not w:
        return [None] * n
    types = cfg.get("layer_types")
    if types:
        return [w if (l < len(types) and types[l] in ("sliding_attention", "local_attention")) else None
                for l in range(n)]
    if not cfg.get("use_sliding_window", False):
        return [None] * n
    frm = cfg.get("max_window_layers", 0)
    return [w if l >= frm else None for l in range(n)]


def layer_is_sparse(cfg: dict, l: int) -> bool:
    """Routed iff experts exist, l is not in mlp_only_layers and (l+1) % decoder_sparse_step == 0.
    (The reference decides by tensor presence, src/model.rs:422; with random weights the
    configuration has to say.)"""
    if cfg.get("num_experts", 0) <= 0 or l in (cfg.get("mlp_only_layers") or []):
        return False
    return (l + 1) % cfg.get("decoder_sparse_step", 1) == 0


def head_dim_of(cfg: dict) -> int:
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


# --------------------------------------------------------------------------- parts
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """src/model.rs:211-216: x / sqrt(mean(x^2) + eps) * w, row-wise."""
    s = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * s * w


def rope_inv_freq(theta: float, dim: int) -> torch.Tensor:
    """src/spec.rs:89-96: theta^(-2i/dim), i < dim/2, as float32 values."""
    i = np.arange(dim // 2, dtype=np.float32)
    expo = (np.float32(-2.0) * i / np.float32(dim)).astype(np.float64)
    return torch.from_numpy(np.power(np.float64(np.float32(theta)), expo).astype(np.float32))


def rope(x: torch.Tensor, positions: torch.Tensor, inv: torch.Tensor) -> torch.Tensor:
    """src/model.rs:324-333: half-split pairs (i, i + d/2); angle = f32(pos) * inv[i] in float32.
    x: [T, heads, d]."""
    half = x.shape[-1] // 2
    ang = (positions.to(torch.float32)[:, None] * inv[None, :]).to(F64)     # float32 product, then widened
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def attention(q, k, v, window: Optional[int]) -> torch.Tensor:
    """src/model.rs:794-827: scale 1/sqrt(d); query p sees [max(0, p+1-w), p]; softmax subtracts
    the max; kv head = h / (heads / kv_heads).  q: [T, nh, d], k, v: [T, nkv, d] -> [T, nh*d]."""
    T, nh, d = q.shape
    rep = nh // k.shape[1]
    out = torch.zeros(T, nh, d, dtype=F64)
    scale = 1.0 / math.sqrt(d)
    for p in range(T):
        lo = max(0, p + 1 - window) if window else 0
        for h in range(nh):
            kh = h // rep
            s = (k[lo:p + 1, kh] @ q[p, h]) * scale
            s = torch.exp(s - s.max())
            s = s / s.sum()
            out[p, h] = s @ v[lo:p + 1, kh]
    return out.reshape(T, nh * d)


def attention_block(cfg, w, p, n, positions, window) -> torch.Tensor:
    """src/model.rs:704-734, 829-833: projections (+ bias when the tensor exists), rotary on q and
    k, attention, output projection without bias."""
    nh, nkv, d = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"]), head_dim_of(cfg)
    T = n.shape[0]

    def proj(name):
        y = n @ w[p + f"self_attn.{name}.weight"].T
        b = w.get(p + f"self_attn.{name}.bias")
        return y + b if b is not None else y

    inv = rope_inv_freq(cfg.get("rope_theta", 10000.0), d)
    q = rope(proj("q_proj").reshape(T, nh, d), positions, inv)
    k = rope(proj("k_proj").reshape(T, nkv, d), positions, inv)
    v = proj("v_proj").reshape(T, nkv, d)
    return attention(q, k, v, window) @ w[p + "self_attn.o_proj.weight"].T


def swiglu_mlp(w, prefix, n) -> torch.Tensor:
    """src/model.rs:26-35: down(silu(gate n) * up n), silu(a) = a / (1 + exp(-a))."""
    g = n @ w[prefix + "gate_proj.weight"].T
    u = n @ w[prefix + "up_proj.weight"].T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w[prefix + "down_proj.weight"].T


def route(cfg, w, p, n, forced=None):
    """src/model.rs:844-897: softmax over all experts, top k by descending score (tie: lower index,
    scripts/oracle.py:323), w = max(sc, 0), optional renormalisation by max(sum, 1e-20), scaling.
    ``forced`` ([T][k] expert ids) replaces the pick and keeps the rest, in the manner of the
    reference's routing overrides (src/model.rs:238-252)."""
    logits = n @ w[p + "mlp.gate.weight"].T
    sc = torch.softmax(logits, dim=-1)
    k = cfg["num_experts_per_tok"]
    picks, weights = [], []
    for i in range(n.shape[0]):
        order = sorted(range(sc.shape[1]), key=lambda e: (-float(sc[i, e]), e))[:k]
        if forced is not None:
            order = [int(e) for e in forced[i]]
        ww = torch.stack([sc[i, e].clamp(min=0.0) for e in order])
        if cfg.get("norm_topk_prob", False):
            ww = ww / ww.sum().clamp(min=1e-20)
        ww = ww * cfg.get("routed_scaling_factor", 1.0)
        picks.append(order)
        weights.append(ww)
    return picks, weights


def moe_block(cfg, w, p, n, trace=None, forced=None) -> torch.Tensor:
    """src/model.rs:902-970: weighted sum of the picked experts, then the shared expert scaled by
    sigmoid(shared_expert_gate . n)."""
    picks, weights = route(cfg, w, p, n, forced)
    if trace is not None:
        trace.append((picks, weights))
    out = torch.zeros_like(n)
    for i in range(n.shape[0]):
        for e, ww in zip(picks[i], weights[i]):
            out[i] += ww * swiglu_mlp(w, p + f"mlp.experts.{e}.", n[i:i + 1])[0]
    if p + "mlp.shared_expert.gate_proj.weight" in w:
        y = swiglu_mlp(w, p + "mlp.shared_expert.", n)
        g = w.get(p + "mlp.shared_expert_gate.weight")
        if g is not None:
            y = y * (1.0 / (1.0 + torch.exp(-(n @ g.T))))
        out = out + y
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], trace=None, forced=None) -> torch.Tensor:
    """Logits [T, vocab] for every position of one whole sequence (src/model.rs:646-687, 578-589).
    ``trace`` (a list) receives (picks, weights) per routed layer; ``forced`` (one [T][k] list per
    routed layer, in layer order) fixes the picks."""
    forced = list(forced) if forced is not None else None
    eps = cfg.get("rms_norm_eps", 1e-6)
    wins = layer_windows(cfg)
    positions = torch.arange(len(tokens))
    x = w["model.embed_tokens.weight"][torch.tensor(tokens)].clone()
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        n = rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        x = x + attention_block(cfg, w, p, n, positions, wins[l])
        n = rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
        if layer_is_sparse(cfg, l):
            x = x + moe_block(cfg, w, p, n, trace, forced.pop(0) if forced is not None else None)
        else:
            x = x + swiglu_mlp(w, p + "mlp.", n)
    nx = rmsnorm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return nx @ head.T


# --------------------------------------------------------------------------- sampling
class Rng:
    """xorshift64* (src/sample.rs:4-19)."""

    def __init__(self, seed: int):
        self.s = ((seed * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF) | 1

    def next_f32(self) -> float:
        x = self.s
        x ^= x >> 12
        x ^= (x << 25) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 27
        self.s = x
        return float(np.float32(((x * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF) >> 40) / np.float32(1 << 24))


def sample(logits: np.ndarray, history: List[int], rng: Rng, temp=0.0, top_p=0.95, top_k=0, repeat_penalty=1.0,
           repeat_window=64) -> int:
    """src/sample.rs:80-140, in float32 as there."""
    l = np.array(logits, dtype=np.float32).copy()
    if repeat_penalty != 1.0:
        for t in list(reversed(history))[:repeat_window]:
            l[t] = l[t] / np.float32(repeat_penalty) if l[t] > 0 else l[t] * np.float32(repeat_penalty)
    if temp <= 0.0:
        return int(np.argmax(l))                       # the first maximum (strict > in the reference)
    k = len(l) if top_k == 0 else min(top_k, len(l))
    idx = np.lexsort((np.arange(len(l)), -l))[:k]      # descending; equal logits by index
    mx = l[idx[0]]
    probs = np.exp((l[idx] - mx) / np.float32(temp)).astype(np.float32)
    probs = probs / np.cumsum(probs, dtype=np.float32)[-1]
    if 0.0 < top_p < 1.0:
        acc = np.cumsum(probs, dtype=np.float32)       # sequential float32 sum, as the reference's loop
        hit = acc >= np.float32(top_p)
        cut = int(np.argmax(hit)) + 1 if hit.any() else len(probs)
        probs, idx = probs[:cut], idx[:cut]
        probs = probs / np.cumsum(probs, dtype=np.float32)[-1]
    if len(idx) == 1:
        return int(idx[0])
    r = np.float32(rng.next_f32())
    hit = r < np.cumsum(probs, dtype=np.float32)
    return int(idx[int(np.argmax(hit))]) if hit.any() else int(idx[-1])

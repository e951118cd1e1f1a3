"""Tiny configurations, model folders and replay cuts shared by the tests."""
from __future__ import annotations

import copy
import os
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_qwen2moe as plain

# Two tiny configurations of the architecture that differ in every size and option.
CONFIG_A = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=64,
    norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[], intermediate_size=128,
    vocab_size=256, rope_theta=1e4, rms_norm_eps=1e-6, use_sliding_window=False, tie_word_embeddings=False,
    max_position_embeddings=4096, eos_token_id=255,
)
CONFIG_B = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
    num_experts=8, num_experts_per_tok=3, moe_intermediate_size=48, shared_expert_intermediate_size=128,
    norm_topk_prob=True, decoder_sparse_step=2, mlp_only_layers=[2], intermediate_size=160,
    vocab_size=384, rope_theta=1e6, rms_norm_eps=1e-5, use_sliding_window=True, sliding_window=8,
    max_window_layers=1, tie_word_embeddings=True, max_position_embeddings=4096, eos_token_id=[7, 383],
)
# heads of 64 (the tcgen05 prompt attention and the fastest decode kernels take this size), grouped
# 2:1, a window of 70 that crosses a page of 64 on the second layer, sizes that are no power of two
CONFIG_C = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=2, hidden_size=160, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
    num_experts=5, num_experts_per_tok=2, moe_intermediate_size=40, shared_expert_intermediate_size=72,
    norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[], intermediate_size=96,
    vocab_size=300, rope_theta=5e4, rms_norm_eps=1e-6, use_sliding_window=True, sliding_window=70,
    max_window_layers=1, tie_word_embeddings=False, max_position_embeddings=4096, eos_token_id=299,
)
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}


class ModelFolders:
    """Random-weight model folders, made on demand in a temporary root."""

    def __init__(self, root: str):
        self.root = root
        self._made: Dict[tuple, str] = {}

    def get(self, name: str, dtype: str = "float32", seed: int = 0, std: float = 0.02, overrides=None) -> str:
        import moe_b200

        key = (name, dtype, seed, std, repr(sorted((overrides or {}).items())))
        if key not in self._made:
            cfg = copy.deepcopy(CONFIGS[name])
            cfg.update(overrides or {})
            d = os.path.join(self.root, f"{name}_{dtype}_{seed}_{len(self._made)}")
            moe_b200.write_random_model(d, cfg, seed, std=std, dtype=dtype)
            self._made[key] = d
        return self._made[key]


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def plain_logits(model_dir: str, tokens: Sequence[int]) -> torch.Tensor:
    cfg, w = plain.read_model(model_dir)
    return plain.forward(cfg, w, list(tokens))


def routing_margin(model_dir: str, tokens: Sequence[int]) -> float:
    """Smallest relative gap between the last picked and the first unpicked expert's
    router probability over all tokens and routed layers (plain implementation)."""
    cfg, w = plain.read_model(model_dir)
    gaps = []
    orig = plain.route

    def spy(cfg_, w_, p, n, forced=None):
        sc = torch.softmax(n @ w_[p + "mlp.gate.weight"].T, dim=-1)
        k = cfg_["num_experts_per_tok"]
        s, _ = torch.sort(sc, dim=-1, descending=True)
        if sc.shape[1] > k:
            gaps.append(float(((s[:, k - 1] - s[:, k]) / s[:, k - 1]).min()))
        return orig(cfg_, w_, p, n, forced)

    plain.route = spy
    try:
        plain.forward(cfg, w, list(tokens))
    finally:
        plain.route = orig
    return min(gaps) if gaps else 1.0


# ----------------------------------------------------------------------------- replay cuts
def replay_whole(engine, requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    """Each request alone, whole, logits at every place."""
    out = {}
    for rid, toks in requests.items():
        s = engine.new_sequence()
        out[rid] = engine.step([s], [toks], [list(range(len(toks)))]).cpu()
        engine.release(s)
    return out


def replay_tail(engine, requests: Dict[str, List[int]], tail: int = 32) -> Dict[str, torch.Tensor]:
    """Each request alone: all but the last ``tail`` tokens in one step, then one by one."""
    out = {}
    for rid, toks in requests.items():
        s = engine.new_sequence()
        head = max(1, len(toks) - tail)
        rows = [engine.step([s], [toks[:head]], [list(range(head))]).cpu()]
        for t in toks[head:]:
            rows.append(engine.step([s], [[t]], [[0]]).cpu())
        engine.release(s)
        out[rid] = torch.cat(rows, dim=0)
    return out


def replay_batches(engine, requests: Dict[str, List[int]], batch_size: int) -> Dict[str, torch.Tensor]:
    """Batches of ``batch_size`` requests, one batch after another.  A batch starts with
    the first half of every request in one step, then decodes one token each; a request
    that has run out of tokens ends and leaves the batch."""
    ids = list(requests)
    out = {}
    for b0 in range(0, len(ids), batch_size):
        live = ids[b0:b0 + batch_size]
        slots = {r: engine.new_sequence() for r in live}
        done = {r: max(1, len(requests[r]) // 2) for r in live}
        rows = {r: [] for r in live}
        lg = engine.step([slots[r] for r in live], [requests[r][:done[r]] for r in live],
                         [list(range(done[r])) for r in live]).cpu()
        o = 0
        for r in live:
            rows[r].append(lg[o:o + done[r]])
            o += done[r]
        while True:
            for r in [r for r in live if done[r] >= len(requests[r])]:
                engine.release(slots.pop(r))
                live.remove(r)
            if not live:
                break
            lg = engine.step([slots[r] for r in live], [[requests[r][done[r]]] for r in live],
                             [[0] for _ in live]).cpu()
            for i, r in enumerate(live):
                rows[r].append(lg[i:i + 1])
                done[r] += 1
        for r in rows:
            out[r] = torch.cat(rows[r], dim=0)
    return out


def max_rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max |ref|."""
    return float((got.double() - ref.double()).abs().max() / ref.double().abs().max().clamp(min=1e-30))


# ----------------------------------------------------------------------------- routing-aware comparison
def routed_parts(model):
    """The routed feed-forwards in the order the schedule runs them."""
    return [model.blocks[e.layer].ffn for e in model.spec.schedule
            if model.blocks[e.layer].ffn.kind == "routed_experts"]


def whole_with_picks(engine, tokens: Sequence[int]):
    """One request alone and whole -> (logits [T, V] on the CPU, [layer][T][k] expert picks)."""
    parts = routed_parts(engine.model)      # a part appears once per run of its layer
    for p in parts:
        p.trace = []
    try:
        s = engine.new_sequence()
        lg = engine.step([s], [list(tokens)], [list(range(len(tokens)))]).cpu()
        engine.release(s)
        taken = {}
        picks = []
        for p in parts:
            i = taken.get(id(p), 0)
            picks.append(p.trace[i][0].cpu().tolist())
            taken[id(p)] = i + 1
    finally:
        for p in parts:
            p.trace = None
    return lg, picks


def compare_with_plain(model_dir: str, engine, tokens: Sequence[int], flip_margin: float):
    """Engine (whole request) against the plain implementation.

    Top-k routing is discontinuous: where two experts' probabilities are closer than the
    arithmetic's own noise, either pick is right.  So the plain implementation is run with the
    engine's picks, and every pick that differs from its own free choice must sit at a margin
    below ``flip_margin``.  Returns (max relative error of the logits, fraction of differing picks)."""
    cfg, w = plain.read_model(model_dir)
    got, picks = whole_with_picks(engine, tokens)
    free = []
    plain.forward(cfg, w, list(tokens), trace=free)
    ref = plain.forward(cfg, w, list(tokens), forced=picks)
    differing = total = 0
    k = cfg["num_experts_per_tok"]
    li = 0
    for l in range(cfg["num_hidden_layers"]):
        if not plain.layer_is_sparse(cfg, l):
            continue
        for i in range(len(tokens)):
            total += 1
            if sorted(picks[li][i]) != sorted(free[li][0][i]):
                differing += 1
        li += 1
    if differing:
        # legitimacy of the flips: recompute the margins where they happened
        margins = flip_margins(cfg, w, tokens, picks)
        assert max(margins) < flip_margin, f"a routing pick differs at margin {max(margins):.3g}"
    return max_rel_err(got, ref), differing / max(total, 1)


def flip_margins(cfg, w, tokens, picks) -> List[float]:
    """For every (layer, token) whose forced pick differs from the free one: the relative gap
    between the probabilities of the experts that were swapped."""
    out = []
    state = {"li": 0}
    orig = plain.route

    def spy(cfg_, w_, p, n, forced=None):
        sc = torch.softmax(n @ w_[p + "mlp.gate.weight"].T, dim=-1)
        k = cfg_["num_experts_per_tok"]
        for i in range(n.shape[0]):
            free = sorted(range(sc.shape[1]), key=lambda e: (-float(sc[i, e]), e))[:k]
            if forced is not None and sorted(free) != sorted(int(e) for e in forced[i]):
                lost = [e for e in free if e not in forced[i]]
                gained = [int(e) for e in forced[i] if e not in free]
                hi, lo = max(float(sc[i, e]) for e in lost), min(float(sc[i, e]) for e in gained)
                out.append((hi - lo) / hi)
        return orig(cfg_, w_, p, n, forced)

    plain.route = spy
    try:
        plain.forward(cfg, w, list(tokens), forced=picks)
    finally:
        plain.route = orig
    return out

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
# heads of 128 (the size the benchmark's shape has), 2 query heads on 1 kv head, a width that is not
# heads x head size, a window of 80 that crosses a page on the second layer, no q/k/v bias
CONFIG_D = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=2, hidden_size=264, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
    num_experts=6, num_experts_per_tok=2, moe_intermediate_size=56, shared_expert_intermediate_size=88,
    norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], intermediate_size=120,
    vocab_size=331, rope_theta=1e5, rms_norm_eps=1e-6, use_sliding_window=True, sliding_window=80,
    max_window_layers=1, tie_word_embeddings=False, max_position_embeddings=4096, eos_token_id=330,
    qkv_bias=False,
)
# sizes that the fast kernels refuse, so that the bfloat16 path takes its other kernels: a width that is
# no multiple of 8 (no TMA row), heads of 48 (no tensor-core attention, rows of 96 bytes in the cache),
# one expert a token, no shared expert, one layer, expert and dense sizes that are odd multiples of 4
CONFIG_E = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=2, hidden_size=100, num_attention_heads=3, num_key_value_heads=3, head_dim=48,
    num_experts=3, num_experts_per_tok=1, moe_intermediate_size=20, shared_expert_intermediate_size=0,
    norm_topk_prob=False, decoder_sparse_step=2, mlp_only_layers=[], intermediate_size=44,
    vocab_size=97, rope_theta=3e4, rms_norm_eps=1e-5, use_sliding_window=True, sliding_window=33,
    max_window_layers=0, tie_word_embeddings=True, max_position_embeddings=4096, eos_token_id=96,
)
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E}


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
    """For every (layer, token) whose forced pick differs from the free one: its margin (``pick_margins``)."""
    return plain_with_picks(cfg, w, tokens, picks)[1]


# ----------------------------------------------------------------------------- any schedule, against plain
def run_schedule(engine, steps):
    """Run ``steps`` -- each {"entries": [(request, tokens, wanted places)], "end": [requests]} --
    through ``engine.step`` with the routed parts recording their picks.

    Returns (logits, picks): logits[(request, position)] is a CPU row of logits for every wanted
    place; picks[i][(request, position)] the experts that the i-th routed layer of the schedule
    took for that token.  Positions count from the request's first token."""
    parts = routed_parts(engine.model)
    slots, done = {}, {}
    logits, picks = {}, [dict() for _ in parts]
    try:
        for st in steps:
            for p in parts:
                p.trace = []
            entries = st["entries"]
            for rid, _, _ in entries:
                if rid not in slots:
                    slots[rid], done[rid] = engine.new_sequence(), 0
            if entries:
                lg = engine.step([slots[r] for r, _, _ in entries], [t for _, t, _ in entries],
                                 [w for _, _, w in entries])
                lg = lg.float().cpu() if lg is not None else None
                taken, row, tok_row = {}, 0, 0
                recorded = []
                times = {id(p): sum(1 for x in parts if x is p) for p in parts}     # runs of a part in one pass
                for p in parts:
                    i = taken.get(id(p), 0)
                    # (a step that the engine runs in pieces leaves one record per piece and run: the
                    # pieces' tokens, one after another, are the step's tokens in their order; a step
                    # replayed from a padded graph also records its rows of no sequence, with picks of -1)
                    mine = p.trace[i::times[id(p)]]
                    recorded.append([pick for rec in mine for pick in rec[0].cpu().tolist() if pick[0] >= 0])
                    taken[id(p)] = i + 1
                for rid, toks, want in entries:
                    for w in want:
                        logits[(rid, done[rid] + w)] = lg[row]
                        row += 1
                    for j in range(len(toks)):
                        for li in range(len(parts)):
                            picks[li][(rid, done[rid] + j)] = recorded[li][tok_row + j]
                    tok_row += len(toks)
                    done[rid] += len(toks)
            for rid in st.get("end", []):
                engine.release(slots.pop(rid))
    finally:
        for p in parts:
            p.trace = None
        for s_ in slots.values():
            engine.release(s_)
    return logits, picks


def pick_margins(cfg, logits: torch.Tensor, forced) -> List[float]:
    """For every token whose forced pick differs from the free one (top k of ``logits`` [T, E], ties
    to the lower index): the gap between the router logits of the experts that were swapped, as a
    fraction of the root mean square of the layer's router logits.

    Why that measure: a router logit is a sum over the hidden state, so an error of relative size
    eps in the state moves each logit by about eps times the logits' own scale, whatever the width
    and the weights' scale are; which of two experts wins is decided by the difference of two
    logits.  (The gap between two logits is also the relative gap between their probabilities.)"""
    out = []
    if forced is None:
        return out
    k = cfg["num_experts_per_tok"]
    rms = float(logits.pow(2).mean().sqrt().clamp(min=1e-30))
    for i in range(logits.shape[0]):
        free = sorted(range(logits.shape[1]), key=lambda e: (-float(logits[i, e]), e))[:k]
        mine = [int(e) for e in forced[i]]
        if sorted(free) != sorted(mine):
            lost = [e for e in free if e not in mine]
            gained = [e for e in mine if e not in free]
            hi, lo = max(float(logits[i, e]) for e in lost), min(float(logits[i, e]) for e in gained)
            out.append((hi - lo) / rms)
    return out


def plain_with_picks(cfg, w, tokens, forced):
    """The plain implementation with the given picks -> (logits [T, V], the margins of the picks
    that differ from its own free choice, see ``pick_margins``)."""
    margins = []
    orig = plain.route

    def spy(cfg_, w_, p, n, forced_=None):
        margins.extend(pick_margins(cfg_, n @ w_[p + "mlp.gate.weight"].T, forced_))
        return orig(cfg_, w_, p, n, forced_)

    plain.route = spy
    try:
        ref = plain.forward(cfg, w, list(tokens), forced=forced)
    finally:
        plain.route = orig
    return ref, margins


def check_schedule_against_plain(model_dir, requests, logits, picks, tol, flip_margin, max_flips=0.05):
    """Every wanted place of every request against the plain implementation run with the engine's
    picks.  A pick may differ from the plain implementation's own only at a margin below
    ``flip_margin``; the logits may differ by ``tol`` of the request's largest logit."""
    cfg, w = plain.read_model(model_dir)
    flips = total = 0
    checked = 0
    for rid, toks in requests.items():
        forced = [[layer[(rid, i)] for i in range(len(toks))] for layer in picks]
        ref, margins = plain_with_picks(cfg, w, toks, forced)
        assert not margins or max(margins) < flip_margin, f"{rid}: a routing pick differs at margin {max(margins):.3g}"
        flips += len(margins)
        total += len(toks) * max(len(picks), 1)
        scale = float(ref.abs().max())
        for (r, pos), row in logits.items():
            if r != rid:
                continue
            err = float((row.double() - ref[pos]).abs().max()) / scale
            assert err < tol, f"{rid} at position {pos} of {len(toks)}: relative error {err:.3g}"
            checked += 1
    assert checked == len(logits) and checked > 0
    assert flips <= max_flips * total, f"routing differs too often: {flips} of {total}"


def batches_schedule(requests: Dict[str, List[int]], batch_size: int, prompt_len, want_all: bool = True):
    """Batches of ``batch_size`` requests one after another: the first ``prompt_len(request)`` tokens
    of each in one step, then one token each; a request that has run out of tokens ends."""
    ids = list(requests)
    steps = []
    for b0 in range(0, len(ids), batch_size):
        live = ids[b0:b0 + batch_size]
        done = {r: max(1, min(len(requests[r]), prompt_len(r))) for r in live}
        entries = [(r, requests[r][:done[r]], list(range(done[r])) if want_all else [done[r] - 1]) for r in live]
        while True:
            ends = [r for r in live if done[r] >= len(requests[r])]
            steps.append({"entries": entries, "end": ends})
            live = [r for r in live if r not in ends]
            if not live:
                break
            entries = [(r, [requests[r][done[r]]], [0]) for r in live]
            for r in live:
                done[r] += 1
    return steps


def whole_schedule(requests):
    """Each request alone and whole, logits at every place."""
    return [{"entries": [(r, list(t), list(range(len(t))))], "end": [r]} for r, t in requests.items()]


def tail_schedule(requests, tail: int = 32):
    """Each request alone: all but the last ``tail`` tokens in one step, then one by one."""
    steps = []
    for r, t in requests.items():
        head = max(1, len(t) - tail)
        steps.append({"entries": [(r, list(t[:head]), list(range(head)))], "end": [r] if head == len(t) else []})
        for i in range(head, len(t)):
            steps.append({"entries": [(r, [t[i]], [0])], "end": [r] if i == len(t) - 1 else []})
    return steps


def stacked(logits, rid, n):
    return torch.stack([logits[(rid, i)] for i in range(n)])

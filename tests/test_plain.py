"""The plain implementation itself (CPU): against the reference's oracle, and part by part."""
import json
import math
import os

import numpy as np
import torch

import helpers
import plain_qwen2moe as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qwen2moe_oracle")


def test_plain_matches_the_reference_oracle():
    """tests/golden/make_golden.py ran scripts/oracle.py of the reference on a tiny random model."""
    cfg, w = plain.read_model(GOLDEN)
    exp = json.load(open(os.path.join(GOLDEN, "expected.json")))
    got = plain.forward(cfg, w, exp["tokens"])
    ref = torch.tensor(exp["logits"], dtype=torch.float64)
    assert got.shape == ref.shape == (10, 48)
    # the oracle forms rotary angles in double, the reference engine and this file in float32
    assert float((got - ref).abs().max()) < 1e-5
    assert torch.equal(got.argmax(-1), ref.argmax(-1))
    assert plain.layer_windows(cfg) == [None, 3] and [plain.layer_is_sparse(cfg, l) for l in (0, 1)] == [False, True]


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    got = plain.rmsnorm(x, w, 1e-6)
    s = 1.0 / math.sqrt(12.5 + 1e-6)
    assert torch.allclose(got, torch.tensor([[3 * s * 2, 4 * s * 0.5]], dtype=torch.float64), atol=1e-15)


def test_rope_is_half_split_and_position_zero_is_identity():
    inv = plain.rope_inv_freq(10000.0, 8)
    assert torch.allclose(inv.double(), torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=torch.float64), rtol=1e-6)
    x = torch.arange(8, dtype=torch.float64).reshape(1, 1, 8) + 1
    assert torch.allclose(plain.rope(x, torch.tensor([0]), inv), x)
    y = plain.rope(x, torch.tensor([3]), inv)[0, 0]
    a, b, ang = 1.0, 5.0, 3.0 * 1.0                   # pair (0, 4)
    assert abs(float(y[0]) - (a * math.cos(ang) - b * math.sin(ang))) < 1e-6
    assert abs(float(y[4]) - (a * math.sin(ang) + b * math.cos(ang))) < 1e-6


def test_attention_window_includes_self_and_window_ge_context_is_no_window():
    torch.manual_seed(0)
    q, k, v = (torch.randn(9, 4, 16, dtype=torch.float64), torch.randn(9, 2, 16, dtype=torch.float64),
               torch.randn(9, 2, 16, dtype=torch.float64))
    full = plain.attention(q, k, v, None)
    assert torch.allclose(plain.attention(q, k, v, 9), full) and torch.allclose(plain.attention(q, k, v, 50), full)
    one = plain.attention(q, k, v, 1)                  # window 1: each position sees only itself
    assert torch.allclose(one.reshape(9, 4, 16)[:, 0], v[:, 0]) and torch.allclose(one.reshape(9, 4, 16)[:, 3], v[:, 1])
    w3 = plain.attention(q, k, v, 3)
    assert torch.allclose(w3[:3], full[:3]) and not torch.allclose(w3[3:], full[3:])


def test_router_picks_weights_and_ties():
    cfg = dict(num_experts_per_tok=2, norm_topk_prob=False)
    w = {"p.mlp.gate.weight": torch.tensor([[1.0], [3.0], [3.0], [0.0]], dtype=torch.float64)}
    picks, weights = plain.route(cfg, w, "p.", torch.ones(1, 1, dtype=torch.float64))
    sc = torch.softmax(torch.tensor([1.0, 3.0, 3.0, 0.0], dtype=torch.float64), 0)
    assert picks == [[1, 2]]                           # tie: lower index first
    assert torch.allclose(weights[0], sc[[1, 2]])
    cfg["norm_topk_prob"] = True
    cfg["routed_scaling_factor"] = 2.0
    _, weights = plain.route(cfg, w, "p.", torch.ones(1, 1, dtype=torch.float64))
    assert torch.allclose(weights[0], torch.tensor([1.0, 1.0], dtype=torch.float64))   # 0.5 each, times 2


def test_shared_expert_gate_and_bias_change_the_result(model_dirs):
    d = model_dirs.get("A", "float32", seed=5, std=0.2)
    cfg, w = plain.read_model(d)
    toks = helpers.random_tokens(256, 6, 1)
    base = plain.forward(cfg, w, toks)
    w2 = dict(w)
    w2["model.layers.0.mlp.shared_expert_gate.weight"] = w["model.layers.0.mlp.shared_expert_gate.weight"] + 5.0
    w3 = dict(w)
    w3["model.layers.1.self_attn.k_proj.bias"] = w["model.layers.1.self_attn.k_proj.bias"] + 1.0
    assert not torch.allclose(plain.forward(cfg, w2, toks), base)
    assert not torch.allclose(plain.forward(cfg, w3, toks), base)
    assert base.shape == (6, 256) and torch.isfinite(base).all()


def test_causality_a_prefix_has_the_same_logits(model_dirs):
    d = model_dirs.get("B", "float32", seed=2, std=0.2)
    cfg, w = plain.read_model(d)
    toks = helpers.random_tokens(384, 14, 3)
    whole = plain.forward(cfg, w, toks)
    assert torch.allclose(plain.forward(cfg, w, toks[:9]), whole[:9], atol=1e-12)


def test_xorshift_and_sampler_follow_the_reference():
    r = plain.Rng(0)
    assert r.s == 1                                     # 0 * k | 1
    vals = [plain.Rng(7).next_f32() for _ in range(1)]
    assert 0.0 <= vals[0] < 1.0
    # src/sample.rs:146-174
    assert plain.sample([0.1, 5.0, -2.0], [], plain.Rng(1)) == 1
    l = [1.0, 2.0, 3.0, 0.5]
    assert plain.sample(l, [], plain.Rng(7)) == plain.sample(l, [], plain.Rng(99)) == 2
    assert plain.sample([0.0, 0.2, 9.0], [], plain.Rng(3), temp=1.0, top_k=1) == 2
    assert plain.sample([3.0, 2.0], [0], plain.Rng(1), repeat_penalty=2.0) == 1
    # temperature sampling follows the distribution
    rng = plain.Rng(11)
    counts = np.zeros(4)
    for _ in range(4000):
        counts[plain.sample([1.0, 2.0, 0.5, -0.5], [], rng, temp=1.0, top_p=1.0)] += 1
    p = np.exp([1.0, 2.0, 0.5, -0.5])
    assert np.abs(counts / 4000 - p / p.sum()).max() < 0.03

"""Adding to the library from outside: a toy mixer with state of its own and a toy architecture,
both defined here, are registered, given random weights, loaded, and stepped through the
engine -- without a change to the library's files.  The toy model also names a layer twice in
its schedule and lets one layer read another layer's cache."""
import json

import pytest
import torch

import gpu_util as G
import helpers
import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu


def register_toy():
    import moe_b200
    from moe_b200.cache import StateRequest
    from moe_b200.config import Architecture, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from moe_b200.parts import Part, TensorSpec

    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + W_in n_t;  out_t = W_out s_t.  The carry s lives in the cache's
        per-sequence state of fixed size; tokens of a sequence are scanned in order."""
        category, kind = "mixer", "toy_decay"
        graph_safe = True

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden, self.decay = int(self.params["hidden_size"]), float(self.params["decay"])

        def tensors(self):
            return {"in_proj.weight": TensorSpec((self.hidden, self.hidden)),
                    "out_proj.weight": TensorSpec((self.hidden, self.hidden))}

        def kv_request(self):
            return None

        def state_request(self):
            return StateRequest((self.hidden,), torch.float32)

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.w_in, self.w_out = tensors["in_proj.weight"].float(), tensors["out_proj.weight"].float()

        def forward(self, rt, h, batch, cache_view, state):
            """The scan as device operations only (no value comes back to the host), so that a step
            may be captured: out_t = decay^(j+1) carry + sum_{i <= t, same sequence} decay^(t-i) u_i,
            j being the token's place among its sequence's tokens of this step."""
            assert cache_view is None and state is not None
            u = h.act.float() @ self.w_in.T
            T = u.shape[0]
            seq = batch.seq_of_token.long()                          # -1: a row of no sequence
            live = (seq >= 0).unsqueeze(1)
            sq = seq.clamp(min=0)
            rows = torch.arange(T, device=u.device)
            gap = rows.unsqueeze(1) - rows.unsqueeze(0)              # t - i
            same = (seq.unsqueeze(1) == seq.unsqueeze(0)) & (gap >= 0) & live
            weights = torch.where(same, torch.pow(torch.full_like(gap, self.decay, dtype=torch.float32),
                                                  gap.clamp(min=0).float()), torch.zeros((), device=u.device))
            place = rows - batch.cu_seqlens.long()[sq]               # j
            carry = state[batch.slots.long()[sq]]
            out = weights @ u + torch.pow(torch.full_like(place, self.decay, dtype=torch.float32),
                                          (place + 1).float()).unsqueeze(1) * carry
            out = torch.where(live, out, torch.zeros((), device=u.device))
            # the carry after the step is the output at each sequence's last token; a sequence without
            # tokens (padding of a captured step) sits in the padding slot, whose state nobody reads
            cu = batch.cu_seqlens.long()
            last = (cu[1:] - 1).clamp(min=0)
            has = (cu[1:] > cu[:-1]).unsqueeze(1)
            slot = batch.slots.long()
            state.index_copy_(0, slot, torch.where(has, out[last], state[slot]))
            return (out @ self.w_out.T).contiguous()

    moe_b200.register_part("mixer", "toy_decay", DecayMixer)

    def parse(cfg):
        return dict(cfg)

    def spec_of(c):
        H, V = c["hidden_size"], c["vocab_size"]
        norm = lambda p: PartSpec("rmsnorm", {"size": H, "eps": c["eps"]}, p)
        attn = lambda p, own: PartSpec("gqa_attention", {
            "hidden_size": H, "num_heads": c["heads"], "num_kv_heads": c["kv_heads"], "head_dim": c["head_dim"],
            "qkv_bias": False, "window": None, "own_kv": own,
            "position": {"kind": "rotary", "theta": c["theta"], "rotary_dim": c["head_dim"]}}, p)
        dense = lambda p: PartSpec("dense_swiglu", {"hidden_size": H, "size": c["ffn"]}, p)
        routed = lambda p: PartSpec("routed_experts", {"hidden_size": H, "num_experts": 4, "top_k": 2,
                                                       "expert_size": c["ffn"] // 2, "norm_topk_prob": True}, p)
        layers = (
            LayerSpec("prenorm", norm("l0.n1."), attn("l0.attn.", True), norm("l0.n2."), dense("l0.ffn.")),
            LayerSpec("prenorm", norm("l1.n1."), PartSpec("toy_decay", {"hidden_size": H, "decay": c["decay"]}, "l1.mix."),
                      norm("l1.n2."), routed("l1.ffn.")),
            LayerSpec("prenorm", norm("l2.n1."), attn("l2.attn.", False), norm("l2.n2."), dense("l2.ffn.")),
        )
        schedule = (ScheduleEntry(0, 0, True), ScheduleEntry(1, 1, True), ScheduleEntry(2, 0, False),
                    ScheduleEntry(1, 2, True))                     # layer 1 runs twice, with a state for each run
        return ModelSpec("ToyDecayForCausalLM", H, V, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "emb."),
                         layers, schedule, norm("final."),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True}, "head."))

    moe_b200.register_architecture(Architecture("ToyDecayForCausalLM", parse, spec_of, dict))


TOY = dict(architectures=["ToyDecayForCausalLM"], hidden_size=48, vocab_size=101, heads=3, kv_heads=1, head_dim=16,
           ffn=64, eps=1e-6, theta=1e4, decay=0.7)


def toy_plain(w, tokens, trace=None, forced=None):
    """The toy model, whole sequence, float64."""
    c = TOY
    cfg = dict(num_attention_heads=c["heads"], num_key_value_heads=c["kv_heads"], head_dim=c["head_dim"],
               rope_theta=c["theta"], num_experts_per_tok=2, norm_topk_prob=True)
    T = len(tokens)
    pos = torch.arange(T)
    inv = plain.rope_inv_freq(c["theta"], c["head_dim"])
    x = w["emb.weight"][torch.tensor(tokens)].clone()
    forced = list(forced) if forced is not None else None

    def ffn_routed(n):
        ww = {k.replace("l1.ffn.", "p.mlp."): v for k, v in w.items() if k.startswith("l1.ffn.")}
        return plain.moe_block(cfg, ww, "p.", n, trace, forced.pop(0) if forced is not None else None)

    def toy(n):
        u = n @ w["l1.mix.in_proj.weight"].T
        out, carry = torch.zeros_like(u), torch.zeros(c["hidden_size"], dtype=torch.float64)
        for t in range(T):
            carry = c["decay"] * carry + u[t]
            out[t] = carry
        return out @ w["l1.mix.out_proj.weight"].T

    # layer 0: attention that owns cache 0
    n = plain.rmsnorm(x, w["l0.n1.weight"], c["eps"])
    k0 = plain.rope((n @ w["l0.attn.k_proj.weight"].T).reshape(T, c["kv_heads"], c["head_dim"]), pos, inv)
    v0 = (n @ w["l0.attn.v_proj.weight"].T).reshape(T, c["kv_heads"], c["head_dim"])
    q0 = plain.rope((n @ w["l0.attn.q_proj.weight"].T).reshape(T, c["heads"], c["head_dim"]), pos, inv)
    x = x + plain.attention(q0, k0, v0, None) @ w["l0.attn.o_proj.weight"].T
    x = x + plain.swiglu_mlp({k.replace("l0.ffn.", "m."): v for k, v in w.items()}, "m.",
                             plain.rmsnorm(x, w["l0.n2.weight"], c["eps"]))
    # layer 1 (first run)
    x = x + toy(plain.rmsnorm(x, w["l1.n1.weight"], c["eps"]))
    x = x + ffn_routed(plain.rmsnorm(x, w["l1.n2.weight"], c["eps"]))
    # layer 2: queries of its own over layer 0's keys and values
    n = plain.rmsnorm(x, w["l2.n1.weight"], c["eps"])
    q2 = plain.rope((n @ w["l2.attn.q_proj.weight"].T).reshape(T, c["heads"], c["head_dim"]), pos, inv)
    x = x + plain.attention(q2, k0, v0, None) @ w["l2.attn.o_proj.weight"].T
    x = x + plain.swiglu_mlp({k.replace("l2.ffn.", "m."): v for k, v in w.items()}, "m.",
                             plain.rmsnorm(x, w["l2.n2.weight"], c["eps"]))
    # layer 1 again
    x = x + toy(plain.rmsnorm(x, w["l1.n1.weight"], c["eps"]))
    x = x + ffn_routed(plain.rmsnorm(x, w["l1.n2.weight"], c["eps"]))
    return plain.rmsnorm(x, w["final.weight"], c["eps"]) @ w["emb.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_stateful_mixer(tmp_path, dtype):
    import moe_b200
    from moe_b200.engine import Engine

    register_toy()
    d = str(tmp_path / "toy")
    moe_b200.write_random_model(d, TOY, seed=3, std=G.STD[dtype][1], dtype=dtype)
    assert json.load(open(d + "/config.json"))["architectures"] == ["ToyDecayForCausalLM"]
    model = moe_b200.load_model(d, dtype=dtype)
    eng = Engine(model, max_tokens=512, max_slots=3)
    assert len(eng.cache.groups) == 1 and len(eng.cache.groups[0].cache_ids) == 1     # only cache 0 holds keys
    assert eng.cache.state(1) is not None and eng.cache.state(2) is not None and eng.cache.state(0) is None

    _, w = plain.read_model(d)
    reqs = {f"r{i}": helpers.random_tokens(101, n, 50 + i) for i, n in enumerate([7, 30, 1, 12, 19])}
    whole = {}
    for rid, toks in reqs.items():
        got, picks = helpers.whole_with_picks(eng, toks)
        ref = toy_plain(w, toks, forced=picks)
        assert helpers.max_rel_err(got, ref) < G.tol(dtype), rid
        whole[rid] = got
    # cut differently, in batches on 3 slots: the state follows each sequence, and a slot that is
    # used again starts from a zero state
    tail = helpers.replay_tail(eng, reqs, 5)
    batched = helpers.replay_batches(eng, reqs, 3)
    for rid in reqs:
        assert helpers.max_rel_err(tail[rid], whole[rid]) < G.tol_cut(dtype)
        assert helpers.max_rel_err(batched[rid], whole[rid]) < G.tol_cut(dtype)
    assert eng.cache.ledger.slots.num_held == 0
    # the mixer is graph-safe, so single-token steps were replayed from captured graphs; the first use
    # of a graph ran the step once, not twice, or the carry would have decayed twice
    assert eng.use_graphs and eng.graphs_of("decode")
    out = moe_b200.generate(eng, [reqs["r0"], reqs["r3"]], max_tokens=4)
    assert [len(o.tokens) for o in out] == [4, 4]
    # state of fixed size cannot be rewound
    from moe_b200.cache import CacheError

    s = eng.new_sequence()
    eng.step([s], [reqs["r0"]])
    with pytest.raises(CacheError):
        eng.truncate(s, 3)
    eng.truncate(s, len(reqs["r0"]))               # to its own length: nothing to take back
    eng.release(s)


def register_toy_switch():
    """A second toy architecture: a position encoding of its own (acting on the 32-bit projections
    through ``apply``) and a feed-forward with routing of its own (each token goes to ONE of two
    small experts, picked by the larger of two router logits)."""
    import moe_b200
    from moe_b200.config import Architecture, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from moe_b200.parts import Part, TensorSpec

    class GrowingScale(Part):
        """q_p *= 1 / (1 + a p), k_j *= (1 + a j): a score then carries (1 + a j) / (1 + a p)."""
        category, kind = "position", "toy_growing_scale"

        def __init__(self, spec):
            super().__init__(spec)
            self.a = float(self.params["a"])

        def rotary_table(self):
            return None, 0

        def attention_scale(self):
            return 1.0

        def apply(self, rt, qkv32, nh, nkv, hd, positions):
            f = (1.0 + self.a * positions.to(torch.float32)).unsqueeze(1)
            qkv32[:, : nh * hd] /= f
            qkv32[:, nh * hd: (nh + nkv) * hd] *= f

    class SwitchFFN(Part):
        category, kind = "ffn", "toy_switch"
        wants32 = True

        def __init__(self, spec):
            super().__init__(spec)
            self.hidden, self.size = int(self.params["hidden_size"]), int(self.params["size"])
            self.trace = None

        def tensors(self):
            t = {"router.weight": TensorSpec((2, self.hidden))}
            for e in range(2):
                t[f"e{e}.up.weight"] = TensorSpec((self.size, self.hidden))
                t[f"e{e}.down.weight"] = TensorSpec((self.hidden, self.size))
            return t

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.w = {k: v.float() for k, v in tensors.items()}

        def forward(self, rt, h, batch):
            n = h.f32
            pick = (n @ self.w["router.weight"].T).argmax(dim=1)
            if self.trace is not None:
                self.trace.append(pick.clone())
            out = torch.zeros_like(n)
            for e in range(2):
                rows = (pick == e).nonzero().flatten()
                if rows.numel():
                    out[rows] = torch.relu(n[rows] @ self.w[f"e{e}.up.weight"].T) @ self.w[f"e{e}.down.weight"].T
            return out.contiguous()

    moe_b200.register_part("position", "toy_growing_scale", GrowingScale)
    moe_b200.register_part("ffn", "toy_switch", SwitchFFN)

    def spec_of(c):
        H, V = c["hidden_size"], c["vocab_size"]
        norm = lambda p: PartSpec("rmsnorm", {"size": H, "eps": c["eps"]}, p)
        attn = lambda p, position, window: PartSpec("gqa_attention", {
            "hidden_size": H, "num_heads": c["heads"], "num_kv_heads": c["kv_heads"], "head_dim": c["head_dim"],
            "qkv_bias": True, "window": window, "own_kv": True, "position": position}, p)
        layers = (
            LayerSpec("prenorm", norm("l0.n1."), attn("l0.attn.", {"kind": "toy_growing_scale", "a": c["a"]}, None),
                      norm("l0.n2."), PartSpec("toy_switch", {"hidden_size": H, "size": c["ffn"]}, "l0.ffn.")),
            LayerSpec("prenorm", norm("l1.n1."),
                      attn("l1.attn.", {"kind": "rotary", "theta": c["theta"], "rotary_dim": c["head_dim"] // 2}, c["window"]),
                      norm("l1.n2."), PartSpec("dense_swiglu", {"hidden_size": H, "size": c["ffn"]}, "l1.ffn.")),
        )
        return ModelSpec("ToySwitchForCausalLM", H, V, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, "emb."),
                         layers, (ScheduleEntry(0, 0, True), ScheduleEntry(1, 1, True)), norm("final."),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": False}, "head."))

    moe_b200.register_architecture(Architecture("ToySwitchForCausalLM", dict, spec_of, dict))


SWITCH = dict(architectures=["ToySwitchForCausalLM"], hidden_size=40, vocab_size=77, heads=4, kv_heads=2, head_dim=32,
              ffn=24, eps=1e-5, theta=5e3, a=0.05, window=6)


def switch_plain(w, tokens, picks):
    """The second toy model, whole sequence, float64, with the engine's expert picks."""
    c = SWITCH
    T, nh, nkv, hd = len(tokens), c["heads"], c["kv_heads"], c["head_dim"]
    pos = torch.arange(T)
    x = w["emb.weight"][torch.tensor(tokens)].clone()

    def qkv(p, n):
        return [(n @ w[p + f"{m}_proj.weight"].T + w[p + f"{m}_proj.bias"]).reshape(T, heads, hd)
                for m, heads in (("q", nh), ("k", nkv), ("v", nkv))]

    # layer 0: the toy position encoding, then the switch feed-forward
    q, k, v = qkv("l0.attn.", plain.rmsnorm(x, w["l0.n1.weight"], c["eps"]))
    f = (1.0 + c["a"] * pos.double()).reshape(T, 1, 1)
    x = x + plain.attention(q / f, k * f, v, None) @ w["l0.attn.o_proj.weight"].T
    n = plain.rmsnorm(x, w["l0.n2.weight"], c["eps"])
    out = torch.zeros_like(n)
    for t in range(T):
        e = int(picks[t])
        out[t] = torch.relu(n[t] @ w[f"l0.ffn.e{e}.up.weight"].T) @ w[f"l0.ffn.e{e}.down.weight"].T
    x = x + out
    # layer 1: rotary on half of each head, a window of 6, a dense feed-forward
    q, k, v = qkv("l1.attn.", plain.rmsnorm(x, w["l1.n1.weight"], c["eps"]))
    rot = hd // 2
    inv = plain.rope_inv_freq(c["theta"], rot)
    part = lambda z: torch.cat([plain.rope(z[..., :rot], pos, inv), z[..., rot:]], dim=-1)   # the rest passes through
    x = x + plain.attention(part(q), part(k), v, c["window"]) @ w["l1.attn.o_proj.weight"].T
    x = x + plain.swiglu_mlp({kk.replace("l1.ffn.", "m."): vv for kk, vv in w.items()}, "m.",
                             plain.rmsnorm(x, w["l1.n2.weight"], c["eps"]))
    return plain.rmsnorm(x, w["final.weight"], c["eps"]) @ w["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_its_own_position_encoding_and_routing(tmp_path, dtype):
    import moe_b200
    from moe_b200.engine import Engine

    register_toy_switch()
    d = str(tmp_path / "switch")
    moe_b200.write_random_model(d, SWITCH, seed=11, std=G.STD[dtype][1], dtype=dtype)
    model = moe_b200.load_model(d, dtype=dtype)
    eng = Engine(model, max_tokens=512, max_slots=2)
    assert len(eng.cache.groups) == 2                      # all keys for layer 0, a ring for layer 1's window
    ffn = model.blocks[0].ffn
    _, w = plain.read_model(d)
    reqs = {f"r{i}": helpers.random_tokens(77, n, 80 + i) for i, n in enumerate([9, 26, 2, 15])}
    whole = {}
    for rid, toks in reqs.items():
        ffn.trace = []
        s = eng.new_sequence()
        got = eng.step([s], [toks], [list(range(len(toks)))]).cpu()
        eng.release(s)
        picks, ffn.trace = ffn.trace[0].cpu().tolist(), None
        assert helpers.max_rel_err(got, switch_plain(w, toks, picks)) < G.tol(dtype), rid
        whole[rid] = got
    tail = helpers.replay_tail(eng, reqs, 4)
    batched = helpers.replay_batches(eng, reqs, 2)
    for rid in reqs:
        assert helpers.max_rel_err(tail[rid], whole[rid]) < G.tol_cut(dtype), rid
        assert helpers.max_rel_err(batched[rid], whole[rid]) < G.tol_cut(dtype), rid
    assert eng.cache.ledger.slots.num_held == 0


def test_unknown_part_kind_is_a_clear_error():
    from moe_b200.config.spec import PartSpec
    from moe_b200.parts import make_part

    with pytest.raises(KeyError) as e:
        make_part("mixer", PartSpec("no_such_mixer", {}))
    assert "gqa_attention" in str(e.value)

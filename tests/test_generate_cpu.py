"""The generation loop's decisions, driven by a fake stepper (CPU).

Mirrors the reference's tests/speculative.rs: N tokens cost N - 1 decode steps
(:66-69), the token budget is exact (:136-144), a callback halts (:149-166), and
what was fed equals the committed history (:101-131)."""
from typing import Dict, List

import pytest

from moe_b200.engine.generate import CALLER, CONTEXT, EOS, LENGTH, GenerationStats, generate
from moe_b200.sampling.params import SamplingParams

V = 97


def next_token(history: List[int]) -> int:
    return (sum(history) * 31 + 7 * len(history)) % V


class FakeStepper:
    """Next token is a function of everything fed so far, so any slip in what the loop
    feeds (a token twice, a token of another request, a missing one) changes the output."""

    def __init__(self, num_slots=4):
        self.free = list(range(num_slots))[::-1]
        self.fed: Dict[int, List[int]] = {}
        self.seeds: Dict[int, int] = {}
        self.calls = []                    # (kind, number of sequences)
        self.max_live = 0
        self.released = []

    def new_sequence(self):
        s = self.free.pop()
        assert s not in self.fed, "slot handed out twice"
        self.fed[s] = []
        self.max_live = max(self.max_live, len(self.fed))
        return s

    def release(self, slot):
        assert slot in self.fed, "slot released twice"
        del self.fed[slot]
        self.free.append(slot)
        self.released.append(slot)

    def seed(self, slots, seeds):
        for s, v in zip(slots, seeds):
            self.seeds[s] = v

    def step_and_sample(self, slots, tokens, histories, params):
        assert len(set(slots)) == len(slots)
        kinds = {len(t) == 1 and len(self.fed[s]) > 0 for s, t in zip(slots, tokens)}
        assert len(kinds) == 1, "a step mixes prompts and single tokens"
        self.calls.append(("decode" if kinds.pop() else "prefill", len(slots)))
        out = []
        for s, t, h in zip(slots, tokens, histories):
            self.fed[s].extend(t)
            assert list(h) == self.fed[s], "history differs from what the cache holds"
            out.append(next_token(self.fed[s]))
        return out


def expected(prompt, n, eos=()):
    h, out = list(prompt), []
    while len(out) < n:
        t = next_token(h)
        if t in eos:
            return out, EOS
        h.append(t)
        out.append(t)
    return out, LENGTH


PROMPTS = [[5, 9, 2], [1], [4, 4, 4, 4, 4, 4, 4], [8, 3], [2, 7, 1, 8, 2, 8]]


@pytest.mark.parametrize("n", [1, 2, 3, 5, 11])
def test_token_budget_is_exact_and_n_tokens_cost_n_minus_1_steps(n):
    st = FakeStepper()
    stats = GenerationStats()
    res = generate(st, PROMPTS[:3], max_tokens=n, stats=stats)
    for p, r in zip(PROMPTS, res):
        assert r.tokens == expected(p, n)[0] and r.stop == LENGTH and r.steps == n - 1
    assert stats.decode_steps == n - 1 and st.calls[0] == ("prefill", 3)
    assert not st.fed and sorted(st.released) == [0, 1, 2]


def test_zero_budget_runs_nothing():
    st = FakeStepper()
    res = generate(st, PROMPTS[:2], max_tokens=0)
    assert [r.tokens for r in res] == [[], []] and st.calls == []


def test_eos_is_neither_emitted_nor_counted_and_the_batch_shrinks():
    # choose as eos the 3rd token request 0 would generate
    full, _ = expected(PROMPTS[0], 8)
    eos = {full[2]}
    st = FakeStepper()
    res = generate(st, PROMPTS[:3], max_tokens=8, eos=eos)
    for p, r in zip(PROMPTS, res):
        toks, why = expected(p, 8, eos)
        assert r.tokens == toks and r.stop == why
    assert res[0].stop == EOS and len(res[0].tokens) == 2 and eos.isdisjoint(res[0].tokens)
    sizes = [n for kind, n in st.calls if kind == "decode"]
    assert sizes[0] == 3 and sizes[-1] < 3 and sizes == sorted(sizes, reverse=True)   # shorter requests end earlier
    assert res[0].finish_reason == "stop" and res[1].finish_reason in ("length", "stop")


def test_eos_as_first_token_emits_nothing():
    first = next_token(PROMPTS[1])
    res = generate(FakeStepper(), [PROMPTS[1]], max_tokens=5, eos=[first])
    assert res[0].tokens == [] and res[0].stop == EOS and res[0].steps == 0


def test_callback_halts_only_its_own_request():
    seen = []

    def cb(i, tok):
        seen.append((i, tok))
        return not (i == 1 and len([1 for j, _ in seen if j == 1]) == 3)

    res = generate(FakeStepper(), PROMPTS[:3], max_tokens=6, on_token=cb)
    assert res[1].stop == CALLER and len(res[1].tokens) == 3
    assert res[0].stop == LENGTH and len(res[0].tokens) == 6 and len(res[2].tokens) == 6
    for i in range(3):
        assert [t for j, t in seen if j == i] == res[i].tokens      # every emitted token was shown, in order


def test_context_limit_stops_before_the_cache_overflows():
    p = PROMPTS[2]                                   # 7 tokens
    res = generate(FakeStepper(), [p], max_tokens=50, ctx=10)
    # the cache holds ctx positions at most: 7 prompt + 3 fed tokens; the token sampled then is not emitted
    assert res[0].stop == CONTEXT and len(res[0].tokens) == 3 and res[0].finish_reason == "length"
    res = generate(FakeStepper(), [p], max_tokens=50, ctx=7)
    assert res[0].stop == CONTEXT and res[0].tokens == []


def test_batches_follow_one_another_and_slots_are_reused():
    st = FakeStepper(num_slots=2)
    res = generate(st, PROMPTS, max_tokens=4, batch_size=2)
    for p, r in zip(PROMPTS, res):
        assert r.tokens == expected(p, 4)[0] and r.prompt_tokens == len(p)
    assert st.max_live == 2 and len(st.released) == 5 and not st.fed
    assert [c for c in st.calls if c[0] == "prefill"] == [("prefill", 2), ("prefill", 2), ("prefill", 1)]


def test_each_request_gets_its_own_seed():
    st = FakeStepper()
    seen = {}
    orig = st.seed
    st.seed = lambda slots, seeds: (seen.update(zip(slots, seeds)), orig(slots, seeds))
    generate(st, PROMPTS[:3], max_tokens=1, sampling=SamplingParams(temp=0.8, seed=40))
    assert sorted(seen.values()) == [40, 41, 42]


def test_slots_are_returned_when_a_step_raises():
    st = FakeStepper()

    def boom(*a, **k):
        raise RuntimeError("device fault")

    st.step_and_sample = boom
    with pytest.raises(RuntimeError):
        generate(st, PROMPTS[:2], max_tokens=3)
    assert not st.fed and len(st.free) == 4


def test_empty_prompt_is_refused():
    with pytest.raises(ValueError):
        generate(FakeStepper(), [[1], []], max_tokens=2)

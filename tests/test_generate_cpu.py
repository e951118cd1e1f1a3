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


# ---- one step ahead ---------------------------------------------------------------------------------
class AheadStepper(FakeStepper):
    """A stepper with ``begin``/``finish``: the loop may begin a step before it has finished the one
    before and feed LAST_TOKEN, which is replaced here, as on the device, by the token sampled last
    for that slot.  ``room`` bounds the tokens held, to make a step begun ahead fail for lack of room."""

    def __init__(self, num_slots=4, room=None):
        super().__init__(num_slots)
        self.last: Dict[int, int] = {}
        self.room = room
        self.open = 0                      # steps begun and not finished
        self.most_open = 0
        self.refused = 0

    def begin(self, slots, tokens, histories, params, from_last=False):
        from moe_b200.cache.allocator import CacheError
        from moe_b200.engine.generate import LAST_TOKEN

        if self.room is not None and sum(len(v) for v in self.fed.values()) + sum(len(t) for t in tokens) > self.room:
            self.refused += 1
            raise CacheError("the cache is full")
        real = []
        for s, t in zip(slots, tokens):
            if list(t) == [LAST_TOKEN]:
                assert from_last, "LAST_TOKEN fed without from_last"
                real.append([self.last[s]])
            else:
                assert all(x >= 0 for x in t)
                real.append(list(t))
        # the host's history lags by the token still in flight: compare what it does know
        for s, t, h in zip(slots, real, histories):
            known = self.fed[s] + t
            assert list(h) == known[:len(h)] and len(known) - len(h) in (0, 1)
        out = FakeStepper.step_and_sample(self, slots, real, [self.fed[s] + t for s, t in zip(slots, real)], params)
        for s, tok in zip(slots, out):
            self.last[s] = tok
        self.open += 1
        self.most_open = max(self.most_open, self.open)
        return out

    def finish(self, handle):
        self.open -= 1
        return handle

    def step_and_sample(self, slots, tokens, histories, params):
        return self.finish(self.begin(slots, tokens, histories, params))


def same(a, b):
    assert [(r.tokens, r.stop, r.steps, r.prompt_tokens) for r in a] == [(r.tokens, r.stop, r.steps, r.prompt_tokens)
                                                                         for r in b]


@pytest.mark.parametrize("n", [1, 2, 3, 9])
def test_one_step_ahead_gives_the_same_results(n):
    full, _ = expected(PROMPTS[0], 8)
    for kw in (dict(), dict(eos={full[2]}), dict(ctx=9), dict(batch_size=2), dict(eos={next_token(PROMPTS[1])})):
        a, b = AheadStepper(), FakeStepper()
        sa, sb = GenerationStats(), GenerationStats()
        same(generate(a, PROMPTS[:4], max_tokens=n, stats=sa, **kw), generate(b, PROMPTS[:4], max_tokens=n, stats=sb, **kw))
        assert sa.decode_tokens == sb.decode_tokens and sa.prefill_tokens == sb.prefill_tokens
        assert not a.fed and a.open == 0 and (a.most_open == 2 or n == 1)
        same(generate(AheadStepper(), PROMPTS[:4], max_tokens=n, lookahead=False, **kw),
             generate(FakeStepper(), PROMPTS[:4], max_tokens=n, **kw))


def test_one_step_ahead_with_a_callback_that_halts():
    def make():
        seen = []

        def cb(i, tok):
            seen.append(i)
            return not (i == 1 and seen.count(1) == 3)
        return cb

    same(generate(AheadStepper(), PROMPTS[:3], max_tokens=6, on_token=make()),
         generate(FakeStepper(), PROMPTS[:3], max_tokens=6, on_token=make()))


def test_a_step_begun_ahead_that_finds_no_room_is_begun_again_when_the_tokens_are_known():
    # room for the prompts and 3 more tokens each: the last step ahead is refused, then fits
    # because request 0 has stopped by then
    full, _ = expected(PROMPTS[0], 8)
    st = AheadStepper(room=sum(len(p) for p in PROMPTS[:2]) + 5)
    res = generate(st, PROMPTS[:2], max_tokens=5, eos={full[2]})
    same(res, generate(FakeStepper(), PROMPTS[:2], max_tokens=5, eos={full[2]}))
    assert st.refused >= 1 and not st.fed


def test_repeat_penalty_turns_looking_ahead_off():
    st = AheadStepper()
    generate(st, PROMPTS[:2], max_tokens=4, sampling=SamplingParams(temp=0.7, repeat_penalty=1.3))
    assert st.most_open == 1
    with pytest.raises(ValueError):
        generate(AheadStepper(), PROMPTS[:2], max_tokens=4, sampling=SamplingParams(repeat_penalty=1.3), lookahead=True)


# ---- what the model thought of each token ---------------------------------------------------------
class ProbingStepper(AheadStepper):
    """Brings, like the engine's handle, a probe per row: here (minus the token, [(token, -1.0)])."""

    class Handle(list):
        probes = None

    def begin(self, slots, tokens, histories, params, from_last=False, logprobs=None):
        out = self.Handle(AheadStepper.begin(self, slots, tokens, histories, params, from_last))
        self.asked = logprobs
        if logprobs is not None:
            out.probes = [(-float(t), [(t, -1.0)] * logprobs) for t in out]
        return out


@pytest.mark.parametrize("lookahead", [False, True])
def test_logprobs_follow_the_emitted_tokens(lookahead):
    full, _ = expected(PROMPTS[0], 8)
    st = ProbingStepper()
    outs = generate(st, PROMPTS[:3], max_tokens=6, eos={full[3]}, logprobs=2, lookahead=lookahead)
    assert st.asked == 2
    for o in outs:
        # one entry per EMITTED token (the end-of-sequence token is not one), in order
        assert [lp for lp, _ in o.logprobs] == [-float(t) for t in o.tokens]
        assert all(top == [(t, -1.0)] * 2 for t, (_, top) in zip(o.tokens, o.logprobs))
    assert outs[0].stop == "eos" and len(outs[0].tokens) == 3
    plain_outs = generate(AheadStepper(), PROMPTS[:3], max_tokens=6, eos={full[3]})
    same(outs, plain_outs)
    assert all(o.logprobs is None for o in plain_outs)
    with pytest.raises(ValueError):
        generate(FakeStepper(), PROMPTS[:1], max_tokens=2, logprobs=1)       # no begin / finish
    with pytest.raises(ValueError):
        generate(ProbingStepper(), PROMPTS[:1], max_tokens=2, logprobs=65)

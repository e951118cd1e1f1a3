"""The device sampler against the plain sampler written from src/sample.rs."""
import numpy as np
import pytest
import torch

import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def sampler():
    from moe_b200.sampling.sampler import DeviceSampler

    return DeviceSampler(torch.zeros(16, dtype=torch.int64, device=DEV), DEV)


def P(**kw):
    from moe_b200.sampling.params import SamplingParams

    return SamplingParams(**kw)


def test_greedy_is_the_first_maximum(sampler):
    logits = torch.randn(5, 1003, device=DEV)
    logits[2, 17] = logits[2, 900] = 50.0           # a tie: the first wins
    logits[3] = -1.0                                # all equal: index 0
    slots = torch.arange(5, dtype=torch.int32, device=DEV)
    got = sampler.sample(logits.clone(), slots, P()).cpu().tolist()
    want = [plain.sample(logits[i].cpu().numpy(), [], plain.Rng(0)) for i in range(5)]
    assert got == want and got[2] == 17 and got[3] == 0


def test_greedy_over_many_chunks_ties_nan_and_the_last_token_table(sampler):
    """A large row is cut into chunks: a tie across chunks goes to the lowest index; NaN counts as
    -inf; a row of -inf gives 0; the per-slot table of last tokens receives every pick."""
    from moe_b200.ops import core

    V = 151936 + 7
    torch.manual_seed(3)
    logits = torch.randn(6, V, device=DEV)
    logits[0, 150000] = logits[0, 2049] = logits[0, 77777] = 9.0
    logits[1, V - 1] = 9.0
    logits[2, 5] = float("nan")
    logits[2, 100000] = 8.0
    logits[3] = float("-inf")
    logits[4, 0] = 9.0
    logits[5] = -0.0
    logits[5, 4097] = 0.0                           # -0 and +0 are equal: index 0
    slots = torch.tensor([4, 0, 9, 2, 7, 1], dtype=torch.int32, device=DEV)
    out = torch.full((6,), -5, dtype=torch.int32, device=DEV)
    last = torch.full((12,), -7, dtype=torch.int32, device=DEV)
    for kernel in (None, "global"):
        out.fill_(-5), last.fill_(-7)
        core.sample(logits, slots, sampler.rng_states, out, last_token=last, kernel=kernel)
        assert out.cpu().tolist() == [2049, V - 1, 100000, 0, 0, 0], kernel
        want = [-7] * 12
        for s, t in zip(slots.tolist(), out.cpu().tolist()):
            want[s] = t
        assert last.cpu().tolist() == want
    # again: the workspace was left as it was found
    core.sample(logits, slots, sampler.rng_states, out)
    assert out.cpu().tolist() == [2049, V - 1, 100000, 0, 0, 0]


def test_sampling_writes_the_last_token_table_and_ignores_nan(sampler):
    from moe_b200.ops import core

    for V in (300, 20000, 151936):
        logits = torch.full((3, V), -30.0, device=DEV)
        logits[0, V - 3] = 5.0                       # one candidate carries all the weight
        logits[1, 7] = 5.0
        logits[1, 8] = float("nan")
        logits[2, V // 2] = 5.0
        slots = torch.tensor([2, 5, 3], dtype=torch.int32, device=DEV)
        out = torch.zeros(3, dtype=torch.int32, device=DEV)
        last = torch.full((8,), -7, dtype=torch.int32, device=DEV)
        sampler.seed([2, 5, 3], [1, 2, 3])
        core.sample(logits, slots, sampler.rng_states, out, temp=0.7, top_p=0.9, last_token=last)
        assert out.cpu().tolist() == [V - 3, 7, V // 2]
        assert last.cpu().tolist() == [-7, -7, V - 3, V // 2, -7, 7, -7, -7]


@pytest.mark.parametrize("vocab", [50, 1003, 5000, 20000, 70001, 151936, 210007])
@pytest.mark.parametrize("kw", [dict(temp=0.8, top_p=1.0), dict(temp=0.8), dict(temp=1.3, top_k=20, top_p=1.0),
                                dict(temp=0.5, top_k=40, top_p=0.9), dict(temp=1.0, top_k=1)])
def test_seeded_sampling_follows_the_plain_sampler(sampler, vocab, kw):
    """Same seed, same logits: the same tokens, draw after draw (the generator state advances only
    when there is more than one candidate).  The reference adds 32-bit probabilities one after the
    other, the kernel block-wise, so a draw that lands within that rounding of a boundary of the
    cumulative distribution may fall to the other side: a token that differs from the plain
    sampler's must have the drawn number within rounding of its own stretch of the exact
    cumulative distribution."""
    rows, draws = 4, 12
    torch.manual_seed(vocab)
    logits = (torch.randn(rows, vocab, device=DEV) * 2.5).contiguous()
    slots = torch.tensor([3, 9, 0, 5], dtype=torch.int32, device=DEV)
    sampler.seed(slots.tolist(), [11, 12, 13, 14])
    rngs = [plain.Rng(s) for s in (11, 12, 13, 14)]
    host = logits.cpu().numpy()
    # the rounding of the plain sampler's sequential 32-bit sum over the vocabulary (its normaliser):
    # each addition errs by up to 2^-24 of the sum so far
    tol = 1e-5 if vocab <= 1003 else min(1e-3, vocab * 2.0 ** -24)
    exact = total = 0
    for _ in range(draws):
        got = sampler.sample(logits.clone(), slots, P(**kw)).cpu().tolist()
        for i in range(rows):
            before = rngs[i].s
            want = plain.sample(host[i], [], rngs[i], **kw)
            total += 1
            if got[i] == want:
                exact += 1
                continue
            assert rngs[i].s != before, "one candidate only, and another token"
            peek = plain.Rng(0)
            peek.s = before
            r = peek.next_f32()
            # the exact distribution over the candidates, in 64-bit
            order = np.lexsort((np.arange(vocab), -host[i]))
            if kw.get("top_k", 0):
                order = order[:kw["top_k"]]
            p64 = np.exp((host[i][order].astype(np.float64) - float(host[i].max())) / kw["temp"])
            p64 /= p64.sum()
            top_p = kw.get("top_p", 0.95)
            if 0.0 < top_p < 1.0:
                cut = int(np.searchsorted(np.cumsum(p64), top_p)) + 1
                order, p64 = order[:cut], p64[:cut] / p64[:cut].sum()
            cdf = np.concatenate([[0.0], np.cumsum(p64)])
            at = np.where(order == got[i])[0]
            assert len(at) == 1, f"row {i}: {got[i]} is no candidate"
            j = int(at[0])
            assert cdf[j] - tol <= r <= cdf[j + 1] + tol, \
                f"row {i}: got {got[i]} (rank {j}, [{cdf[j]}, {cdf[j + 1]}]), drawn {r}, plain {want}"
    # where a token's probability is far above that rounding, the same tokens
    assert exact >= total - (2 if vocab <= 1003 else total // 2)
    # the generator states agree at the end: as many numbers were drawn on both sides
    states = sampler.rng_states.cpu().numpy().view(np.uint64)
    assert [int(states[s]) for s in slots.tolist()] == [r.s for r in rngs]


def test_repeat_penalty_once_per_occurrence(sampler):
    logits = torch.tensor([[3.0, 2.9, -1.0, 2.0], [0.5, -0.2, 0.4, 0.3]], device=DEV)
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    hist = [[0, 0, 2], [1, 3]]
    lg = logits.clone()
    got = sampler.sample(lg, slots, P(repeat_penalty=2.0), histories=hist).cpu().tolist()
    want = [plain.sample(logits[i].cpu().numpy(), hist[i], plain.Rng(0), repeat_penalty=2.0) for i in range(2)]
    assert got == want == [1, 0]
    assert torch.allclose(lg[0].cpu(), torch.tensor([0.75, 2.9, -2.0, 2.0]))   # 3 / 2 / 2, and -1 * 2


def test_temperature_sampling_follows_the_distribution(sampler):
    logits = torch.tensor([[1.0, 2.0, 0.5, -0.5]], device=DEV).repeat(2000, 1).contiguous()
    rng = torch.zeros(2001, dtype=torch.int64, device=DEV)
    from moe_b200.sampling.sampler import DeviceSampler

    s = DeviceSampler(rng, DEV)
    slots = torch.arange(2000, dtype=torch.int32, device=DEV)
    s.seed(slots.tolist(), list(range(100, 2100)))
    got = s.sample(logits, slots, P(temp=1.0, top_p=1.0)).cpu().numpy()
    p = np.exp([1.0, 2.0, 0.5, -0.5])
    assert np.abs(np.bincount(got, minlength=4) / 2000 - p / p.sum()).max() < 0.04


@pytest.mark.parametrize("vocab,top", [(97, 0), (97, 5), (300, 64), (151936, 20), (5, 8)])
def test_logprobs_and_alternatives_from_raw_logits(vocab, top):
    """src/generate.rs:91-105: logprob = logit - logsumexp; the strongest alternatives first, of equal
    logits the lower id first; fewer candidates than asked for leave -1."""
    from moe_b200.ops import core

    torch.manual_seed(vocab + top)
    rows = 3
    logits = (torch.randn(rows, vocab, device=DEV) * 3).contiguous()
    logits[0, 1] = logits[0, 3] = logits[0].max() + 1.0          # a tie at the top: the lower id first
    if vocab > 50:
        logits[1, 7] = float("nan")                              # no candidate
        logits[2, 11] = float("-inf")
    toks = torch.tensor([3, 0, vocab - 1], dtype=torch.int32, device=DEV)
    lp, ids, lps = core.logprobs(logits, toks, top)
    torch.cuda.synchronize()
    clean = torch.nan_to_num(logits.double().cpu(), nan=-1e300)
    ref = torch.log_softmax(clean, -1)
    for r in range(rows):
        assert abs(float(lp[r]) - float(ref[r, int(toks[r])])) < 1e-4
        n = min(top, vocab - (1 if r == 1 and vocab > 50 else 0))
        order = sorted(range(vocab), key=lambda i: (-float(clean[r, i]), i))
        order = [i for i in order if not (r == 1 and vocab > 50 and i == 7)][:n]
        assert ids[r, :n].tolist() == order, (r, ids[r].tolist()[:8], order[:8])
        assert ids[r, n:].tolist() == [-1] * (top - n)
        got = lps[r, :n].double().cpu()
        want = ref[r, order]
        fin = torch.isfinite(want)
        assert torch.equal(torch.isfinite(got), fin) and float((got[fin] - want[fin]).abs().max() if fin.any() else 0) < 1e-4
    if top >= 2:
        assert ids[0, :2].tolist() == [1, 3]

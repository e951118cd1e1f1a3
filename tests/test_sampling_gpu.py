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


@pytest.mark.parametrize("vocab", [50, 1003, 151936])
@pytest.mark.parametrize("kw", [dict(temp=0.8, top_p=1.0), dict(temp=0.8), dict(temp=1.3, top_k=20, top_p=1.0),
                                dict(temp=0.5, top_k=40, top_p=0.9), dict(temp=1.0, top_k=1)])
def test_seeded_sampling_follows_the_plain_sampler(sampler, vocab, kw):
    """Same seed, same logits: the same tokens, draw after draw (the generator state advances only
    when there is more than one candidate).  A draw that lands within rounding of a boundary of
    the cumulative distribution may differ -- the reference sums 32-bit probabilities one after the
    other, the kernel sums them block-wise -- and must then sit at the same place of the cumulative
    distribution to 1e-4."""
    rows, draws = 4, 12
    torch.manual_seed(vocab)
    logits = (torch.randn(rows, vocab, device=DEV) * 2.5).contiguous()
    slots = torch.tensor([3, 9, 0, 5], dtype=torch.int32, device=DEV)
    sampler.seed(slots.tolist(), [11, 12, 13, 14])
    rngs = [plain.Rng(s) for s in (11, 12, 13, 14)]
    host = logits.cpu().numpy()
    exact = total = 0
    for _ in range(draws):
        got = sampler.sample(logits.clone(), slots, P(**kw)).cpu().tolist()
        for i in range(rows):
            want = plain.sample(host[i], [], rngs[i], **kw)
            total += 1
            if got[i] == want:
                exact += 1
            else:
                order = np.argsort(-host[i], kind="stable")
                ra, rb = int(np.where(order == got[i])[0][0]), int(np.where(order == want)[0][0])
                # the reference adds 32-bit probabilities one after the other, the kernel block-wise:
                # deep in the tail of a large vocabulary the two sums part by rounding, and the picks
                # then sit at the same place of the exact cumulative distribution (a sequential 32-bit
                # sum of 150k terms is itself only good to a few 1e-4)
                p64 = np.exp((host[i][order].astype(np.float64) - float(host[i].max())) / kw["temp"])
                cdf = np.cumsum(p64) / p64.sum()
                assert abs(cdf[ra] - cdf[rb]) < (1e-5 if vocab < 100000 else 1e-3), f"row {i}: got {got[i]} (rank {ra}), plain {want} (rank {rb})"
    assert exact >= total - (2 if vocab < 100000 else total // 2)
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

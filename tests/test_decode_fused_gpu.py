"""The fused kernels of a decode step against the separate kernels they replace."""
import pytest
import torch

import gpu_util as G
import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def core():
    from moe_b200.ops import core as c

    c.lib()
    return c


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot,window", [(4, 2, 16, 16, None), (3, 1, 32, 32, 8), (2, 2, 128, 64, None)])
def test_rope_commit_equals_rope_split_then_kv_commit(core, dt, nh, nkv, hd, rot, window):
    from moe_b200.cache import KVCache, KVRequest

    lens = [0, 63, 64, 200]                                   # the new token's position in each sequence
    B = len(lens)
    torch.manual_seed(hd)
    qkv = torch.randn(B + 1, (nh + 2 * nkv) * hd, device=DEV)     # one padding row at the end
    inv = plain.rope_inv_freq(1e4, rot).to(DEV)
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    results = []
    for fused in (False, True):
        cache = KVCache({0: KVRequest(nkv, hd, window)}, {0: None}, 2048, B, dt, DEV)
        view = cache.view(0)
        slots = [cache.acquire() for _ in range(B)]
        for s, n in zip(slots, lens):
            G.give_pages(cache, s, n + 1)
        batch = G.make_batch(DEV, slots + [cache.padding_slot], lens + [0], [1] * (B + 1))
        batch.seq_of_token[B] = -1
        q = torch.zeros(B + 1, nh, hd, device=DEV, dtype=dt)
        if fused:
            core.rope_commit(qkv, batch.pos, inv, nh, nkv, hd, rot, q, view, batch, st)
        else:
            k = torch.empty(B + 1, nkv, hd, device=DEV, dtype=dt)
            v = torch.empty(B + 1, nkv, hd, device=DEV, dtype=dt)
            core.rope_split(qkv, batch.pos, inv, nh, nkv, hd, rot, q, k, v)
            core.kv_commit(k, v, view, batch, st)
        results.append((q.clone(), view.group.storage.clone()))
    assert int(st[0]) == 0
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    assert float(results[1][1][:, :, 0].abs().sum()) == 0.0     # the scratch page was not written


@pytest.mark.parametrize("E,k,H,norm,T", [(60, 4, 2048, False, 8), (8, 3, 96, True, 1), (4, 2, 64, False, 64),
                                           (200, 8, 72, True, 13)])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
def test_route_dispatch_equals_router_align_gather(core, E, k, H, norm, T, wdt):
    torch.manual_seed(E + T)
    h = torch.randn(T, H, device=DEV)
    wr = torch.randn(E, H, device=DEV).to(wdt)
    wsg = torch.randn(H, device=DEV).to(wdt)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    if T > 4:
        seq[T - 2] = -1                                           # a padding row
    act = h.to(torch.bfloat16)
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    idx, w, sg, offs, sorted_token, pos, xs = core.route_dispatch(h, wr, k, norm, 1.5, shared_gate_w=wsg,
                                                                 seq_of_token=seq, gather=act, status=st)
    idx2 = torch.empty(T, k, dtype=torch.int32, device=DEV)
    w2 = torch.empty(T, k, device=DEV)
    sg2 = torch.empty(T, device=DEV)
    core.router(h, wr, k, norm, 1.5, idx2, w2, shared_gate_w=wsg, shared_gate=sg2, seq_of_token=seq)
    offs2 = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    st2 = torch.empty(T * k, dtype=torch.int32, device=DEV)
    pos2 = torch.empty(T * k, dtype=torch.int32, device=DEV)
    core.moe_align(idx2, T, k, E, offs2, st2, pos2, st)
    assert int(st[0]) == 0
    assert torch.equal(idx, idx2) and torch.equal(w, w2) and torch.equal(sg, sg2) and torch.equal(offs, offs2)
    total = int(offs[-1])
    flat = idx.reshape(-1).cpu()
    seen = set()
    for pair in range(T * k):                                     # the inversion is a valid one
        e, p = int(flat[pair]), int(pos[pair])
        if e < 0:
            assert p == -1
            continue
        assert int(offs[e]) <= p < int(offs[e + 1]) and p not in seen and int(sorted_token[p]) == pair // k
        seen.add(p)
    assert len(seen) == total
    assert torch.equal(xs[:total], act[sorted_token[:total].long()])

"""The tcgen05 attention kernel on steps whose sequences go on from the cache (keys before the step
from the cache's pages, the step's own keys from its buffers) against the plain attention function:
unequal pasts and unequal numbers of new tokens in one batch, fresh sequences among them, grouped
heads, windows whose ring has wrapped and whose edge falls inside a page, a far key in the cache that
must dominate.  Pages that no sequence has written hold huge numbers, so that a key that should be
masked shows."""
import math

import pytest
import torch

import gpu_util as G
import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def libs():
    from moe_b200.ops import core, tc

    core.lib(), tc.lib()
    return core, tc


def case(libs, nh, nkv, hd, window, before, new, seed=0, edit=None):
    """-> (output of the kernel, plain reference), rows of all sequences one after another."""
    from moe_b200.cache import KVCache, KVRequest

    core, tc = libs
    torch.manual_seed(seed)
    B = len(new)
    cache = KVCache({0: KVRequest(nkv, hd, window)}, {0: None}, max_tokens=64 * 40, max_slots=B + 1,
                    dtype=torch.bfloat16, device=DEV)
    cache.groups[0].storage.fill_(3e30)
    view = cache.view(0)
    slots = [cache.acquire() for _ in range(B)]
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    K = [torch.randn(a + b, nkv, hd, device=DEV).to(torch.bfloat16) for a, b in zip(before, new)]
    V = [torch.randn(a + b, nkv, hd, device=DEV).to(torch.bfloat16) for a, b in zip(before, new)]
    Q = [torch.randn(b, nh, hd, device=DEV).to(torch.bfloat16) for b in new]
    if edit:
        edit(Q, K, V)
    live = [i for i in range(B) if before[i] > 0]
    if live:                                         # the past goes through the cache
        for i in live:
            G.give_pages(cache, slots[i], before[i])
        b0 = G.make_batch(DEV, [slots[i] for i in live], [0] * len(live), [before[i] for i in live])
        core.kv_commit(torch.cat([K[i][:before[i]] for i in live]).contiguous(),
                       torch.cat([V[i][:before[i]] for i in live]).contiguous(), view, b0, st)
    for i in range(B):
        G.give_pages(cache, slots[i], before[i] + new[i])
    b1 = G.make_batch(DEV, slots, before, new)
    q = torch.cat(Q).contiguous()
    kn = torch.cat([K[i][before[i]:] for i in range(B)]).contiguous()
    vn = torch.cat([V[i][before[i]:] for i in range(B)]).contiguous()
    out = torch.full((q.shape[0], nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    assert tc.attention_cached(q, kn, vn, view, b1, out, nh=nh, window=window, scale=1.0 / math.sqrt(hd), status=st)
    torch.cuda.synchronize()
    assert st[:2].tolist() == [0, 0], st.tolist()
    refs = []
    for i in range(B):
        full_q = torch.zeros(before[i] + new[i], nh, hd, dtype=torch.float64)
        full_q[before[i]:] = Q[i].double().cpu()
        refs.append(plain.attention(full_q, K[i].double().cpu(), V[i].double().cpu(), window)[before[i]:])
    return out.double().cpu(), torch.cat(refs)


PASTS = [([0, 0, 0], [5, 70, 131]),                       # fresh sequences only: no tile from the cache
         ([10, 100], [7, 30]),
         ([130, 64, 0], [70, 129, 200]),                  # past a page's and a tile's edge; a fresh one among them
         ([700, 128, 127, 129, 1], [300, 1, 5, 257, 128]),
         ([63, 64, 65, 191, 192, 193], [1, 2, 64, 65, 3, 130])]


@pytest.mark.parametrize("nh,nkv,hd", [(6, 3, 64), (2, 2, 128), (5, 1, 128), (4, 1, 64)])
@pytest.mark.parametrize("window", [None, 1, 8, 64, 70, 100, 128, 200, 300])
def test_against_plain(libs, nh, nkv, hd, window):
    for n, (before, new) in enumerate(PASTS):
        out, ref = case(libs, nh, nkv, hd, window, before, new, seed=n + hd + (window or 0))
        assert torch.isfinite(out).all(), (before, new)
        o = 0
        for a, b in zip(before, new):
            err = float((out[o:o + b] - ref[o:o + b]).abs().max())
            assert err < 2e-2 * float(ref[o:o + b].abs().max()), (before, new, a, b, err)
            o += b


@pytest.mark.parametrize("hd", [64, 128])
def test_a_far_key_in_the_cache_and_the_windows_edge(libs, hd):
    """One key of the past is made to stand out (query and key scaled): without a window every new
    query must return that key's value; with a window the key counts exactly while it is inside."""
    past, new, far = 600, 150, 37

    def edit(Q, K, V):
        d = torch.zeros(hd, device=DEV)
        d[3] = 1.0
        K[0][far, 0] = (40 * d).to(torch.bfloat16)
        Q[0][:, :] = (40 * d).to(torch.bfloat16)

    out, ref = case(libs, 2, 1, hd, None, [past], [new], edit=edit)
    assert float((out - ref).abs().max()) < 2e-2 * float(ref.abs().max())
    for w in (past - far + 1, past - far + 75):           # inside for the first query only / for the first 75
        out, ref = case(libs, 2, 1, hd, w, [past], [new], edit=edit)
        assert float((out - ref).abs().max()) < 2e-2 * float(ref.abs().max())
        inside = w - (past - far)                         # queries that still see the far key
        assert float((out[:inside] - out[0]).abs().max()) < 1e-2          # they all return its value
        assert float((out[inside] - out[0]).abs().max()) > 0.1            # the next one does not


def test_what_it_does_not_take(libs):
    from moe_b200.cache import KVCache, KVRequest

    core, tc = libs
    cache = KVCache({0: KVRequest(2, 48, None)}, {0: None}, max_tokens=256, max_slots=2, dtype=torch.bfloat16, device=DEV)
    s = cache.acquire()
    G.give_pages(cache, s, 20)
    b = G.make_batch(DEV, [s], [10], [10])
    q = torch.zeros(10, 2, 48, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros(10, 96, device=DEV, dtype=torch.bfloat16)
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    assert not tc.attention_cached(q, q, q, cache.view(0), b, out, nh=2, window=None, scale=1.0, status=st)

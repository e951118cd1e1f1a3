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


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot,window", [(4, 2, 32, 32, None), (3, 1, 64, 32, 72), (2, 2, 128, 128, None),
                                                  (5, 1, 128, 64, 100), (6, 2, 16, 16, None), (2, 1, 48, 48, None),
                                                  (28, 4, 128, 128, None), (7, 1, 64, 64, 150)])
def test_attention_decode_fused_equals_rope_commit_then_attention(core, dt, nh, nkv, hd, rot, window):
    """Rotation + append + attention + merge in one launch against the three launches it replaces:
    the same cache afterwards and the same output.  Sequences at a page's first and last place, in
    the middle of a ring that has wrapped, and a padding row."""
    from moe_b200.cache import KVCache, KVRequest

    lens = [0, 63, 64, 200, 321]
    B = len(lens)
    torch.manual_seed(hd + nh)
    qkv = torch.randn(B + 1, (nh + 2 * nkv) * hd, device=DEV)
    inv = plain.rope_inv_freq(1e4, rot).to(DEV)
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    outs = []
    fast_ok = (hd * (4 if dt == torch.float32 else 2)) in (64, 128, 256, 512)
    for fused in (False, True):
        cache = KVCache({0: KVRequest(nkv, hd, window)}, {0: None}, 4096, B, dt, DEV)
        view = cache.view(0)
        g = torch.Generator(device=DEV).manual_seed(7)
        view.group.storage.copy_(torch.randn(view.group.storage.shape, device=DEV, generator=g).to(dt))
        slots = [cache.acquire() for _ in range(B)]
        for s, n in zip(slots, lens):
            G.give_pages(cache, s, n + 1)
        batch = G.make_batch(DEV, slots + [cache.padding_slot], lens + [0], [1] * (B + 1))
        batch.seq_of_token[B] = -1
        out = torch.full((B + 1, nh * hd), 7.0, device=DEV, dtype=dt)
        scale = 1.0 / hd ** 0.5
        if fused:
            done = core.attention_decode_fused(qkv, inv, rot, view, batch, out, nh=nh, window=window, scale=scale,
                                               status=st)
            assert done == fast_ok
            if not done:
                return
        else:
            q = torch.zeros(B + 1, nh, hd, device=DEV, dtype=dt)
            core.rope_commit(qkv, batch.pos, inv, nh, nkv, hd, rot, q, view, batch, st)
            core.attention_decode(q, view, batch, out, nh=nh, window=window, scale=scale, status=st)
        outs.append((out.float().clone(), view.group.storage.float().clone()))
    assert int(st[0]) == 0
    tol = 1e-5 if dt == torch.float32 else 2.0 ** -7
    assert torch.allclose(outs[0][1], outs[1][1], rtol=tol, atol=tol * 1e-2)          # the cache
    assert float(outs[1][0][B].abs().sum()) == 0.0                                       # padding row: zeros
    err = (outs[0][0] - outs[1][0]).abs().max() / outs[0][0].abs().max()
    assert float(err) < tol, float(err)
    # the tickets are left at zero
    assert int(core._tickets(DEV, 1).abs().sum()) == 0


@pytest.mark.parametrize("E,k,H,norm,T", [(60, 4, 2048, False, 8), (8, 3, 96, True, 1), (4, 2, 64, False, 64),
                                           (200, 8, 72, True, 13), (5, 5, 100, True, 3)])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
def test_norm_route_equals_rmsnorm_then_route_dispatch(core, E, k, H, norm, T, wdt):
    """Norm + router + dispatch in one launch against the separate kernels: the same stream, the
    same normalised rows, the same picks (unless two experts are closer than rounding), a valid
    inversion and the gathered rows."""
    torch.manual_seed(E + T)
    bf16 = wdt == torch.bfloat16
    x0 = torch.randn(T, H, device=DEV)
    delta = torch.randn(T, H, device=DEV)
    nw = 1.0 + 0.1 * torch.randn(H, device=DEV)
    wr = torch.randn(E, H, device=DEV).to(wdt)
    wsg = torch.randn(H, device=DEV).to(wdt)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    if T > 4:
        seq[T - 2] = -1                                           # a padding row
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    eps = 1e-5
    # the separate kernels
    x1 = x0.clone()
    o32 = torch.empty(T, H, device=DEV)
    o16 = torch.empty(T, H, device=DEV, dtype=torch.bfloat16) if bf16 else None
    core.rmsnorm(x1, nw, eps, delta=delta, out32=o32, out16=o16, write_back=True, status=st)
    idx1, w1, sg1, offs1, _, _, _ = core.route_dispatch(o32, wr, k, norm, 1.5, shared_gate_w=wsg, seq_of_token=seq,
                                                       gather=o16, status=st)
    # the fused kernel
    x2 = x0.clone()
    res = core.norm_route(x2, delta, nw, eps, wr, k, norm, 1.5, bf16=bf16, shared_gate_w=wsg, seq_of_token=seq,
                          status=st)
    assert res is not None
    out32, out16, idx, w, sg, offs, sorted_token, pos, xs = res
    assert int(st[0]) == 0
    assert torch.equal(x1, x2)
    if bf16:
        assert out32 is None and float((out16.float() - o16.float()).abs().max()) <= 2.0 ** -7 * float(o16.float().abs().max())
    else:
        assert out16 is None and torch.allclose(out32, o32, rtol=1e-5, atol=1e-6)
    # picks: equal, or the probabilities of the differing experts agree to rounding
    probs = torch.softmax(o32.double() @ wr.double().T, dim=-1)
    for t in range(T):
        a, b = set(idx1[t].tolist()), set(idx[t].tolist())
        if a != b:
            diff = sorted(a ^ b)
            assert a != {-1} and float(probs[t, diff].max() - probs[t, diff].min()) < 1e-5, (t, a, b)
        else:
            order = torch.argsort(idx[t]), torch.argsort(idx1[t])
            assert torch.allclose(w[t][order[0]], w1[t][order[1]], rtol=1e-4, atol=1e-7)
    assert torch.allclose(sg, sg1, rtol=1e-4, atol=1e-6)
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
    assert (xs is not None) == (bf16 and (H * 2) % 16 == 0)
    if xs is not None:
        assert torch.equal(xs[:total], out16[sorted_token[:total].long()])
    assert int(core._tickets(DEV, 1).abs().sum()) == 0


@pytest.mark.parametrize("T,H,E,k,rows", [(8, 2048, 60, 4, None), (5, 96, 6, 3, [4, 0, 2]), (300, 264, 9, 2, None),
                                          (3, 100, 4, 4, None)])
@pytest.mark.parametrize("bf16", [False, True])
def test_rmsnorm_with_uncombined_delta_equals_combine_then_rmsnorm(core, T, H, E, k, rows, bf16):
    """The norm that forms the routed experts' delta inside its own kernel against the combine
    kernel followed by the plain norm: the same stream and the same normalised rows."""
    from moe_b200.parts.feedforward import CombineDelta

    torch.manual_seed(T + H)
    x0 = torch.randn(T, H, device=DEV)
    nw = 1.0 + 0.1 * torch.randn(H, device=DEV)
    P = T * k
    y = torch.randn(P, H, device=DEV)
    pos = torch.randperm(P, device=DEV).to(torch.int32)
    if T > 2:
        pos[k] = -1                                               # a pair without an expert
    w = torch.rand(T, k, device=DEV)
    shared = torch.randn(T, H, device=DEV)
    gate = torch.rand(T, device=DEV)
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    r = None if rows is None else torch.tensor(rows, dtype=torch.int32, device=DEV)
    n = T if rows is None else len(rows)
    outs = []
    for fused in (False, True):
        x = x0.clone()
        o32 = torch.empty(n, H, device=DEV)
        o16 = torch.empty(n, H, device=DEV, dtype=torch.bfloat16) if bf16 else None
        cd = CombineDelta(y, pos, w.reshape(-1), k, shared, gate, T, H)
        if fused:
            assert core.rmsnorm_combine(x, cd, nw, 1e-6, rows=r, out32=o32, out16=o16, write_back=rows is None,
                                        status=st) == (H % 4 == 0)
            if H % 4:
                return
        else:
            delta = torch.empty(T, H, device=DEV)
            core.moe_combine(y, pos, w.reshape(-1), k, delta, shared=shared, shared_gate=gate)
            core.rmsnorm(x, nw, 1e-6, delta=delta, rows=r, out32=o32, out16=o16, write_back=rows is None, status=st)
        outs.append((x, o32, o16))
    assert int(st[0]) == 0
    assert torch.allclose(outs[0][0], outs[1][0], rtol=1e-6, atol=1e-6)
    assert torch.allclose(outs[0][1], outs[1][1], rtol=1e-5, atol=1e-6)
    if bf16:
        assert float((outs[0][2].float() - outs[1][2].float()).abs().max()) <= 2.0 ** -7 * float(outs[0][2].float().abs().max())
    if rows is not None:
        assert torch.equal(outs[1][0], x0)                        # selected rows: the stream is left alone


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,where,seen", [(None, 0, True), (None, 299, True), (None, "self", True),
                                                (100, 201, True), (100, 200, False), (100, "self", True)])
def test_fused_decode_attention_finds_one_key_among_hundreds(core, dt, window, where, seen):
    """Random keys would hide a key that is skipped or taken twice.  Here every cached key is zero
    except ONE, which points along the query, and only its value is non-zero: the output is about
    0.9 if that key is seen and 0 if not.  The key sits at the sequence's first position, at its
    last cached one, at the window's first position, just before the window, or it is the step's
    own key (which the fused kernel takes from the q/k/v row, not from the cache)."""
    from moe_b200.cache import KVCache, KVRequest

    nh, nkv, hd, p = 2, 1, 64, 300                               # the new token's position
    cache = KVCache({0: KVRequest(nkv, hd, window)}, {0: None}, 1024, 2, dt, DEV)
    view, grp = cache.view(0), cache.groups[0]
    slot = cache.acquire()
    G.give_pages(cache, slot, p + 1)
    batch = G.make_batch(DEV, [slot], [p], [1])
    u = torch.zeros(hd, device=DEV)
    u[5] = 8.0
    qkv = torch.zeros(1, (nh + 2 * nkv) * hd, device=DEV)
    qkv[0, :hd] = u                                              # head 0 asks for u; head 1 asks for nothing
    if where == "self":
        qkv[0, nh * hd:(nh + 1) * hd] = u                        # the step's own key ...
        qkv[0, (nh + 1) * hd:] = 1.0                             # ... and value
    else:
        r = where % grp.ring if grp.ring else where
        page = int(grp.table[slot, r // 64])
        view.k[page, 0, r % 64] = u.to(dt)
        view.v[page, 0, r % 64] = 1.0
    out = torch.full((1, nh * hd), 7.0, device=DEV, dtype=dt)
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    assert core.attention_decode_fused(qkv, None, 0, view, batch, out, nh=nh, window=window, scale=1.0 / 8.0, status=st)
    assert int(st[0]) == 0
    n = min(window, p + 1) if window else p + 1                  # keys the query sees
    want = float(torch.exp(torch.tensor(8.0)) / (torch.exp(torch.tensor(8.0)) + n - 1)) if seen else 0.0
    head0, head1 = out[0, :hd].float(), out[0, hd:].float()
    assert float((head0 - want).abs().max()) < 1e-2, (float(head0[0]), want)
    assert float((head1 - (1.0 / n if seen else 0.0)).abs().max()) < 1e-3      # head 1: a plain mean of the values

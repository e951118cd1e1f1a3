"""Each kernel alone against a plain PyTorch float32/float64 reference of the same op, at
sizes other than the engine's tiny configurations (widths and vocabularies that are no power
of two, odd head counts, head sizes in steps of 16)."""
import math

import numpy as np
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


def status():
    return torch.zeros(4, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_embed(core, dt):
    V, H, T = 301, 72, 19
    table = torch.randn(V, H, device=DEV).to(dt)
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    out = torch.empty(T, H, device=DEV)
    st = status()
    core.embed(table, ids, out, st)
    assert torch.equal(out, table[ids.long()].float()) and int(st[0]) == 0
    ids[3] = V
    core.embed(table, ids, out, st)
    assert int(st[0]) & 1


@pytest.mark.parametrize("H", [48, 100, 2048, 5000])
def test_rmsnorm_with_residual_rows_and_bf16_copy(core, H):
    T, eps = 13, 1e-5
    x = torch.randn(T, H, device=DEV) * 3
    delta = torch.randn(T, H, device=DEV)
    w = torch.rand(H, device=DEV) + 0.5
    ref_sum = x.double() + delta.double()
    ref = ref_sum / torch.sqrt((ref_sum ** 2).mean(-1, keepdim=True) + eps) * w.double()
    o32, o16 = torch.empty(T, H, device=DEV), torch.empty(T, H, device=DEV, dtype=torch.bfloat16)
    x1 = x.clone()
    core.rmsnorm(x1, w, eps, delta=delta, out32=o32, out16=o16, status=status())
    assert torch.allclose(x1.double(), ref_sum, atol=1e-6)                 # the sum was written back
    assert torch.allclose(o32.double(), ref, atol=2e-6, rtol=1e-5)
    assert torch.equal(o16, o32.to(torch.bfloat16))                        # rounded from the 32-bit value
    rows = torch.tensor([7, 0, 7, 12], dtype=torch.int32, device=DEV)
    x2 = x.clone()
    o = torch.empty(4, H, device=DEV)
    core.rmsnorm(x2, w, eps, delta=delta, rows=rows, out32=o, status=status())
    assert torch.equal(x2, x)                                              # a row subset leaves x alone
    assert torch.allclose(o.double(), ref[rows.long()], atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("adt,wdt,odt", [(torch.float32, torch.float32, torch.float32),
                                         (torch.bfloat16, torch.bfloat16, torch.float32),
                                         (torch.bfloat16, torch.float32, torch.bfloat16),
                                         (torch.float32, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (37, 53, 19), (130, 200, 96), (64, 64, 16), (3, 1000, 333), (8, 2048, 1408),
                                    (16, 61, 2048), (13, 331, 1100), (17, 40, 2052)])
def test_gemm_generic_any_size_and_dtype(core, adt, wdt, odt, M, N, K):
    a = torch.randn(M, K, device=DEV).to(adt)
    w = torch.randn(N, K, device=DEV).to(wdt)
    b = torch.randn(N, device=DEV)
    out = torch.empty(M, N, device=DEV, dtype=odt)
    core.gemm_generic(a, w, out, bias=b, status=status())
    ref = a.double() @ w.double().T + b.double()
    tol = 1e-5 if odt == torch.float32 else 1e-2
    assert float((out.double() - ref).abs().max() / ref.abs().max()) < tol


def test_gemm_generic_gives_a_row_the_same_to_the_bit_alone_and_among_many(core):
    """Few rows and many rows take different kernels; both add the products of one output in the
    order of k with one accumulator, so a token's projection does not depend on its company."""
    torch.manual_seed(4)
    for K, N in ((2048, 300), (1100, 64), (72, 1000)):
        a = torch.randn(200, K, device=DEV)
        w = torch.randn(N, K, device=DEV)
        many = torch.empty(200, N, device=DEV)
        core.gemm_generic(a, w, many, status=status())
        for rows in ([5], [0, 17, 199], list(range(40, 48))):
            few = torch.empty(len(rows), N, device=DEV)
            core.gemm_generic(a[rows].contiguous(), w, few, status=status())
            assert torch.equal(few, many[rows]), (K, N, rows)


def test_gemm_generic_is_true_32_bit(core):
    """Values that a reduced-precision matrix mode (tf32: 10 bits of mantissa) would destroy."""
    K = 256
    a = (1.0 + torch.arange(K, device=DEV, dtype=torch.float32) * 2.0 ** -20).reshape(1, K)
    w = torch.ones(1, K, device=DEV)
    w[0, 1::2] = -1.0
    out = torch.empty(1, 1, device=DEV)
    core.gemm_generic(a, w, out, status=status())
    ref = float((a.double() @ w.double().T)[0, 0])          # = -128 * 2^-20, lost entirely at 10 bits
    assert abs(float(out[0, 0]) - ref) < 1e-7 and abs(ref) > 1e-5


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("counts", [[0, 70, 3, 0, 9], [2, 0, 11, 1, 8], [0, 0, 1, 0, 0]])     # many rows; few rows: another kernel
def test_gemm_generic_grouped_with_gather(core, dt, counts):
    G_, N, K, S = 5, 45, 1070, 23
    a = torch.randn(S, K, device=DEV).to(dt)
    w = torch.randn(G_, N, K, device=DEV).to(dt)
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    M = sum(counts)
    rows = torch.randint(0, S, (M,), device=DEV, dtype=torch.int32)
    out = torch.full((M, N), float("nan"), device=DEV)
    core.gemm_generic(a, w, out, a_rows=rows, group_offsets=offs, status=status())
    ref = torch.empty(M, N, dtype=torch.float64, device=DEV)
    o = 0
    for g, c in enumerate(counts):
        ref[o:o + c] = a[rows[o:o + c].long()].double() @ w[g].double().T
        o += c
    assert float((out.double() - ref).abs().max() / ref.abs().max()) < 1e-5
    st = status()
    rows[M // 2] = S + 4
    core.gemm_generic(a, w, out, a_rows=rows, group_offsets=offs, status=st)
    assert int(st[0]) & 16


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot,window", [(4, 2, 16, 16, None), (3, 1, 32, 16, 70), (2, 2, 128, 128, 130)])
def test_rope_split_with_commit_equals_rope_split_then_kv_commit(core, dt, nh, nkv, hd, rot, window):
    """Whole prompts of unequal lengths (one longer than the window's ring) and a padding row: the
    launch that also appends to the cache leaves the cache as the separate launch does."""
    from moe_b200.cache import KVCache, KVRequest

    lens = [1, 63, 200, 65]
    B, T = len(lens), sum(lens) + 1
    torch.manual_seed(hd)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV)
    inv = plain.rope_inv_freq(1e4, rot).to(DEV)
    st = status()
    results = []
    for fused in (False, True):
        cache = KVCache({0: KVRequest(nkv, hd, window)}, {0: None}, 2048, B, dt, DEV)
        view = cache.view(0)
        slots = [cache.acquire() for _ in range(B)]
        for s, n in zip(slots, lens):
            G.give_pages(cache, s, n)
        batch = G.make_batch(DEV, slots + [cache.padding_slot], [0] * (B + 1), lens + [1])
        batch.seq_of_token[T - 1] = -1
        q = torch.zeros(T, nh, hd, device=DEV, dtype=dt)
        k = torch.zeros(T, nkv, hd, device=DEV, dtype=dt)
        v = torch.zeros(T, nkv, hd, device=DEV, dtype=dt)
        if fused:
            assert core.rope_split(qkv, batch.pos, inv, nh, nkv, hd, rot, q, k, v, commit=(view, batch), status=st)
        else:
            core.rope_split(qkv, batch.pos, inv, nh, nkv, hd, rot, q, k, v)
            core.kv_commit(k, v, view, batch, st)
        results.append((q.clone(), k.clone(), v.clone(), view.group.storage.clone()))
    assert int(st[0]) == 0
    for a, b in zip(*results):
        assert torch.equal(a, b)
    assert float(results[1][3].abs().sum()) > 0 and float(results[1][3][:, :, 0].abs().sum()) == 0.0   # not the scratch page


@pytest.mark.parametrize("nh,nkv,hd,rot", [(3, 1, 32, 32), (4, 2, 16, 16), (5, 5, 48, 48), (2, 1, 64, 32), (2, 2, 16, 0),
                                           (2, 1, 20, 12)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rope_split(core, nh, nkv, hd, rot, dt):
    T = 11
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV)
    pos = torch.tensor([0, 1, 2, 3, 100, 1000, 4095, 7, 8, 9, 31999], dtype=torch.int32, device=DEV)
    inv = plain.rope_inv_freq(1e6, rot).to(DEV) if rot else None
    q = torch.empty(T, nh, hd, device=DEV, dtype=dt)
    k = torch.empty(T, nkv, hd, device=DEV, dtype=dt)
    v = torch.empty(T, nkv, hd, device=DEV, dtype=dt)
    core.rope_split(qkv, pos, inv, nh, nkv, hd, rot, q, k, v)
    src = qkv.double().cpu()
    qs, ks, vs = (src[:, :nh * hd].reshape(T, nh, hd), src[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd),
                  src[:, (nh + nkv) * hd:].reshape(T, nkv, hd))
    if rot:
        qs = torch.cat([plain.rope(qs[..., :rot], pos.cpu(), inv.cpu()), qs[..., rot:]], -1)
        ks = torch.cat([plain.rope(ks[..., :rot], pos.cpu(), inv.cpu()), ks[..., rot:]], -1)
    tol = 5e-6 if dt == torch.float32 else 1e-2
    for got, ref in ((q, qs), (k, ks), (v, vs)):
        assert float((got.double().cpu() - ref).abs().max()) < tol * float(ref.abs().max())


def _attention_case(core, dt, nh, nkv, hd, window, lens_before, lens_new, seed=0, ring_wrap=False):
    """Random keys: some already in the cache (written by kv_commit in an earlier 'step'), some new."""
    from moe_b200.cache import KVCache, KVRequest

    torch.manual_seed(seed)
    B = len(lens_new)
    cache = KVCache({0: KVRequest(nkv, hd, window)}, {0: None}, max_tokens=4096, max_slots=B + 1, dtype=dt, device=DEV)
    view = cache.view(0)
    slots = [cache.acquire() for _ in range(B)]
    st = status()
    K = [torch.randn(a + b, nkv, hd, device=DEV).to(dt) for a, b in zip(lens_before, lens_new)]
    V = [torch.randn(a + b, nkv, hd, device=DEV).to(dt) for a, b in zip(lens_before, lens_new)]
    Q = [torch.randn(b, nh, hd, device=DEV).to(dt) for b in lens_new]
    live = [i for i in range(B) if lens_before[i] > 0]
    if live:                                         # the past goes through the cache
        for i in live:
            G.give_pages(cache, slots[i], lens_before[i])
        b0 = G.make_batch(DEV, [slots[i] for i in live], [0] * len(live), [lens_before[i] for i in live])
        core.kv_commit(torch.cat([K[i][:lens_before[i]] for i in live]).contiguous(),
                       torch.cat([V[i][:lens_before[i]] for i in live]).contiguous(), view, b0, st)
    for i in range(B):
        G.give_pages(cache, slots[i], lens_before[i] + lens_new[i])
    b1 = G.make_batch(DEV, slots, lens_before, lens_new)
    q = torch.cat(Q).contiguous()
    kn = torch.cat([K[i][lens_before[i]:] for i in range(B)]).contiguous()
    vn = torch.cat([V[i][lens_before[i]:] for i in range(B)]).contiguous()
    out = torch.empty(q.shape[0], nh * hd, device=DEV, dtype=dt)
    scale = 1.0 / math.sqrt(hd)
    core.attention_generic(q, kn, vn, view, b1, out, nh=nh, window=window, scale=scale, use_local=True, status=st)
    # the tiled kernel (64 queries to a block) gives the same as the plain one
    tiled = torch.full_like(out, float("nan"))
    assert core.attention_tiled(q, kn, vn, view, b1, tiled, nh=nh, window=window, scale=scale, use_local=True, status=st)
    cut = 2e-6 if dt == torch.float32 else 1e-2
    assert float((tiled.double() - out.double()).abs().max()) <= cut * float(out.double().abs().max())
    # after the commit, the same queries must see the same thing from the cache alone
    core.kv_commit(kn, vn, view, b1, st)
    out2 = torch.empty_like(out)
    if all(n == 1 for n in lens_new):
        # the decode kernel (split along the keys) and the plain kernel, both over the cache alone
        core.attention_decode(q, view, b1, out2, nh=nh, window=window, scale=scale, status=st)
        out3 = torch.empty_like(out)
        core.attention_generic(q, kn, vn, view, b1, out3, nh=nh, window=window, scale=scale, use_local=False, status=st)
        assert float((out3.double() - out2.double()).abs().max()) < 2e-2 * float(out3.double().abs().max())
    elif window is None:
        core.attention_generic(q, kn, vn, view, b1, out2, nh=nh, window=window, scale=scale, use_local=False, status=st)
        t2 = torch.full_like(out, float("nan"))
        assert core.attention_tiled(q, kn, vn, view, b1, t2, nh=nh, window=window, scale=scale, use_local=False, status=st)
        assert float((t2.double() - out2.double()).abs().max()) <= cut * float(out2.double().abs().max())
    else:
        out2 = None
    assert int(st[0]) == 0
    refs = []
    for i in range(B):
        full_q = torch.zeros(lens_before[i] + lens_new[i], nh, hd, dtype=torch.float64)
        full_q[lens_before[i]:] = Q[i].double().cpu()
        r = plain.attention(full_q, K[i].double().cpu(), V[i].double().cpu(), window)
        refs.append(r[lens_before[i]:])
    return out.double().cpu(), (out2.double().cpu() if out2 is not None else None), torch.cat(refs)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (3, 1, 32, 8), (6, 3, 48, 100), (2, 2, 128, None),
                                               (5, 1, 80, 70), (1, 1, 256, 64), (28, 4, 128, None), (7, 1, 64, 150)])
def test_attention_over_cache_and_new_keys(core, dt, nh, nkv, hd, window):
    tol = 2e-5 if dt == torch.float32 else 2e-2
    # prompts from an empty cache, unequal lengths
    out, out2, ref = _attention_case(core, dt, nh, nkv, hd, window, [0, 0, 0], [5, 70, 131])
    assert float((out - ref).abs().max()) < tol * float(ref.abs().max())
    # one token each, over caches of unequal lengths (several pages; a ring that has wrapped)
    out, out2, ref = _attention_case(core, dt, nh, nkv, hd, window, [63, 64, 200, 1], [1, 1, 1, 1], seed=1)
    assert float((out - ref).abs().max()) < tol * float(ref.abs().max())
    assert out2 is not None and float((out2 - ref).abs().max()) < tol * float(ref.abs().max())
    # a continuation by several tokens
    out, out2, ref = _attention_case(core, dt, nh, nkv, hd, window, [10, 100], [7, 30], seed=2)
    assert float((out - ref).abs().max()) < tol * float(ref.abs().max())
    # chunks of a long prompt: more than one tile of queries, past a page's and a tile's edge
    out, out2, ref = _attention_case(core, dt, nh, nkv, hd, window, [130, 64, 0], [70, 129, 200], seed=3)
    assert float((out - ref).abs().max()) < tol * float(ref.abs().max())


@pytest.mark.parametrize("E,k,H,norm,scale", [(10, 3, 72, True, 1.0), (60, 4, 200, False, 1.0), (7, 7, 33, True, 2.5),
                                               (130, 8, 64, False, 0.5)])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [29, 150])              # few tokens and many: two kernels
def test_router_and_shared_gate(core, E, k, H, norm, scale, wdt, T):
    h = torch.randn(T, H, device=DEV)
    wr = torch.randn(E, H, device=DEV).to(wdt)
    wsg = torch.randn(H, device=DEV).to(wdt)
    idx = torch.empty(T, k, dtype=torch.int32, device=DEV)
    wt = torch.empty(T, k, device=DEV)
    sg = torch.empty(T, device=DEV)
    core.router(h, wr, k, norm, scale, idx, wt, shared_gate_w=wsg, shared_gate=sg)
    cfg = dict(num_experts_per_tok=k, norm_topk_prob=norm, routed_scaling_factor=scale)
    picks, weights = plain.route(cfg, {"p.mlp.gate.weight": wr.double().cpu()}, "p.", h.double().cpu())
    assert idx.cpu().tolist() == picks
    assert torch.allclose(wt.double().cpu(), torch.stack(weights), rtol=2e-5, atol=1e-7)
    ref_g = torch.sigmoid(h.double().cpu() @ wsg.double().cpu())
    assert torch.allclose(sg.double().cpu(), ref_g, rtol=2e-5, atol=1e-7)


def test_router_ties_go_to_the_lower_index_and_padding_rows_get_no_expert(core):
    E, k, H = 6, 2, 16
    wr = torch.zeros(E, H, device=DEV)
    wr[1, 0] = wr[4, 0] = wr[5, 0] = 1.0                      # experts 1, 4, 5 tie at the top
    h = torch.ones(3, H, device=DEV)
    idx = torch.empty(3, k, dtype=torch.int32, device=DEV)
    wt = torch.empty(3, k, device=DEV)
    seq = torch.tensor([0, -1, 0], dtype=torch.int32, device=DEV)
    core.router(h, wr, k, False, 1.0, idx, wt, seq_of_token=seq)
    assert idx.cpu().tolist() == [[1, 4], [-1, -1], [1, 4]] and float(wt[1].abs().sum()) == 0.0


@pytest.mark.parametrize("T,k,E", [(1, 2, 4), (37, 3, 8), (500, 4, 60), (9, 8, 8)])
def test_moe_align_inverts_the_table(core, T, k, E):
    torch.manual_seed(T)
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32).to(DEV)
    if T > 5:
        idx[3] = -1                                            # a padding row
    offs = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    st_ = torch.full((T * k,), -7, dtype=torch.int32, device=DEV)
    pp = torch.empty(T * k, dtype=torch.int32, device=DEV)
    s = status()
    core.moe_align(idx, T, k, E, offs, st_, pp, s)
    offs, st_, pp, flat = offs.cpu(), st_.cpu(), pp.cpu(), idx.cpu().reshape(-1)
    counts = torch.bincount(flat[flat >= 0].long(), minlength=E)
    assert offs.tolist() == [0] + torch.cumsum(counts, 0).tolist() and int(s[0]) == 0
    seen = set()
    for pair in range(T * k):
        e, p = int(flat[pair]), int(pp[pair])
        if e < 0:
            assert p == -1
            continue
        assert offs[e] <= p < offs[e + 1] and p not in seen and int(st_[p]) == pair // k
        seen.add(p)
    assert len(seen) == int(offs[-1])
    idx[0, 0] = E
    core.moe_align(idx, T, k, E, torch.empty(E + 1, dtype=torch.int32, device=DEV), st_.to(DEV), pp.to(DEV), s)
    assert int(s[0]) & 4


@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_swiglu_and_combine(core, odt):
    M, I = 21, 37
    gu = torch.randn(M, 2 * I, device=DEV) * 3
    act = torch.empty(M, I, device=DEV, dtype=odt)
    core.swiglu(gu, act)
    g, u = gu[:, :I].double(), gu[:, I:].double()
    ref = g / (1 + torch.exp(-g)) * u
    err = (act.double() - ref).abs()
    assert bool((err <= (1e-6 if odt == torch.float32 else 2.0 ** -8) * ref.abs() + 1e-6).all())
    T, k, H = 7, 3, 50
    y = torch.randn(T * k, H, device=DEV)
    pos = torch.randperm(T * k, device=DEV).to(torch.int32)
    pos[4] = -1
    w = torch.rand(T, k, device=DEV)
    sh, sgate = torch.randn(T, H, device=DEV), torch.rand(T, device=DEV)
    out = torch.empty(T, H, device=DEV)
    core.moe_combine(y, pos, w, k, out, shared=sh, shared_gate=sgate)
    ref = torch.zeros(T, H, dtype=torch.float64, device=DEV)
    for t in range(T):
        for j in range(k):
            p = int(pos[t * k + j])
            if p >= 0:
                ref[t] += w[t, j].double() * y[p].double()
        ref[t] += sgate[t].double() * sh[t].double()
    assert torch.allclose(out.double(), ref, atol=1e-5)


def test_table_update_and_seed_rng(core):
    table = torch.zeros(5, 9, dtype=torch.int32, device=DEV)
    upd = torch.tensor([1, 2, 33, 4, 8, 44, 0, 0, 55], dtype=torch.int32, device=DEV)
    core.table_update(table, upd, 3)
    assert int(table[1, 2]) == 33 and int(table[4, 8]) == 44 and int(table[0, 0]) == 55 and int(table.sum()) == 132
    states = torch.zeros(6, dtype=torch.int64, device=DEV)
    slots = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    seeds = torch.tensor([7, 0], dtype=torch.int64, device=DEV)
    core.seed_rng(states, slots, seeds)
    got = states.cpu().numpy().view(np.uint64)
    assert int(got[4]) == plain.Rng(7).s and int(got[1]) == plain.Rng(0).s and int(got[0]) == 0


def test_three_bfloat16_terms_hold_a_float32_exactly(core):
    torch.manual_seed(0)
    x = torch.randn(37, 264, device=DEV) * torch.logspace(-6, 6, 264, device=DEV)
    x[0, :4] = torch.tensor([0.0, -0.0, 1.0, 3.0e38], device=DEV)
    p = core.split3(x).float().reshape(37, 3, 264)
    assert torch.equal(p[:, 0] + p[:, 1] + p[:, 2], x)                  # added in this order, nothing is lost
    assert torch.equal(p[:, 0], x.to(torch.bfloat16).float())            # the first term is the rounded value


@pytest.mark.parametrize("T,E,k,H,gate", [(300, 60, 4, 2048, True), (1000, 7, 2, 264, False), (2048, 64, 8, 3584, True)])
def test_router_logits_on_the_tensor_cores_equal_the_32_bit_ones(core, T, E, k, H, gate):
    """A prompt's router logits as a tensor-core product of the activations' three bfloat16 terms
    against the bfloat16 router rows: the same logits as the 32-bit kernel to a few units of the
    last place of a sum of H terms, and the same picks wherever two experts are not closer than that."""
    from moe_b200.ops import tc

    torch.manual_seed(T + E)
    h = torch.randn(T, H, device=DEV)
    wr = (torch.randn(E, H, device=DEV) * 0.05).to(torch.bfloat16)
    wg = (torch.randn(H, device=DEV) * 0.05).to(torch.bfloat16) if gate else None
    rows = torch.cat([wr] + ([wg.reshape(1, -1)] if gate else []), dim=0)
    w3 = torch.cat([rows, rows, rows], dim=1).contiguous()
    logits = torch.empty(T, rows.shape[0], device=DEV)
    assert tc.gemm_tc(core.split3(h), w3, logits, bn=64, splits=8, status=status())
    ref = h.double() @ rows.double().T
    scale = float(ref.abs().max())
    assert float((logits.double() - ref).abs().max()) < 3e-6 * scale
    idx, w = torch.empty(T, k, dtype=torch.int32, device=DEV), torch.empty(T, k, device=DEV)
    sg = torch.empty(T, device=DEV) if gate else None
    core.router_topk(logits, k, True, 1.0, idx, w, num_experts=E, shared_gate=sg)
    idx2, w2 = torch.empty_like(idx), torch.empty_like(w)
    sg2 = torch.empty(T, device=DEV) if gate else None
    core.router(h, wr, k, True, 1.0, idx2, w2, shared_gate_w=wg, shared_gate=sg2)
    same = (idx.sort(dim=1).values == idx2.sort(dim=1).values).all(dim=1)
    top = torch.sort(ref[:, :E], dim=1, descending=True).values
    margin = (top[:, k - 1] - top[:, k]) / scale if E > k else torch.ones(T, device=DEV, dtype=torch.float64)
    assert bool((same | (margin < 1e-5)).all())
    assert float(same.float().mean()) > 0.99
    assert torch.allclose(w[same], w2[same], atol=1e-5)
    if gate:
        assert torch.allclose(sg, sg2, atol=1e-5)

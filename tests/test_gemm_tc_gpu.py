"""The tcgen05 / TMA matrix product against a float64 product of the same bfloat16 values:
plain and SwiGLU epilogues, every token tile, K splits, groups with gaps, ragged edges."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def tc():
    from moe_b200.ops import tc as t

    t.lib()
    return t


@pytest.fixture(autouse=True, params=["pairs", "single", "two-accumulators"])
def pairing(request, tc):
    """Many tokens take pairs of CTAs on tiles of 256 features (cta_group::2), or, switched off, one
    CTA per tile; SwiGLU for many tokens has one accumulator (gate and up rows interleaved by the
    loads) or, switched off, two: every test runs all ways."""
    tc.lib().moe_tc_set_pair(1 if request.param == "pairs" else 0)
    tc.lib().moe_tc_set_swiglu_interleaved(0 if request.param == "two-accumulators" else 1)
    yield
    tc.lib().moe_tc_set_pair(0)
    tc.lib().moe_tc_set_swiglu_interleaved(1)


def status():
    return torch.zeros(4, dtype=torch.int32, device=DEV)


def rel(got, ref):
    return float((got.double() - ref).abs().max() / ref.abs().max().clamp(min=1e-30))


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 200, 72), (13, 2056, 2048), (64, 384, 200), (100, 130, 1408),
                                    (300, 256, 512), (2, 6144, 2048)])
@pytest.mark.parametrize("bn", [16, 64, 256])
@pytest.mark.parametrize("splits", [1, 3, 12])    # up to 8: summed inside a cluster; more: through global memory
def test_plain(tc, M, N, K, bn, splits):
    torch.manual_seed(M * 1000 + N + K)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.1).to(torch.bfloat16)
    b = torch.randn(N, device=DEV)
    ref = x.double() @ w.double().T + b.double()
    for odt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        out = torch.full((M, N), float("nan"), device=DEV, dtype=odt)
        st = status()
        assert tc.gemm_tc(x, w, out, bias=b, bn=bn, splits=splits, status=st)
        assert int(st[0]) == 0 and rel(out, ref) < tol
    assert int(tc.workspace(DEV).tickets.sum()) == 0          # tickets are left at zero


@pytest.mark.parametrize("M,I,K", [(5, 128, 64), (8, 1408, 2048), (70, 48, 96), (33, 200, 520)])
@pytest.mark.parametrize("bn", [16, 128])
@pytest.mark.parametrize("splits", [1, 4, 9])
def test_swiglu(tc, M, I, K, bn, splits):
    torch.manual_seed(M + I)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device=DEV) * 0.1).to(torch.bfloat16)
    g, u = x.double() @ w[:I].double().T, x.double() @ w[I:].double().T
    ref = g / (1 + torch.exp(-g)) * u
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    st = status()
    assert tc.gemm_tc(x, w, out, swiglu=True, bn=bn, splits=splits, status=st)
    assert int(st[0]) == 0
    err = (out.double() - ref).abs()
    assert bool((err <= 2.0 ** -8 * ref.abs() + 1e-3 * float(ref.abs().max())).all())


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("bn", [16, 32, 128, 256])
@pytest.mark.parametrize("splits", [1, 2])
def test_grouped(tc, swiglu, bn, splits):
    G, N, K = 7, 160, 264
    counts = [0, 40, 1, 0, 17, 130, 3]                      # empty groups; one longer than a tile
    M = sum(counts)
    torch.manual_seed(bn)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(G, (2 * N if swiglu else N), K, device=DEV) * 0.1).to(torch.bfloat16)
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    out = torch.full((M, N), float("nan"), device=DEV)
    st = status()
    assert tc.gemm_tc(x, w, out, swiglu=swiglu, group_offsets=offs, bn=bn, splits=splits, status=st)
    ref = torch.empty(M, N, dtype=torch.float64, device=DEV)
    o = 0
    for g, c in enumerate(counts):
        xs = x[o:o + c].double()
        if swiglu:
            a, b = xs @ w[g, :N].double().T, xs @ w[g, N:].double().T
            ref[o:o + c] = a / (1 + torch.exp(-a)) * b
        else:
            ref[o:o + c] = xs @ w[g].double().T
        o += c
    assert int(st[0]) == 0 and rel(out, ref) < 2e-5


@pytest.mark.parametrize("swiglu,bn", [(False, 256), (False, 128), (True, 128)])
def test_many_tiles_per_cta(tc, swiglu, bn):
    """More tiles than SMs: the persistent form walks several tiles per CTA, its stage ring wraps
    across tile borders and both accumulator buffers are used again and again."""
    M, N, K = 2304 + 40, 8192 + 72, 264
    torch.manual_seed(bn)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * N if swiglu else N, K, device=DEV) * 0.1).to(torch.bfloat16)
    out = torch.full((M, N), float("nan"), device=DEV)
    st = status()
    assert tc.gemm_tc(x, w, out, swiglu=swiglu, bn=bn, splits=1, status=st)
    if swiglu:
        a, b = x.double() @ w[:N].double().T, x.double() @ w[N:].double().T
        ref = a / (1 + torch.exp(-a)) * b
    else:
        ref = x.double() @ w.double().T
    assert int(st[0]) == 0 and rel(out, ref) < 2e-5


def test_grouped_many_tiles_per_cta(tc):
    """Sixty groups of uneven size (some empty), more tiles than SMs."""
    G, N, K = 60, 1408, 200
    rng = np.random.default_rng(5)
    counts = rng.integers(0, 300, size=G)
    counts[[3, 17, 59]] = 0
    M = int(counts.sum())
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(G, 2 * N, K, device=DEV) * 0.1).to(torch.bfloat16)
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    out = torch.full((M, N), float("nan"), device=DEV)
    st = status()
    assert tc.gemm_tc(x, w, out, swiglu=True, group_offsets=offs, bn=256, splits=1, status=st)
    ref = torch.empty(M, N, dtype=torch.float64, device=DEV)
    o = 0
    for g, c in enumerate(counts.tolist()):
        xs = x[o:o + c].double()
        a, b = xs @ w[g, :N].double().T, xs @ w[g, N:].double().T
        ref[o:o + c] = a / (1 + torch.exp(-a)) * b
        o += c
    assert int(st[0]) == 0 and rel(out, ref) < 2e-5


def test_refused_shapes_return_false(tc):
    x = torch.randn(4, 68, device=DEV).to(torch.bfloat16)       # K no multiple of 8 elements... 68 is not
    w = torch.randn(128, 68, device=DEV).to(torch.bfloat16)
    out = torch.empty(4, 128, device=DEV)
    assert tc.gemm_tc(x[:, :66].contiguous(), w[:, :66].contiguous(), out, status=status()) is False
    assert tc.gemm_tc(x.float(), w, out, status=status()) is False


def test_gather_rows(tc):
    src = torch.randn(50, 72, device=DEV).to(torch.bfloat16)
    rows = torch.randint(0, 50, (33,), device=DEV, dtype=torch.int32)
    st = status()
    assert torch.equal(tc.gather_rows(src, rows, 33, st), src[rows.long()]) and int(st[0]) == 0


@pytest.mark.parametrize("fault", [1, 2])
@pytest.mark.parametrize("tokens,splits", [(8, 4), (8, 16), (40, 1), (300, 1)])
def test_a_wait_that_runs_out_is_reported_and_the_next_product_is_right(fault, tokens, splits):
    """Every wait on a barrier inside the tensor-core products is bounded.  Here the bound is made
    short (2 ms) and one role of the kernel is told to do nothing (the producer loads nothing, or the MMA
    issuer issues nothing), so the other roles' waits run out: the kernel returns by itself, the
    status word says so, ``check_status`` raises, and the next, ordinary product is right, which
    shows that tensor memory was given back.  Nothing faults and nothing hangs: a wait that runs out
    is an ordinary exit path.  (8 tokens in 4 K splits: a cluster; in 16: partial sums in global
    memory; 40: one CTA a tile, the whole K; 300: the persistent form.)"""
    from moe_b200.ops import core, tc

    torch.manual_seed(0)
    K, N = 1024, 384
    x = (torch.randn(tokens, K, device=DEV) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().T
    status = core.new_status(DEV)
    out = torch.zeros(tokens, N, device=DEV)
    L = tc.lib()
    L.moe_tc_set_pair(0)                        # (the form on pairs of CTAs, off by default, has no such switch)
    L.moe_tc_set_wait_test.argtypes = [ctypes.c_int, ctypes.c_uint]
    L.moe_tc_set_wait_test.restype = None
    L.moe_tc_set_wait_test(fault, 2000)
    try:
        assert tc.gemm_tc(x, w, out, splits=splits, status=status)
        torch.cuda.synchronize()
    finally:
        L.moe_tc_set_wait_test(0, 0)
    assert int(status[0]) & 8, "the wait that ran out was not reported"
    with pytest.raises(core.KernelError) as e:
        core.check_status(status)
    assert "wait" in str(e.value) and "tensor-core product" in str(e.value) and "site 0x" in str(e.value)
    assert int(status[0]) == 0 and int(status[1]) == 0          # reported once, then cleared
    for _ in range(3):                          # tensor memory and barriers are in order again
        assert tc.gemm_tc(x, w, out, splits=splits, status=status)
    torch.cuda.synchronize()
    core.check_status(status)
    assert float((out - ref).abs().max()) < 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("tokens", [5, 40, 77, 150, 260])
def test_the_products_of_a_small_model_with_a_width_of_264(tc, tokens):
    """Every product of one layer at the sizes of one of the engine tests' configurations (width 264,
    2 + 2 heads of 128, 6 experts of 56 with 2 picked, shared expert 88, vocabulary 331), with the
    token tile the library itself picks: K below one 64-element block (56, 88), three feature tiles
    of which the last has 8 rows, groups of a few dozen rows."""
    from moe_b200.ops.tc import token_tile

    H, E, k, mi, si, V = 264, 6, 2, 56, 88, 331
    torch.manual_seed(tokens)

    def check(x, w, out_cols, swiglu=False, offs=None, bn=None):
        out = torch.full((x.shape[0], out_cols), float("nan"), device=DEV)
        st = status()
        assert tc.gemm_tc(x, w, out, swiglu=swiglu, group_offsets=offs, bn=bn, status=st)
        torch.cuda.synchronize()
        assert int(st[0]) == 0
        groups = [(0, x.shape[0], w)] if offs is None else [
            (int(offs[g]), int(offs[g + 1]), w[g]) for g in range(w.shape[0])]
        for a, b, wg in groups:
            xs = x[a:b].double()
            if swiglu:
                n = wg.shape[0] // 2
                g_, u_ = xs @ wg[:n].double().T, xs @ wg[n:].double().T
                ref = g_ / (1 + torch.exp(-g_)) * u_
            else:
                ref = xs @ wg.double().T
            if b > a:
                assert rel(out[a:b], ref) < 2e-5

    rnd = lambda *shape: (torch.randn(*shape, device=DEV) * 0.1).to(torch.bfloat16)
    x = torch.randn(tokens, H, device=DEV).to(torch.bfloat16)
    check(x, rnd(512, H), 512)                                     # q | k | v
    check(torch.randn(tokens, 256, device=DEV).to(torch.bfloat16), rnd(H, 256), H)       # attention output
    check(x, rnd(2 * si, H), si, swiglu=True)                      # shared gate | up
    check(torch.randn(tokens, si, device=DEV).to(torch.bfloat16), rnd(H, si), H)          # shared down
    check(x, rnd(V, H), V)                                         # output projection on every row
    P = tokens * k
    cuts = np.sort(np.random.default_rng(tokens).integers(0, P + 1, size=E - 1))
    offs = torch.tensor(np.concatenate([[0], cuts, [P]]), dtype=torch.int32, device=DEV)
    bn = token_tile(P / E)
    check(torch.randn(P, H, device=DEV).to(torch.bfloat16), rnd(E, 2 * mi, H), mi, swiglu=True, offs=offs, bn=bn)
    check(torch.randn(P, mi, device=DEV).to(torch.bfloat16), rnd(E, H, mi), H, offs=offs, bn=bn)

"""The tcgen05 / TMA matrix product against a float64 product of the same bfloat16 values:
plain and SwiGLU epilogues, every token tile, K splits, groups with gaps, ragged edges."""
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

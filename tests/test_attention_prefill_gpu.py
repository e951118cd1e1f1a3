"""The tensor-core prefill attention kernels (tcgen05 for head sizes 64 and 128, mma.sync for
16 ... 128) against the plain attention function: unequal sequences in one batch, grouped heads,
windows whose edge falls inside and across key tiles, a far key that must dominate."""
import math

import pytest
import torch

import gpu_util as G
import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def tc():
    from moe_b200.ops import tc as t

    t.lib()
    return t


def run(tc, q, k, v, lens, nh, nkv, hd, window, kernel="mma"):
    """kernel "tcgen05": the status word is given, so head sizes 64 and 128 take the tcgen05 kernel;
    "mma": no status word, the mma.sync kernel."""
    batch = G.make_batch(DEV, list(range(len(lens))), [0] * len(lens), lens)
    out = torch.full((sum(lens), nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    st = torch.zeros(4, dtype=torch.int32, device=DEV) if kernel == "tcgen05" else None
    assert tc.attention_prefill(q, k, v, batch, out, nh=nh, nkv=nkv, hd=hd, window=window, scale=1.0 / math.sqrt(hd),
                                status=st)
    assert st is None or int(st[0]) == 0
    return out


@pytest.mark.parametrize("kernel,nh,nkv,hd", [("mma", 4, 2, 16), ("mma", 3, 1, 32), ("mma", 6, 3, 64), ("mma", 2, 2, 128),
                                              ("mma", 5, 1, 128), ("tcgen05", 6, 3, 64), ("tcgen05", 2, 2, 128),
                                              ("tcgen05", 5, 1, 128)])
@pytest.mark.parametrize("window", [None, 1, 8, 64, 100, 128, 200])
def test_against_plain(tc, kernel, nh, nkv, hd, window):
    torch.manual_seed(hd + (window or 0))
    lens = [1, 63, 64, 65, 200, 7, 127, 128, 129, 300]
    T = sum(lens)
    q = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16)
    k = torch.randn(T, nkv, hd, device=DEV).to(torch.bfloat16)
    v = torch.randn(T, nkv, hd, device=DEV).to(torch.bfloat16)
    out = run(tc, q, k, v, lens, nh, nkv, hd, window, kernel).double().cpu()
    o = 0
    for n in lens:
        ref = plain.attention(q[o:o + n].double().cpu(), k[o:o + n].double().cpu(), v[o:o + n].double().cpu(), window)
        err = float((out[o:o + n] - ref).abs().max())
        assert err < 2e-2 * float(ref.abs().max()), (n, err)
        o += n
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
def test_a_far_key_among_hundreds_and_the_windows_edge(tc, kernel):
    """One key is made to stand out (query and key scaled): without a window the last query must
    return that key's value; with a window the key counts exactly while it is inside."""
    nh = nkv = 1
    hd, n, far = 64, 700, 5
    torch.manual_seed(1)
    q = (torch.randn(n, 1, hd) * 0.1)
    k = (torch.randn(n, 1, hd) * 0.1)
    v = torch.randn(n, 1, hd)
    u = torch.zeros(hd)
    u[3] = 1.0
    k[far, 0] = 40.0 * u
    q[n - 1, 0] = 40.0 * u                      # score 1600 / 8 = 200 against key `far`
    q[far + 99, 0] = 40.0 * u
    q[far + 100, 0] = 40.0 * u
    qd, kd, vd = (t.to(DEV).to(torch.bfloat16) for t in (q, k, v))
    full = run(tc, qd, kd, vd, [n], nh, nkv, hd, None, kernel).float().cpu()
    assert torch.allclose(full[n - 1], vd[far, 0].float().cpu(), atol=2e-2)
    win = run(tc, qd, kd, vd, [n], nh, nkv, hd, 100, kernel).float().cpu()
    # position far + 99 still sees `far` (window 100 includes itself); far + 100 no longer does
    assert torch.allclose(win[far + 99], vd[far, 0].float().cpu(), atol=2e-2)
    assert not torch.allclose(win[far + 100], vd[far, 0].float().cpu(), atol=0.2)
    ref = plain.attention(qd.double().cpu(), kd.double().cpu(), vd.double().cpu(), 100)
    assert float((win.double() - ref).abs().max()) < 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("window", [None, 80])
@pytest.mark.parametrize("lens", [[5], [77], [150], [260], [150, 260, 9]])
def test_two_heads_on_one_kv_head_of_128(tc, kernel, window, lens):
    """The sizes of one of the engine tests' configurations: 2 query heads on 1 kv head of 128, a
    window of 80, single sequences shorter and longer than a tile (the tensors end inside a tile)."""
    nh, nkv, hd = 2, 1, 128
    torch.manual_seed(sum(lens))
    T = sum(lens)
    q = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16)
    k = torch.randn(T, nkv, hd, device=DEV).to(torch.bfloat16)
    v = torch.randn(T, nkv, hd, device=DEV).to(torch.bfloat16)
    out = run(tc, q, k, v, lens, nh, nkv, hd, window, kernel).double().cpu()
    o = 0
    for n in lens:
        ref = plain.attention(q[o:o + n].double().cpu(), k[o:o + n].double().cpu(), v[o:o + n].double().cpu(), window)
        assert float((out[o:o + n] - ref).abs().max()) < 2e-2 * float(ref.abs().max()), n
        o += n


@pytest.mark.parametrize("kernel,hd", [("tcgen05", 64), ("tcgen05", 128), ("mma", 64)])
@pytest.mark.parametrize("window", [None, 150])
def test_the_running_maximum_jumps_in_a_later_tile_for_some_rows_only(tc, kernel, hd, window):
    """A key in the SECOND key tile scores far above everything before it, but only for a few
    queries scattered over the rows of a warp: those rows' accumulated output has to be rescaled
    (the maximum moves by much more than the slack the kernel allows itself), their neighbours' not.
    Random inputs never do this: their scores stay within the slack after the first tile."""
    nh = nkv = 1
    n, far = 400, 200
    torch.manual_seed(3)
    q, k, v = torch.randn(n, 1, hd) * 0.1, torch.randn(n, 1, hd) * 0.1, torch.randn(n, 1, hd)
    u = torch.zeros(hd)
    u[5] = 1.0
    k[far, 0] = 30.0 * u
    hot = [far, far + 3, far + 17, far + 40, far + 41, far + 100, far + 149, far + 150, n - 1]
    for r in hot:
        q[r, 0] = 30.0 * u                       # score 900 / sqrt(hd) against key `far`, about 0 against the others
    qd, kd, vd = (t.to(DEV).to(torch.bfloat16) for t in (q, k, v))
    out = run(tc, qd, kd, vd, [n], nh, nkv, hd, window, kernel).double().cpu()
    ref = plain.attention(qd.double().cpu(), kd.double().cpu(), vd.double().cpu(), window)
    assert torch.isfinite(out).all()
    assert float((out - ref).abs().max()) < 2e-2 * float(ref.abs().max())
    for r in hot:
        inside = window is None or far >= r + 1 - window
        assert torch.allclose(out[r].float(), vd[far, 0].float().cpu(), atol=2e-2) == inside, r

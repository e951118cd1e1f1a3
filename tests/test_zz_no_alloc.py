"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some hosts of this library may not allocate device memory while they call it: a server that
has given all free GPU memory to its own pool, a loop that cannot take the device-wide
synchronisation of an allocation, a plugin whose interface forbids it.  For them the library
exports moe_attention_decode_noalloc, whose scratch is a fixed array inside the library
(csrc/attention_decode_noalloc.h).  This test calls it several times in a row with different
data and sizes, compares each result with the ordinary entry point's (bit for bit) and with a
restatement in float64, and checks that calls it cannot serve (too large for the built-in scratch,
missing or misaligned memory, no heads) are refused on the host.  (Named test_zz_* so that pytest
collects it last.)"""
import ctypes
import math

import pytest
import torch

import gpu_util as G

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def c_entry():
    from moe_b200.ops import build

    L = ctypes.CDLL(build.build("core"))
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    L.moe_attention_decode_noalloc.argtypes = [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, P]
    L.moe_attention_decode_noalloc.restype = I
    L.moe_attention_decode_noalloc_need.argtypes = [I, I, I, I]
    L.moe_attention_decode_noalloc_need.restype = ctypes.c_longlong
    L.moe_noalloc_strerror.argtypes = [I]
    L.moe_noalloc_strerror.restype = ctypes.c_char_p
    return L


def make_case(dt, nh, nkv, hd, window, lens, seed):
    """A cache filled through the library's own append kernel, and one query per sequence.
    Also returns the keys and values as written, per sequence, for the plain restatement."""
    from moe_b200.cache import KVCache, KVRequest
    from moe_b200.ops import core

    torch.manual_seed(seed)
    B = len(lens)
    cache = KVCache({0: KVRequest(nkv, hd, window)}, {0: None}, max_tokens=4096, max_slots=B, dtype=dt, device=DEV)
    view = cache.view(0)
    slots = [cache.acquire() for _ in range(B)]
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    for s, n in zip(slots, lens):
        G.give_pages(cache, s, n)
    fill = G.make_batch(DEV, slots, [0] * B, lens)
    k = torch.randn(sum(lens), nkv, hd, device=DEV).to(dt)
    v = torch.randn(sum(lens), nkv, hd, device=DEV).to(dt)
    core.kv_commit(k, v, view, fill, st)
    step = G.make_batch(DEV, slots, [n - 1 for n in lens], [1] * B)     # the query sits at the last position
    # one spare element in front, so that a view shifted by one element is aligned to the element only
    qbuf = torch.randn(B * nh * hd + 8, device=DEV).to(dt)
    return cache, view, step, qbuf, st, k, v


def plain_decode_attention(q, k, v, lens, nh, nkv, window, scale):
    """softmax(q . K^T * scale) V over the last ``window`` keys of each sequence, in float64."""
    out, o = [], 0
    for i, n in enumerate(lens):
        lo = max(0, n - window) if window else 0
        ks, vs = k[o + lo:o + n].double(), v[o + lo:o + n].double()
        o += n
        rows = []
        for h in range(nh):
            kh = h // (nh // nkv)
            s = torch.softmax((ks[:, kh] @ q[i, h].double()) * scale, dim=0)
            rows.append(s @ vs[:, kh])
        out.append(torch.cat(rows))
    return torch.stack(out)


def call_noalloc(L, q, view, step, out, dt, B, nh, nkv, hd, window, scale, nsplit, st):
    g = view.group
    return L.moe_attention_decode_noalloc(
        q.data_ptr(), view.k.data_ptr(), view.v.data_ptr(), out.data_ptr(), 0 if dt == torch.float32 else 1,
        step.seq_of_token.data_ptr(), step.pos.data_ptr(), step.slots.data_ptr(), g.table.data_ptr(),
        g.table.stride(0), g.ring, g.page_size, g.num_pages, B, nh, nkv, hd, int(window or 0), scale, nsplit,
        st.data_ptr(), torch.cuda.current_stream().cuda_stream)


# (head size, lengths, window, seed, key splits or None for the library's own choice, q shifted off 16 bytes)
CALLS = [
    (64, [130, 64, 1, 300], None, 1, 16, False),     # many splits first ...
    (64, [77, 500, 33, 90], 100, 2, None, False),    # ... then the library's choice, in a window
    (64, [40, 9], None, 3, 2, False),                # fewer tokens and splits: most of the array keeps older records
    (48, [200, 31, 64], None, 4, 3, False),          # a head size whose rows take the row-per-lane kernel
    (64, [150, 70], 64, 5, 4, True),                 # q aligned to its element only: the row-per-lane kernel again
]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_calls_in_a_row_match_the_ordinary_entry_point_and_a_plain_restatement(dt):
    """Every call shares the built-in scratch and finds the last call's records in it.  The two
    entry points run the same kernels on the same inputs with the same splits, so their results
    are equal bit for bit; the restatement in float64 shows that both are right."""
    from moe_b200.ops import core

    L = c_entry()
    nh, nkv = 6, 2
    for call, (hd, lens, window, seed, nsplit, shift) in enumerate(CALLS):
        cache, view, step, qbuf, st, k, v = make_case(dt, nh, nkv, hd, window, lens, seed)
        B = len(lens)
        off = 1 if shift else 0
        q = qbuf[off:off + B * nh * hd].view(B, nh, hd)
        assert (q.data_ptr() % 16 != 0) == shift
        scale = 1.0 / math.sqrt(hd)
        nsplit = nsplit or core.decode_splits(DEV, B, nkv)
        g = view.group
        want = torch.empty(B, nh * hd, device=DEV, dtype=dt)
        partial = torch.empty(B * nh * nsplit * (hd + 2), dtype=torch.float32, device=DEV)
        rc = core.lib().moe_attention_decode(
            q.data_ptr(), view.k.data_ptr(), view.v.data_ptr(), want.data_ptr(), partial.data_ptr(),
            0 if dt == torch.float32 else 1, step.seq_of_token.data_ptr(), step.pos.data_ptr(), step.slots.data_ptr(),
            g.table.data_ptr(), g.table.stride(0), g.ring, g.page_size, g.num_pages, B, nh, nkv, hd, int(window or 0),
            scale, nsplit, st.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        got = torch.full((B, nh * hd), float("nan"), device=DEV, dtype=dt)
        code = call_noalloc(L, q, view, step, got, dt, B, nh, nkv, hd, window, scale, nsplit, st)
        assert code == 0, L.moe_noalloc_strerror(code).decode()
        torch.cuda.synchronize()
        assert int(st[0]) == 0
        assert torch.equal(got, want), f"call {call}: the two entry points differ"
        ref = plain_decode_attention(q, k, v, lens, nh, nkv, window, scale).to(DEV)
        tol = 2e-5 if dt == torch.float32 else 1e-2        # bfloat16: the output itself is rounded to 8 bits
        assert float((got.double() - ref).abs().max()) <= tol * float(ref.abs().max()), f"call {call}"


def test_calls_the_entry_point_cannot_serve_are_refused_before_anything_is_launched():
    L = c_entry()
    none = [None] * 4
    idx = [None] * 4

    def call(ptrs, tokens, nh, nkv, hd, nsplit, index=idx):
        return L.moe_attention_decode_noalloc(*ptrs, 1, *index, 0, 0, 64, 2, tokens, nh, nkv, hd, 0, 1.0, nsplit, None,
                                              None)

    need = L.moe_attention_decode_noalloc_need(4096, 64, 128, 32)
    assert need > 2 * 1024 * 1024
    code = call(none, 4096, 64, 8, 128, 32)                       # more scratch than the library holds
    assert code == -2 and b"scratch" in L.moe_noalloc_strerror(code)
    assert call(none, 65535, 65535, 1, 256, 65535) == -2          # a product that would not fit 64 bits
    assert L.moe_attention_decode_noalloc_need(65535, 65535, 256, 65535) == -1
    assert call(none, 4, 6, 4, 64, 1) == -3                       # 6 heads over 4 kv heads
    assert call(none, 4, 0, 1, 64, 1) == -3                       # no heads
    assert call(none, 4, -2, 1, 64, 1) == -3
    assert call(none, 4, 4, 2, 64, 1) == -3                       # no memory given at all
    # addresses are only looked at, never read, before these refusals: made-up ones will do
    ok = [4096, 8192, 12288, 16384]
    some = [256, 512, 768, 1024]
    assert call([ok[0], ok[1] + 8, ok[2], ok[3]], 4, 4, 2, 64, 1, some) == -3      # keys not 16-byte aligned
    assert call([ok[0], ok[1], ok[2] + 2, ok[3]], 4, 4, 2, 64, 1, some) == -3      # values not 16-byte aligned
    assert call([ok[0] + 1, ok[1], ok[2], ok[3]], 4, 4, 2, 64, 1, some) == -3      # q not aligned to bfloat16
    assert b"head layout" in L.moe_noalloc_strerror(-3)

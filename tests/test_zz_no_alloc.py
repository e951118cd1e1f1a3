"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some hosts of this library may not allocate device memory while they call it: a server that
has given all free GPU memory to its own pool, a loop that cannot take the device-wide
synchronisation of an allocation, a plugin whose interface forbids it.  For them the library
exports moe_attention_decode_noalloc, whose scratch is a fixed array inside the library
(csrc/attention_decode_noalloc.h).  This test calls it twice in a row with different data,
compares each result with the ordinary entry point's, and checks that a call too large for the
built-in scratch is refused.  (Named test_zz_* so that pytest collects it last.)"""
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
    """A cache filled through the library's own append kernel, and one query per sequence."""
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
    q = torch.randn(B, nh, hd, device=DEV).to(dt)
    return cache, view, step, q, st


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_two_calls_in_a_row_match_the_ordinary_entry_point(dt):
    from moe_b200.ops import core

    L = c_entry()
    nh, nkv, hd = 6, 2, 64
    stream = torch.cuda.current_stream().cuda_stream
    for call, (lens, window, seed) in enumerate([([130, 64, 1, 300], None, 1), ([77, 500, 33, 90], 100, 2)]):
        cache, view, step, q, st = make_case(dt, nh, nkv, hd, window, lens, seed)
        B = len(lens)
        scale = 1.0 / math.sqrt(hd)
        want = torch.empty(B, nh * hd, device=DEV, dtype=dt)
        core.attention_decode(q, view, step, want, nh=nh, window=window, scale=scale, status=st)
        nsplit = core.decode_splits(DEV, B, nkv)
        got = torch.full((B, nh * hd), float("nan"), device=DEV, dtype=dt)
        g = view.group
        code = L.moe_attention_decode_noalloc(
            q.data_ptr(), view.k.data_ptr(), view.v.data_ptr(), got.data_ptr(), 0 if dt == torch.float32 else 1,
            step.seq_of_token.data_ptr(), step.pos.data_ptr(), step.slots.data_ptr(), g.table.data_ptr(),
            g.table.stride(0), g.ring, g.page_size, g.num_pages, B, nh, nkv, hd, int(window or 0), scale, nsplit,
            st.data_ptr(), stream)
        assert code == 0, L.moe_noalloc_strerror(code).decode()
        torch.cuda.synchronize()
        assert int(st[0]) == 0
        tol = 2e-5 if dt == torch.float32 else 2e-2
        assert float((got.double() - want.double()).abs().max()) <= tol * float(want.double().abs().max()), call


def test_a_call_beyond_the_built_in_scratch_is_refused():
    L = c_entry()
    need = L.moe_attention_decode_noalloc_need(4096, 64, 128, 32)
    assert need > 2 * 1024 * 1024
    code = L.moe_attention_decode_noalloc(None, None, None, None, 1, None, None, None, None, 0, 0, 64, 2, 4096, 64, 8,
                                          128, 0, 1.0, 32, None, None)
    assert code == -2 and b"scratch" in L.moe_noalloc_strerror(code)
    assert L.moe_attention_decode_noalloc(None, None, None, None, 1, None, None, None, None, 0, 0, 64, 2, 4, 6, 4,
                                          64, 0, 1.0, 1, None, None) == -3     # 6 heads over 4 kv heads

"""The host runtime (C++, csrc/host_runtime.cpp): the reservation of a whole step and the packing
of a step's index arrays, against their definitions restated here in Python.  No GPU needed."""
import random

import numpy as np
import pytest

from moe_b200.cache import CacheError, CacheLedger
from moe_b200.cache.allocator import _IP, _ok, host_lib, ints
from moe_b200.engine.batch import fill_host, layout


def test_reserve_is_all_or_nothing():
    led = CacheLedger(4, [6, 3], [0, 1])                       # 5 + 2 usable pages
    a, b, c = led.acquire(), led.acquire(), led.acquire()
    starts, upd = led.reserve([a, b], [130, 1], [8, 0])
    assert starts == [0, 0] and led.length[a] == 130 and led.length[b] == 1
    assert sorted(map(tuple, upd[:, :3].tolist())) == [(0, a, 0), (0, a, 1), (0, a, 2), (0, b, 0), (1, a, 0), (1, b, 0)]
    assert len(set(upd[upd[:, 0] == 0, 3].tolist())) == 4 and 0 not in upd[:, 3].tolist()
    free = [g.pool.num_free for g in led.groups]
    with pytest.raises(CacheError):                               # c fits in the full group, not in the ring's pool
        led.reserve([a, c], [1, 5], [8, 0])
    assert led.length[a] == 130 and led.length[c] == 0 and [g.pool.num_free for g in led.groups] == free
    with pytest.raises(CacheError):                               # the page table of group 0 is 3 entries wide
        led.reserve([b], [200], [3, 0])
    with pytest.raises(ValueError):
        led.reserve([a, a], [1, 1], [8, 0])                       # a slot twice
    with pytest.raises(ValueError):
        led.reserve([a], [0], [8, 0])                             # no token
    with pytest.raises(CacheError):
        led.reserve([3], [1], [8, 0])                             # never acquired
    assert led.length[a] == 130 and [g.pool.num_free for g in led.groups] == free
    starts, upd = led.reserve([a], [62], [8, 0])                  # 192 tokens: still three pages
    assert starts == [130] and upd.shape == (0, 4)


def test_reserve_matches_a_sequence_of_extends():
    rng = random.Random(3)
    one, two = CacheLedger(6, [64, 9], [0, 2]), CacheLedger(6, [64, 9], [0, 2])
    slots = [one.acquire() for _ in range(6)]
    assert slots == [two.acquire() for _ in range(6)]
    for _ in range(30):
        pick = rng.sample(slots, rng.randint(1, 6))
        counts = [rng.randint(1, 150) for _ in pick]
        try:
            starts, upd = one.reserve(pick, counts, [0, 0])
        except CacheError:
            break
        want = []
        for s, n in zip(pick, counts):
            assert starts[pick.index(s)] == two.length[s]
            want += two.extend(s, two.length[s] + n)
        assert [tuple(r) for r in upd.tolist()] == want
    assert all(one.length[s] == two.length[s] for s in slots)


def test_pack_step_layout_and_facts():
    slots, starts = [5, 2, 9], [0, 64, 7]
    tokens = [[11, 12, 13], [21], [31, 32]]
    want = [[0, 2], [], [1]]
    buf = np.full(64, -7, dtype=np.int32)
    info = fill_host(buf, slots, starts, tokens, want)
    T, B, W = 6, 3, 3
    assert [(k, info["offsets"][k][1]) for k, _ in layout(T, B, W)] == layout(T, B, W)
    v = {k: buf[a:a + n].tolist() for k, (a, n) in info["offsets"].items()}
    assert v["token_ids"] == [11, 12, 13, 21, 31, 32]
    assert v["seq_of_token"] == [0, 0, 0, 1, 2, 2]
    assert v["pos"] == [0, 1, 2, 64, 7, 8]
    assert v["cu_seqlens"] == [0, 3, 4, 6]
    assert v["slots"] == slots and v["seq_start"] == starts and v["seq_end"] == [3, 65, 9]
    assert v["want_rows"] == [0, 2, 5]
    assert info["used"] == sum(n for _, n in layout(T, B, W)) and buf[info["used"]] == -7
    assert info["facts"] == dict(num_tokens=6, num_seqs=3, num_want=3, max_new=3, max_end=65, all_decode=False,
                                 all_fresh=False)
    assert fill_host(buf, [1, 2], [0, 0], [[4], [5]], [[0], [0]])["facts"]["all_decode"] is True
    assert fill_host(buf, [1], [0], [[4, 5]], [[]])["facts"] == dict(num_tokens=2, num_seqs=1, num_want=0, max_new=2,
                                                                     max_end=2, all_decode=False, all_fresh=True)
    with pytest.raises(ValueError):
        fill_host(buf, [1], [0], [[4, 5]], [[2]])                 # a wanted place past the step's tokens
    with pytest.raises(ValueError):
        fill_host(np.zeros(5, dtype=np.int32), slots, starts, tokens, want)     # buffer too small


def test_pack_decode_pads_with_rows_of_no_sequence():
    size, B, pad, groups = 8, 3, 99, 2
    n_arrays = sum(n for _, n in layout(size, size, size))
    upd_off = [n_arrays, n_arrays + 3 * size]
    buf = np.full(n_arrays + 2 * 3 * size + 4, -7, dtype=np.int32)
    sl, _ = ints([4, 0, 6])
    st, _ = ints([10, 64, 0])
    tk, _ = ints([7, 8, 9])
    uo, _ = ints(upd_off)
    updates = np.array([[1, 0, 1, 5], [0, 6, 0, 3], [1, 6, 0, 2]], dtype=np.int32)
    _ok(host_lib().moe_pack_decode(buf.ctypes.data_as(_IP), size, B, sl, st, tk, pad, groups, uo,
                                   updates.ctypes.data_as(_IP), 3))
    o, v = 0, {}
    for name, n in layout(size, size, size):
        v[name] = buf[o:o + n].tolist()
        o += n
    assert v["token_ids"] == [7, 8, 9, 0, 0, 0, 0, 0]
    assert v["seq_of_token"] == [0, 1, 2, -1, -1, -1, -1, -1]
    assert v["pos"] == [10, 64, 0] + [0] * 5 and v["seq_start"] == v["pos"]
    assert v["seq_end"] == [11, 65, 1] + [1] * 5
    assert v["cu_seqlens"] == [0, 1, 2, 3, 3, 3, 3, 3, 3]
    assert v["slots"] == [4, 0, 6] + [pad] * 5
    assert v["want_rows"] == list(range(8))
    g0 = buf[upd_off[0]:upd_off[0] + 3 * size].reshape(size, 3).tolist()
    g1 = buf[upd_off[1]:upd_off[1] + 3 * size].reshape(size, 3).tolist()
    assert g0 == [[6, 0, 3]] + [[pad, 0, 0]] * 7
    assert g1 == [[0, 1, 5], [6, 0, 2]] + [[pad, 0, 0]] * 6
    assert buf[-4:].tolist() == [-7] * 4
    with pytest.raises(ValueError):
        _ok(host_lib().moe_pack_decode(buf.ctypes.data_as(_IP), 2, 3, sl, st, tk, pad, groups, uo,
                                       updates.ctypes.data_as(_IP), 3))


def test_pack_padded_pads_tokens_sequences_and_wanted_places():
    tp, bb, wb, pad, groups, cap = 16, 4, 4, 99, 2, 3
    n_arrays = sum(n for _, n in layout(tp, bb, wb))
    upd_off = [n_arrays, n_arrays + 3 * cap]
    buf = np.full(n_arrays + 2 * 3 * cap + 4, -7, dtype=np.int32)
    sl, _ = ints([4, 6])
    st, _ = ints([62, 0])
    ct, _ = ints([3, 5])
    tk, _ = ints([7, 8, 9, 1, 2, 3, 4, 5])
    wc, _ = ints([1, 2])
    wn, _ = ints([2, 0, 4])
    uo, _ = ints(upd_off)
    updates = np.array([[0, 4, 1, 5], [0, 6, 0, 3], [1, 6, 0, 2]], dtype=np.int32)

    def pack(tp=tp, bb=bb, wb=wb, cap=cap, wn=wn):
        _ok(host_lib().moe_pack_padded(buf.ctypes.data_as(_IP), tp, bb, wb, 2, sl, st, ct, tk, wc, wn, pad, groups, uo,
                                       cap, updates.ctypes.data_as(_IP), 3))

    pack()
    o, v = 0, {}
    for name, n in layout(tp, bb, wb):
        v[name] = buf[o:o + n].tolist()
        o += n
    assert v["token_ids"] == [7, 8, 9, 1, 2, 3, 4, 5] + [0] * 8
    assert v["seq_of_token"] == [0] * 3 + [1] * 5 + [-1] * 8
    assert v["pos"] == [62, 63, 64, 0, 1, 2, 3, 4] + [0] * 8
    assert v["cu_seqlens"] == [0, 3, 8, 8, 8]
    assert v["slots"] == [4, 6, pad, pad]
    assert v["seq_start"] == [62, 0, 0, 0] and v["seq_end"] == [65, 5, 0, 0]
    assert v["want_rows"] == [2, 3, 7, 0]
    g0 = buf[upd_off[0]:upd_off[0] + 3 * cap].reshape(cap, 3).tolist()
    g1 = buf[upd_off[1]:upd_off[1] + 3 * cap].reshape(cap, 3).tolist()
    assert g0 == [[4, 1, 5], [6, 0, 3], [pad, 0, 0]]
    assert g1 == [[6, 0, 2]] + [[pad, 0, 0]] * 2
    assert buf[-4:].tolist() == [-7] * 4
    # the same arrays as the unpadded packer writes, where both have something
    plain = np.zeros(64, dtype=np.int32)
    info = fill_host(plain, [4, 6], [62, 0], [[7, 8, 9], [1, 2, 3, 4, 5]], [[2], [0, 4]])
    for name, (a, n) in info["offsets"].items():
        assert v[name][:n] == plain[a:a + n].tolist(), name
    for bad in (dict(tp=7), dict(bb=1), dict(wb=2), dict(cap=1), dict(wn=ints([3, 0, 4])[0])):
        with pytest.raises(ValueError):
            pack(**bad)

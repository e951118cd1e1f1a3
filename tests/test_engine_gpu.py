"""The engine against the plain implementation, in 32-bit and in bfloat16, under every cut.

Mirrors the reference's tests/oracle.rs: token by token (:46-56), whole (:60-69), split
(:71-75), every row (:100-118); plus batches of unequal lengths, which the reference has not."""
import pytest
import torch

import gpu_util as G
import helpers

pytestmark = pytest.mark.gpu

CASES = [(n, dt, std) for n in ("A", "B") for dt in ("float32", "bfloat16") for std in G.STD[dt]]
CASES += [(n, dt, G.STD[dt][-1]) for n in ("C", "E") for dt in ("float32", "bfloat16")]
# D is 264 wide: weights of the same scale would have a gain of 0.2 sqrt(264) = 3.2 a matrix (1.6 to 2.5
# for the others) and amplify every rounding far more; its scales keep the gain that B has
CASES += [("D", dt, G.STD_WIDE[dt]) for dt in ("float32", "bfloat16")]
LENGTHS = [5, 9, 12, 40, 77, 1, 33]


def requests_for(name):
    V = helpers.CONFIGS[name]["vocab_size"]
    lengths = LENGTHS + ([150, 260] if name in "CD" else [])     # C, D: prompts of more than one 128-key tile
    return {f"r{i}": helpers.random_tokens(V, n, 100 + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name,dtype,std", CASES)
def test_each_request_alone_and_whole_matches_plain(model_dirs, name, dtype, std):
    d, eng = G.engine_for(model_dirs, name, dtype, std)
    flips = []
    for rid, toks in requests_for(name).items():
        err, frac = helpers.compare_with_plain(d, eng, toks, G.flip(dtype))
        flips.append(frac)
        assert err < G.tol(dtype), f"{rid}: relative error {err:.3g}"
    assert sum(flips) / len(flips) < (0.001 if dtype == "float32" else 0.05), f"routing differs too often: {flips}"
    assert eng.cache.ledger.slots.num_held == 0


@pytest.mark.parametrize("name,dtype,std", CASES)
def test_last_32_tokens_one_by_one_match_plain_and_whole(model_dirs, name, dtype, std):
    """The cut is compared with the plain implementation directly (with the engine's own picks),
    and with the same engine's whole-prompt result more tightly."""
    d, eng = G.engine_for(model_dirs, name, dtype, std)
    reqs = requests_for(name)
    whole = helpers.replay_whole(eng, reqs)
    logits, picks = helpers.run_schedule(eng, helpers.tail_schedule(reqs, 32))
    helpers.check_schedule_against_plain(d, reqs, logits, picks, G.tol(dtype), G.flip(dtype))
    for rid, toks in reqs.items():
        tail = helpers.stacked(logits, rid, len(toks))
        err = helpers.max_rel_err(tail, whole[rid])
        assert err < G.tol_cut(dtype), f"{rid}: first wrong place {first_bad(tail, whole[rid], G.tol_cut(dtype))}"


@pytest.mark.parametrize("name,dtype,std", CASES)
def test_unequal_batches_one_after_another_match_plain_and_whole(model_dirs, name, dtype, std):
    # 3 slots for 7 requests: every slot is given back and used again
    d, eng = G.engine_for(model_dirs, name, dtype, std, max_tokens=64 * (12 if name in "CD" else 6), max_slots=3)
    reqs = requests_for(name)
    whole = helpers.replay_whole(eng, reqs)
    steps = helpers.batches_schedule(reqs, 3, lambda r: len(reqs[r]) // 2)
    logits, picks = helpers.run_schedule(eng, steps)
    helpers.check_schedule_against_plain(d, reqs, logits, picks, G.tol(dtype), G.flip(dtype))
    for rid, toks in reqs.items():
        batched = helpers.stacked(logits, rid, len(toks))
        err = helpers.max_rel_err(batched, whole[rid])
        assert err < G.tol_cut(dtype), f"{rid}: first wrong place {first_bad(batched, whole[rid], G.tol_cut(dtype))}"
    led = eng.cache.ledger
    assert led.slots.num_held == 0 and all(g.pool.num_free == g.pool.num_pages - 1 for g in led.groups)


def first_bad(got, ref, tol):
    scale = float(ref.abs().max())
    bad = ((got.double() - ref.double()).abs().amax(dim=1) > tol * scale).nonzero()
    return int(bad[0]) if len(bad) else None


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("A", "B") for dt in ("float32", "bfloat16")])
def test_the_first_tokens_of_a_sequence(model_dirs, name, dtype):
    """Positions 0, 1, 2 decoded one by one from an empty slot (a prompt of one token)."""
    d, eng = G.engine_for(model_dirs, name, dtype)
    toks = helpers.random_tokens(helpers.CONFIGS[name]["vocab_size"], 4, 9)
    got = helpers.replay_tail(eng, {"x": toks}, tail=10)["x"]
    err, _ = helpers.compare_with_plain(d, eng, toks, G.flip(dtype))
    whole = helpers.replay_whole(eng, {"x": toks})["x"]
    assert err < G.tol(dtype) and helpers.max_rel_err(got, whole) < G.tol_cut(dtype)


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("A", "B", "D") for dt in ("float32", "bfloat16")])
def test_long_decoding(model_dirs, name, dtype):
    """3 prompt tokens, then 330 tokens one by one: several pages, the window's ring wrapping many
    times (B), and hundreds of keys behind every query."""
    d, eng = G.engine_for(model_dirs, name, dtype)
    toks = helpers.random_tokens(helpers.CONFIGS[name]["vocab_size"], 333, 5)
    logits, picks = helpers.run_schedule(eng, helpers.tail_schedule({"x": toks}, 330))
    helpers.check_schedule_against_plain(d, {"x": toks}, logits, picks, G.tol(dtype), G.flip(dtype))
    one_by_one = helpers.stacked(logits, "x", len(toks))
    err, frac = helpers.compare_with_plain(d, eng, toks, G.flip(dtype))
    whole = helpers.replay_whole(eng, {"x": toks})["x"]
    assert err < G.tol(dtype), f"whole against plain: {err:.3g}"
    cut = helpers.max_rel_err(one_by_one, whole)
    assert cut < G.tol_cut(dtype), f"first wrong place {first_bad(one_by_one, whole, G.tol_cut(dtype))}"


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("A", "B", "C") for dt in ("float32", "bfloat16")])
def test_short_prompts_replayed_from_padded_graphs_equal_the_step_launched_kernel_by_kernel(model_dirs, name, dtype):
    """Whole prompts whose last logits are wanted run from a graph padded to a bucket of token rows
    and of sequences: the logits, and the cache they leave (seen through a decode step), are those
    of the same step without graphs.  Lengths just below, at and above a bucket's and a page's edge."""
    import moe_b200

    vocab = helpers.CONFIGS[name]["vocab_size"]
    d, eng = G.engine_for(model_dirs, name, dtype, max_tokens=64 * 24, max_slots=8)
    model = eng.model
    plain_eng = moe_b200.Engine(model, max_tokens=64 * 24, max_slots=8, use_graphs=False)
    for lens in ([5], [63], [64, 1], [65, 3, 17], [127, 128, 2, 40], [200, 9, 64, 30, 31, 7, 1, 100]):
        prompts = [helpers.random_tokens(vocab, n, 11 + n) for n in lens]
        nxt = [[(7 * n + 1) % vocab] for n in lens]
        out = []
        for e in (eng, plain_eng):
            slots = [e.new_sequence() for _ in lens]
            first = e.step(slots, prompts).float().cpu()
            second = e.step(slots, nxt).float().cpu()
            for s in slots:
                e.release(s)
            out.append((first, second))
        assert eng.graphs_of("prompt"), "the prompt step did not take a graph"
        for a, b in zip(out[0], out[1]):
            assert torch.isfinite(a).all()
            assert helpers.max_rel_err(a, b) < G.tol_cut(dtype), lens


def test_a_reused_slot_never_shows_what_it_held_before(model_dirs):
    """The same request on a fresh engine and on one whose slot and pages held other sequences."""
    import moe_b200
    from moe_b200.engine import Engine

    for name in ("A", "B"):
        d = model_dirs.get(name, "float32", seed=1, std=0.2)
        V = helpers.CONFIGS[name]["vocab_size"]
        toks = helpers.random_tokens(V, 70, 1)
        fresh = Engine(moe_b200.load_model(d, dtype="float32"), max_tokens=256, max_slots=1)
        want = helpers.replay_tail(fresh, {"x": toks}, 20)["x"]
        used = Engine(moe_b200.load_model(d, dtype="float32"), max_tokens=256, max_slots=1)
        for seed in (7, 8):                       # fill every page with other sequences' keys, then give them back
            helpers.replay_whole(used, {"y": helpers.random_tokens(V, 250, seed)})
        got = helpers.replay_tail(used, {"x": toks}, 20)["x"]
        assert torch.equal(got, want)


def test_cache_full_is_an_error_and_changes_nothing(model_dirs):
    from moe_b200.cache import CacheError

    d, eng = G.engine_for(model_dirs, "A", "float32", max_tokens=192, max_slots=2)
    a, b = eng.new_sequence(), eng.new_sequence()
    eng.step([a], [[1] * 64])
    with pytest.raises(CacheError):
        eng.step([a, b], [[2], [3] * 65])          # a needs 1 more page, b needs 2: only 2 are free
    assert eng.length(a) == 64 and eng.length(b) == 0
    eng.step([a, b], [[2], [3] * 10])              # still usable
    eng.release(a), eng.release(b)


def test_a_token_outside_the_vocabulary_is_reported(model_dirs):
    from moe_b200.ops.core import KernelError

    d, eng = G.engine_for(model_dirs, "A", "float32")
    s = eng.new_sequence()
    with pytest.raises(KernelError) as e:
        eng.step([s], [[1, 256, 3]])
    assert "vocabulary" in str(e.value)
    eng.release(s)
    # the engine is still usable
    toks = helpers.random_tokens(256, 5, 0)
    assert helpers.compare_with_plain(d, eng, toks, G.FLIP_F32)[0] < G.TOL_F32


def test_wanted_places_select_rows(model_dirs):
    d, eng = G.engine_for(model_dirs, "B", "float32")
    toks = helpers.random_tokens(384, 20, 4)
    whole = helpers.replay_whole(eng, {"x": toks})["x"]
    s = eng.new_sequence()
    assert eng.step([s], [toks[:10]], [[]]) is None
    got = eng.step([s], [toks[10:]], [[9, 0, 4]]).cpu()
    eng.release(s)
    assert helpers.max_rel_err(got, whole[[19, 10, 14]]) < G.TOL_CUT_F32
    with pytest.raises(ValueError):
        s = eng.new_sequence()
        try:
            eng.step([s], [[1, 2]], [[2]])
        finally:
            eng.release(s)

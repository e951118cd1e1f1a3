"""Schedules of steps beyond "one request alone": many sequences decoded together, steps that mix
fresh prompts with continued ones and with single tokens, prompts fed in chunks.  Every wanted
place is compared with the plain implementation directly, run with the engine's own routing picks
(the reference compares whole, one by one and split with its oracle: tests/oracle.rs:46-75,
100-118; it tiles prompts at 64 tokens, src/main.rs:499-505)."""
import numpy as np
import pytest
import torch

import gpu_util as G
import helpers

pytestmark = pytest.mark.gpu


def engine(model_dirs, name, dtype, max_tokens, max_slots, use_graphs=True):
    """An engine of its own (its pool is smaller than the number of requests) on the session's model."""
    import moe_b200

    d, shared = G.engine_for(model_dirs, name, dtype)
    return d, moe_b200.Engine(shared.model, max_tokens=max_tokens, max_slots=max_slots, use_graphs=use_graphs)


MANY = [("A", 12, True), ("A", 70, True), ("B", 24, True), ("B", 40, False), ("D", 40, True), ("D", 12, False),
        ("C", 33, True), ("E", 20, True), ("E", 9, False), ("A", 140, True)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n,graphs", MANY)
def test_many_sequences_decoded_together_match_plain(model_dirs, name, n, graphs, dtype):
    """``n`` requests of unequal lengths start together and are decoded for 40 to 60 steps, the
    shorter ones ending earlier, so that the batch shrinks through the padded sizes of the captured
    steps; then a second batch of half as many on the same slots.  From 9 sequences on the routed
    experts pick, invert and gather in separate launches and the products take wider token tiles."""
    V = helpers.CONFIGS[name]["vocab_size"]
    rng = np.random.default_rng(n)
    total = n + n // 2
    prompt = {f"r{i}": int(rng.integers(1, 24)) for i in range(total)}
    reqs = {r: helpers.random_tokens(V, p + int(rng.integers(40, 61)), 1000 + i) for i, (r, p) in enumerate(prompt.items())}
    d, eng = engine(model_dirs, name, dtype, max_tokens=128 * n, max_slots=n, use_graphs=graphs)
    steps = helpers.batches_schedule(reqs, n, lambda r: prompt[r], want_all=(n % 2 == 0))
    logits, picks = helpers.run_schedule(eng, steps)
    if graphs:
        sizes = {k[1] for k in eng.graphs_of("decode")}
        assert max(sizes) >= min(n, 64) and len(sizes) >= 3, sizes      # the padded sizes the batch went through
    helpers.check_schedule_against_plain(d, reqs, logits, picks, G.tol(dtype), G.flip(dtype))
    led = eng.cache.ledger
    assert led.slots.num_held == 0 and all(g.pool.num_free == g.pool.num_pages - 1 for g in led.groups)


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("A", "C") for dt in ("float32", "bfloat16")])
def test_a_sequence_decodes_the_same_alone_and_among_63_others(model_dirs, name, dtype):
    V = helpers.CONFIGS[name]["vocab_size"]
    reqs = {f"r{i}": helpers.random_tokens(V, 30 + (i * 7) % 23, 300 + i) for i in range(64)}
    d, eng = engine(model_dirs, name, dtype, max_tokens=64 * 64, max_slots=64)
    alone, _ = helpers.run_schedule(eng, helpers.batches_schedule({"r5": reqs["r5"]}, 1, lambda r: 4))
    among, _ = helpers.run_schedule(eng, helpers.batches_schedule(reqs, 64, lambda r: 4))
    a = torch.stack([alone[("r5", i)] for i in range(len(reqs["r5"]))])
    b = torch.stack([among[("r5", i)] for i in range(len(reqs["r5"]))])
    assert helpers.max_rel_err(b, a) < G.tol_cut(dtype)


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("A", "B", "C", "D", "E") for dt in ("float32", "bfloat16")])
def test_steps_that_mix_fresh_prompts_continued_ones_and_single_tokens(model_dirs, name, dtype):
    """One step may hold a sequence that brings one token, one that goes on by several from a
    position beyond 0, and one that starts with a whole prompt; keys of earlier steps then come from
    the cache and those of the step from its own buffers."""
    V = helpers.CONFIGS[name]["vocab_size"]
    reqs = {"a": helpers.random_tokens(V, 110, 1), "b": helpers.random_tokens(V, 160, 2),
            "c": helpers.random_tokens(V, 150, 3), "d": helpers.random_tokens(V, 9, 4)}
    cuts = [                      # tokens each request brings, step by step (0: it is not in the step)
        dict(a=20, b=70),
        dict(a=1, b=5, c=70),
        dict(a=5, b=1, c=1, d=3),
        dict(a=1, b=1, c=64, d=1),          # c goes on across a page's edge
        dict(a=63, b=1, c=1, d=5),          # a ends exactly on position 89, d ends
        dict(a=1, b=82, c=14),              # b goes on from 78 to 159: past the windows of C and D
        dict(a=19),
    ]
    at = {r: 0 for r in reqs}
    steps = []
    for cut in cuts:
        entries, ends = [], []
        for r, n in cut.items():
            toks = reqs[r][at[r]:at[r] + n]
            assert len(toks) == n
            entries.append((r, toks, list(range(n))))
            at[r] += n
            if at[r] == len(reqs[r]):
                ends.append(r)
        steps.append({"entries": entries, "end": ends})
    assert at == {r: len(t) for r, t in reqs.items()}
    d, eng = engine(model_dirs, name, dtype, max_tokens=64 * 10, max_slots=4)
    logits, picks = helpers.run_schedule(eng, steps)
    # every such step is replayed from the captured graph of its padded shape
    assert eng.graphs_of("prompt") and len(eng.graphs_of("continued")) >= 2 and not eng.graphs_of("decode")
    helpers.check_schedule_against_plain(d, reqs, logits, picks, G.tol(dtype), G.flip(dtype))
    if dtype == "float32":        # the same steps launched kernel by kernel, unpadded
        d, eng = engine(model_dirs, name, dtype, max_tokens=64 * 10, max_slots=4, use_graphs=False)
        again, _ = helpers.run_schedule(eng, steps)
        worst = max(helpers.max_rel_err(logits[k], again[k]) for k in logits)
        assert worst < G.tol_cut(dtype), worst


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("A", "B", "C", "D", "E") for dt in ("float32", "bfloat16")])
@pytest.mark.parametrize("chunk", [64, 50])
def test_a_prompt_fed_in_chunks_matches_plain(model_dirs, name, dtype, chunk):
    V = helpers.CONFIGS[name]["vocab_size"]
    reqs = {"x": helpers.random_tokens(V, 230, 12), "y": helpers.random_tokens(V, 131, 13)}
    steps = []
    longest = max(len(t) for t in reqs.values())
    for o in range(0, longest, chunk):
        entries = [(r, t[o:o + chunk], list(range(len(t[o:o + chunk])))) for r, t in reqs.items() if o < len(t)]
        steps.append({"entries": entries, "end": [r for r, t in reqs.items() if o < len(t) <= o + chunk]})
    d, eng = engine(model_dirs, name, dtype, max_tokens=64 * 8, max_slots=2)
    logits, picks = helpers.run_schedule(eng, steps)
    assert eng.graphs_of("prompt") and eng.graphs_of("continued")
    helpers.check_schedule_against_plain(d, reqs, logits, picks, G.tol(dtype), G.flip(dtype))


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("A", "B", "D") for dt in ("float32", "bfloat16")])
def test_rewinding_then_continuing_equals_a_fresh_sequence(model_dirs, name, dtype):
    """Truncating the cache matches a fresh state (tests/oracle.rs:678-701): after a rewind to
    position n the sequence goes on as if it had never held more."""
    from moe_b200.cache import CacheError

    V = helpers.CONFIGS[name]["vocab_size"]
    d, eng = engine(model_dirs, name, dtype, max_tokens=64 * 8, max_slots=2)
    toks = helpers.random_tokens(V, 60, 21)
    other = helpers.random_tokens(V, 25, 22)
    s = eng.new_sequence()
    eng.step([s], [toks[:40]])
    for t in other:                                  # a continuation that is then taken back
        eng.step([s], [[t]])
    eng.truncate(s, 40)
    assert eng.length(s) == 40
    got = [eng.step([s], [toks[40:50]], [list(range(10))]).float().cpu()]
    got += [eng.step([s], [[t]], [[0]]).float().cpu() for t in toks[50:]]
    got = torch.cat(got)
    f = eng.new_sequence()
    fresh = [eng.step([f], [toks[:40]], [[]])]
    fresh = [eng.step([f], [toks[40:50]], [list(range(10))]).float().cpu()]
    fresh += [eng.step([f], [[t]], [[0]]).float().cpu() for t in toks[50:]]
    fresh = torch.cat(fresh)
    assert helpers.max_rel_err(got, fresh) < 1e-5
    ref = helpers.plain_logits(d, toks)[40:]
    if dtype == "float32":
        assert helpers.max_rel_err(got, ref) < G.TOL_F32
    with pytest.raises(CacheError):
        eng.truncate(s, 61)                          # a rewind cannot lengthen
    # a windowed layer: once its ring has wrapped, a rewind beyond what it still holds is refused
    win = helpers.CONFIGS[name].get("sliding_window") if helpers.CONFIGS[name].get("use_sliding_window") else None
    if win:
        ring = -(-win // 64) * 64
        long = helpers.random_tokens(V, ring + 70, 23)
        eng.step([f], [long[:ring + 70 - 60]])
        n = eng.length(f)
        with pytest.raises(CacheError):
            eng.truncate(f, n - ring)                # the keys before that position are written over
        assert eng.length(f) == n
        eng.truncate(f, n - 1)                       # one step back is always inside the ring's slack or window
    eng.release(s), eng.release(f)


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("A", "B", "D") for dt in ("float32", "bfloat16")])
@pytest.mark.parametrize("piece", [64, 100])
def test_a_step_too_large_for_one_go_is_run_in_pieces_with_the_same_result(model_dirs, name, dtype, piece):
    """The engine runs a step of more than ``max_step_tokens`` tokens in pieces (the reference tiles
    its prompts at 64 tokens and tests that the result does not depend on it: src/main.rs:499-505,
    tests/oracle.rs:71-75): two prompts in ONE step, every place wanted, against the plain
    implementation; and a step that does not fit the cache fails before its first piece."""
    from moe_b200.cache import CacheError

    V = helpers.CONFIGS[name]["vocab_size"]
    reqs = {"x": helpers.random_tokens(V, 230, 31), "y": helpers.random_tokens(V, 131, 32)}
    d, eng = engine(model_dirs, name, dtype, max_tokens=64 * 7, max_slots=2)
    eng.max_step_tokens = piece
    steps = [{"entries": [(r, t, list(range(len(t)))) for r, t in reqs.items()], "end": list(reqs)}]
    before = eng.steps_run
    logits, picks = helpers.run_schedule(eng, steps)
    assert eng.steps_run - before == -(-361 // piece)
    helpers.check_schedule_against_plain(d, reqs, logits, picks, G.tol(dtype), G.flip(dtype))
    a, b = eng.new_sequence(), eng.new_sequence()
    with pytest.raises(CacheError):
        eng.step([a, b], [reqs["x"], reqs["x"]])         # 4 + 4 pages of the 7 there are
    assert eng.length(a) == 0 and eng.length(b) == 0
    eng.release(a), eng.release(b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wanted_places_of_every_kind_through_the_padded_graphs(model_dirs, dtype):
    """A captured step takes any wanted places: none at all, a few, every place, and (outside the
    graphs) a place asked for twice; the rows come back in the order asked for and equal those of a
    step that asks for every place."""
    V = helpers.CONFIGS["C"]["vocab_size"]
    d, eng = engine(model_dirs, "C", dtype, max_tokens=64 * 8, max_slots=3)
    toks = [helpers.random_tokens(V, n, 70 + n) for n in (37, 5, 90)]
    more = [helpers.random_tokens(V, n, 80 + n) for n in (3, 20, 1)]

    def run(want0, want1):
        slots = [eng.new_sequence() for _ in toks]
        a = eng.step(slots, toks, want0)
        b = eng.step(slots, more, want1)
        for s in slots:
            eng.release(s)
        return (None if a is None else a.float().cpu().clone()), (None if b is None else b.float().cpu().clone())

    full0 = [list(range(len(t))) for t in toks]
    full1 = [list(range(len(t))) for t in more]
    ref0, ref1 = run(full0, full1)
    row0 = lambda i, j: ref0[sum(len(t) for t in toks[:i]) + j]
    row1 = lambda i, j: ref1[sum(len(t) for t in more[:i]) + j]
    before = len(eng.graphs_of("prompt")) + len(eng.graphs_of("continued"))
    assert before >= 2
    tol = 1e-6 if dtype == "float32" else G.tol_cut(dtype)
    for want0, want1 in (([[], [], []], [[], [], []]),                    # nothing wanted: the step still runs
                         ([[36], [], [0, 89]], [[2, 0], [19], []]),       # a few, not in ascending order
                         ([[0], [4], [89]], [[2], [19], [0]]),            # one each
                         ([[5, 5, 5] * 20, [], []], [[0, 0, 1, 1, 2, 2], [], []])):   # more places than tokens
        a, b = run(want0, want1)
        for got, want, row in ((a, want0, row0), (b, want1, row1)):
            flat = [(i, j) for i, w in enumerate(want) for j in w]
            if not flat:
                assert got is None
                continue
            assert got.shape[0] == len(flat)
            worst = max(helpers.max_rel_err(got[n], row(i, j)) for n, (i, j) in enumerate(flat))
            assert worst < tol, (want, worst)
    # the cache went on from where the first step left it, whatever was wanted
    assert eng.cache.ledger.slots.num_held == 0


def test_more_shapes_of_step_than_captured_graphs_are_kept(model_dirs):
    """An engine keeps at most MAX_GRAPHS captured steps and drops the one used longest ago; a shape
    that was dropped is captured again and gives the same logits as the first time."""
    from moe_b200.engine import engine as E

    V = helpers.CONFIGS["A"]["vocab_size"]
    d, eng = engine(model_dirs, "A", "float32", max_tokens=64 * 80, max_slots=8)
    first = {}
    shapes = [(b, n, every, fresh) for fresh in (True, False) for every in (False, True)
              for b in (1, 2, 3, 5) for n in (7, 20, 40, 70)]            # 64 padded shapes (a few share a key)
    for rnd in range(2):
        for b, n, every, fresh in shapes:
            slots = [eng.new_sequence() for _ in range(b)]
            if not fresh:
                eng.step(slots, [helpers.random_tokens(V, 3 + i, i) for i in range(b)], [[] for _ in slots])
            toks = [helpers.random_tokens(V, n + i, 10 * n + i) for i in range(b)]
            want = [list(range(len(t))) if every else [len(t) - 1] for t in toks]
            lg = eng.step(slots, toks, want).float().cpu().clone()
            for s in slots:
                eng.release(s)
            key = (b, n, every, fresh)
            if rnd == 0:
                first[key] = lg
            else:
                assert torch.equal(lg, first[key]), key
            assert len(eng._graphs) <= E.MAX_GRAPHS
    assert len(eng._graphs) == E.MAX_GRAPHS            # more shapes were met than are kept
    assert eng.cache.ledger.slots.num_held == 0

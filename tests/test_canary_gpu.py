"""Writes that stray: the cache is filled with a canary value before a schedule of steps of every
kind (prompts, chunks, mixed steps, padded decode graphs, sequences that end and slots that are used
again); afterwards every page that no sequence ever held, and every position of a held page beyond
what its sequence wrote, must still hold the canary (the scratch page 0 takes the rows of no
sequence and is exempt).  The sanitizers are not available on this machine; this is the check in
their place for the kernels that write into the cache (kv_commit, the fused rotation + append of the
decode step, the prompt's rotation + split + append)."""
import pytest
import torch

import gpu_util as G
import helpers

pytestmark = pytest.mark.gpu
CANARY = 7.0


@pytest.mark.parametrize("name,dtype", [(n, dt) for n in ("B", "C", "D", "E") for dt in ("float32", "bfloat16")])
def test_no_kernel_writes_outside_its_sequences_pages(model_dirs, name, dtype):
    import moe_b200

    d, shared = G.engine_for(model_dirs, name, dtype)
    eng = moe_b200.Engine(shared.model, max_tokens=64 * 40, max_slots=6)
    for g in eng.cache.groups:
        g.storage.fill_(CANARY)
    V = helpers.CONFIGS[name]["vocab_size"]
    held = [set() for _ in eng.cache.groups]          # pages a live sequence held at some time
    given_back = [[] for _ in eng.cache.groups]       # every page at every release

    def note(slots):
        for gi, g in enumerate(eng.cache.groups):
            for s in slots:
                n = eng.length(s)
                pages = -(-n // 64) if not g.ring_pages else min(-(-n // 64), g.ring_pages)
                held[gi].update(int(p) for p in g.table[s, :pages].tolist())

    checked = [0]

    def finish(s):
        for gi, g in enumerate(eng.cache.groups):
            n = eng.length(s)
            pages = -(-n // 64) if not g.ring_pages else min(-(-n // 64), g.ring_pages)
            mine = [int(p) for p in g.table[s, :pages].tolist()]
            # the sequence's last page, if no sequence held it before and its ring (if any) has not
            # wrapped: nothing beyond the sequence's length was written
            if mine[-1] not in given_back[gi] and n % 64 and (not g.ring_pages or n <= g.ring):
                torch.cuda.synchronize()
                st = g.storage[:, :, mine[-1], :, n % 64:].float()
                assert bool((st == CANARY).all()), f"group {gi}: written past position {n}"
                checked[0] += 1
            given_back[gi].extend(mine)
        eng.release(s)

    for rnd in range(2):                              # the second round takes the first one's slots and pages again
        seqs = [eng.new_sequence() for _ in range(5)]
        toks = lambda n, seed: helpers.random_tokens(V, n, 100 * rnd + seed)
        eng.step(seqs[:3], [toks(70, 1), toks(5, 2), toks(129, 3)])            # prompts
        note(seqs[:3])
        eng.step(seqs[1:5], [toks(60, 4), toks(1, 5), toks(33, 6), toks(64, 7)])   # continued, single, fresh
        note(seqs)
        for i in range(70):                           # decode, the batch shrinking through the padded sizes
            live = seqs if i < 20 else seqs[:3] if i < 50 else seqs[:1]
            eng.step(live, [[(7 * i + j) % V] for j in range(len(live))])
            note(live)
            if i == 19:
                finish(seqs[3]), finish(seqs[4])
            if i == 49:
                finish(seqs[1]), finish(seqs[2])
        finish(seqs[0])
    eng.rt.check()
    torch.cuda.synchronize()
    for gi, g in enumerate(eng.cache.groups):
        st = g.storage.float()                        # [layer][k|v][page][kv_head][pos][dim]
        never = [p for p in range(1, g.num_pages) if p not in held[gi]]
        assert never, "the pool is too small for this test to show anything"
        assert bool((st[:, :, never] == CANARY).all()), f"group {gi}: a page that no sequence held was written"
        assert bool((st[:, :, sorted(held[gi])] != CANARY).any())
    assert checked[0] >= 1

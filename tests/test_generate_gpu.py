"""Generation through the Python entry point and the command line, on the GPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gpu_util as G
import helpers
import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def engine_logits(eng, tokens):
    return helpers.replay_whole(eng, {"x": list(tokens)})["x"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_batch_of_three(model_dirs, dtype):
    """Configuration A's workload: prompts of 5, 9 and 12 tokens, then 8 greedy steps."""
    import moe_b200

    d, eng = G.engine_for(model_dirs, "A", dtype)
    prompts = [helpers.random_tokens(256, n, 20 + n) for n in (5, 9, 12)]
    stats = moe_b200.GenerationStats()
    outs = moe_b200.generate(eng, prompts, max_tokens=9, eos=(), stats=stats)
    assert [len(o.tokens) for o in outs] == [9, 9, 9] and all(o.stop == "length" for o in outs)
    assert stats.decode_steps == 8 and stats.prefill_tokens == 26
    assert eng.cache.ledger.slots.num_held == 0
    cfg, w = plain.read_model(d)
    for p, o in zip(prompts, outs):
        seq = p + o.tokens
        ref = plain.forward(cfg, w, seq)[len(p) - 1:-1]           # the logits each token was picked from
        if dtype == "float32":
            # greedy on the plain logits gives the same tokens unless two logits are within rounding
            gap = torch.topk(ref, 2, dim=-1).values
            sure = (gap[:, 0] - gap[:, 1]) > 1e-3 * ref.abs().max()
            assert torch.equal(ref.argmax(-1)[sure], torch.tensor(o.tokens)[sure]) and sure.float().mean() > 0.8
        # every generated token is the argmax of the engine's own logits for the same history
        own = engine_logits(eng, seq)[len(p) - 1:-1]
        picked = own[torch.arange(len(o.tokens)), torch.tensor(o.tokens)]
        assert torch.all(picked >= own.max(-1).values - G.tol_cut(dtype) * own.abs().max())


def test_sequences_that_end_earlier_and_batches_in_a_row(model_dirs):
    import moe_b200

    d, eng = G.engine_for(model_dirs, "B", "float32", std=0.2, max_tokens=64 * 4, max_slots=2)
    prompts = [helpers.random_tokens(384, n, 40 + n) for n in (1, 7, 16, 23, 3)]
    free_run = moe_b200.generate(eng, prompts, max_tokens=10, eos=(), batch_size=2)
    # make the 4th token of request 1 an end-of-sequence token: it stops there, the others do not change
    eos = free_run[1].tokens[3]
    outs = moe_b200.generate(eng, prompts, max_tokens=10, eos=[eos], batch_size=2)
    for i, (a, b) in enumerate(zip(free_run, outs)):
        want = a.tokens[:a.tokens.index(eos)] if eos in a.tokens else a.tokens
        assert b.tokens == want and b.stop == ("eos" if eos in a.tokens else "length"), i
    assert outs[1].stop == "eos" and len(outs[1].tokens) <= 3 and eng.cache.ledger.slots.num_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_seeded_temperature_sampling_workload_b(model_dirs, dtype):
    """Configuration B's workload: prompts of 1, 7, 16 and 23 tokens, 12 tokens at temperature 0.8.
    Request i samples with seed + i; the plain sampler on the engine's own logits gives the same."""
    import moe_b200

    d, eng = G.engine_for(model_dirs, "B", dtype)
    prompts = [helpers.random_tokens(384, n, 60 + n) for n in (1, 7, 16, 23)]
    kw = dict(temp=0.8, top_p=0.95, seed=5)
    outs = moe_b200.generate(eng, prompts, max_tokens=12, eos=(), **kw)
    again = moe_b200.generate(eng, prompts, max_tokens=12, eos=(), **kw)
    assert [o.tokens for o in outs] == [o.tokens for o in again]                    # reproducible
    other = moe_b200.generate(eng, prompts, max_tokens=12, eos=(), temp=0.8, seed=6)
    assert [o.tokens for o in outs] != [o.tokens for o in other]
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o.tokens) == 12
        own = engine_logits(eng, p + o.tokens)[len(p) - 1:-1].numpy()
        if dtype == "float32":
            # 32-bit logits do not depend on the cut, so the plain sampler replays the run exactly
            rng = plain.Rng(5 + i)
            agree = sum(plain.sample(own[j], [], rng, temp=0.8, top_p=0.95) == o.tokens[j] for j in range(12))
            assert agree == 12, f"request {i}: {agree} of 12"
        else:
            # bfloat16 logits of a prompt and of a decode step differ by an ulp of some activation
            # (1e-3 of the largest logit), which moves the cumulative distribution: each token must
            # still lie inside the nucleus of the whole-sequence logits, slightly widened
            for j, tok in enumerate(o.tokens):
                p = np.exp((own[j].astype(np.float64) - own[j].max()) / 0.8)
                p /= p.sum()
                order = np.argsort(-p)
                inside = order[:int(np.searchsorted(np.cumsum(p[order]), 0.97)) + 1]
                assert tok in inside, f"request {i}, token {j}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_step_ahead_gives_the_same_tokens(model_dirs, dtype):
    """The loop begins each step before it has read the tokens of the one before (the device feeds
    itself the token it sampled); the results must be those of the loop that waits: greedy and seeded
    sampling, an end-of-sequence token that the counts cannot foresee, a context limit, a callback,
    and batches in a row whose slots are used again while a step of the batch before is still queued."""
    import moe_b200

    d, eng = G.engine_for(model_dirs, "B", dtype, std=0.2, max_tokens=64 * 4, max_slots=3)
    prompts = [helpers.random_tokens(384, n, 70 + n) for n in (1, 7, 16, 23, 3, 64, 65)]
    for kw in (dict(), dict(temp=0.8, top_p=0.9, seed=3), dict(temp=1.1, top_k=5, seed=9)):
        wait = moe_b200.generate(eng, prompts, max_tokens=14, eos=(), batch_size=3, lookahead=False, **kw)
        s1, s2 = moe_b200.GenerationStats(), moe_b200.GenerationStats()
        ahead = moe_b200.generate(eng, prompts, max_tokens=14, eos=(), batch_size=3, lookahead=True, stats=s1, **kw)
        assert [(o.tokens, o.stop, o.steps) for o in ahead] == [(o.tokens, o.stop, o.steps) for o in wait]
        eos = [wait[1].tokens[3], wait[5].tokens[0]]
        a = moe_b200.generate(eng, prompts, max_tokens=14, eos=eos, batch_size=3, ctx=70, lookahead=True, stats=s2, **kw)
        b = moe_b200.generate(eng, prompts, max_tokens=14, eos=eos, batch_size=3, ctx=70, lookahead=False, **kw)
        assert [(o.tokens, o.stop, o.steps) for o in a] == [(o.tokens, o.stop, o.steps) for o in b]
        assert a[1].stop == "eos" and a[5].tokens == [] and a[6].stop == "context"
        assert eng.cache.ledger.slots.num_held == 0
        halt = lambda i, tok: not (i == 2 and tok == wait[2].tokens[4])
        a = moe_b200.generate(eng, prompts, max_tokens=14, eos=(), batch_size=3, on_token=halt, lookahead=True, **kw)
        b = moe_b200.generate(eng, prompts, max_tokens=14, eos=(), batch_size=3, on_token=halt, lookahead=False, **kw)
        assert [(o.tokens, o.stop) for o in a] == [(o.tokens, o.stop) for o in b] and a[2].stop == "caller"
    # a token id of -1 that was not asked for is still an error
    s = eng.new_sequence()
    with pytest.raises(Exception):
        eng.step([s], [[-1]])
    eng.release(s)


def test_one_step_ahead_over_many_pages(model_dirs):
    """140 tokens after prompts that end just before, at and after a page border: every new page of
    the cache is reserved for a step that is begun before the step before it has been read."""
    import moe_b200

    d, eng = G.engine_for(model_dirs, "A", "bfloat16", max_tokens=64 * 12, max_slots=3)
    prompts = [helpers.random_tokens(256, n, 90 + n) for n in (63, 64, 65)]
    wait = moe_b200.generate(eng, prompts, max_tokens=140, eos=(), lookahead=False, temp=0.9, seed=2)
    ahead = moe_b200.generate(eng, prompts, max_tokens=140, eos=(), lookahead=True, temp=0.9, seed=2)
    assert [o.tokens for o in ahead] == [o.tokens for o in wait] and all(len(o.tokens) == 140 for o in ahead)
    assert eng.cache.ledger.slots.num_held == 0


def test_command_line_run_info_bench(model_dirs, tmp_path):
    d = model_dirs.get("A", "bfloat16", seed=1, std=0.08)
    env = dict(os.environ, PYTHONPATH=ROOT)
    run = lambda *a: subprocess.run([sys.executable, os.path.join(ROOT, "bin", "moe"), *a], capture_output=True,
                                    text=True, env=env, timeout=600)
    r = run("run", d, "--ids", "5,17,3,9", "-n", "6", "--no-stream")
    assert r.returncode == 0, r.stderr
    toks = json.loads(r.stdout.strip().splitlines()[-1])
    assert len(toks) == 6 and "decode" in r.stderr and "prefill 4 tok" in r.stderr
    import moe_b200

    _, eng = G.engine_for(model_dirs, "A", "bfloat16")
    assert moe_b200.generate(eng, [[5, 17, 3, 9]], max_tokens=6)[0].tokens == toks
    pf = tmp_path / "prompts.txt"
    pf.write_text("1,2,3\n[9, 8, 7, 6, 5]\n4 4\n")
    r = run("run", d, "--prompts", str(pf), "--tokens=3", "--temp", "0.7", "--seed", "2", "--batch", "2")
    assert r.returncode == 0, r.stderr
    lines = [json.loads(l) for l in r.stdout.strip().splitlines()]
    assert [l["index"] for l in lines] == [0, 1, 2] and all(l["generated"] == len(l["tokens"]) <= 3 for l in lines)
    assert all("logprobs" not in l for l in lines)
    r = run("run", d, "--prompts", str(pf), "--tokens=3", "--logprobs", "2")
    assert r.returncode == 0, r.stderr
    for l in (json.loads(x) for x in r.stdout.strip().splitlines()):
        assert [e["token"] for e in l["logprobs"]] == l["tokens"]
        assert all(len(e["top"]) == 2 and e["logprob"] <= 0 and e["top"][0][1] >= e["top"][1][1] for e in l["logprobs"])
        assert all(e["top"][0][0] == e["token"] for e in l["logprobs"])           # greedy: the strongest was taken
    # the routing trace of one request: a header, then one record per (position, routed layer)
    tr = tmp_path / "routes.jsonl"
    r = run("run", d, "--ids", "5,17,3,9", "-n", "6", "--no-stream", "--trace", str(tr))
    assert r.returncode == 0 and json.loads(r.stdout.strip().splitlines()[-1]) == toks, r.stderr
    recs = [json.loads(x) for x in tr.read_text().splitlines()]
    assert recs[0] == {"model": "Qwen2MoeForCausalLM", "layers": 2, "experts": 4, "top_k": 2}
    fed = [5, 17, 3, 9] + toks[:-1]                       # the last token is sampled, never fed
    assert [(x["pos"], x["layer"]) for x in recs[1:]] == [(p_, l) for p_ in range(len(fed)) for l in (0, 1)]
    assert [x["token"] for x in recs[1::2]] == fed
    cfg_a, w_a = plain.read_model(d)
    picks = []
    plain.forward(cfg_a, w_a, fed, trace=picks)
    agree = 0
    for x in recs[1:]:
        assert len(x["experts"]) == 2 and 0 < sum(w for _, w in x["experts"]) <= 1.0 + 1e-3
        ref = sorted(int(v) for v in picks[x["layer"]][0][x["pos"]])
        agree += sorted(e for e, _ in x["experts"]) == ref
    assert agree >= 0.8 * (len(recs) - 1), agree          # (bfloat16: a close call may fall the other way)
    r = run("info", d)
    assert r.returncode == 0 and "Qwen2MoeForCausalLM" in r.stdout and "4 experts of 32, top-2" in r.stdout
    r = run("bench", d, "--prompt-len", "16", "--tokens", "4", "--batch", "2")
    assert r.returncode == 0 and "decode" in r.stdout and "tok/s" in r.stdout, r.stderr
    assert "roofline" in r.stdout and "% of 7700 GB/s" in r.stdout
    # random weights instead of a folder: the same verbs, nothing written
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(helpers.CONFIG_A))
    r = run("bench", "--random", str(cfg), "--seed", "4", "--prompt-len", "8", "--tokens", "3", "--peak-gbs", "6500",
            "--kernels")
    assert r.returncode == 0 and "% of 6500 GB/s" in r.stdout, r.stderr
    assert "us/step" in r.stdout and "attn_decode" in r.stdout and "launches/step" in r.stdout
    a = run("run", "--random", str(cfg), "--seed", "4", "--ids", "1,2,3", "-n", "5", "--no-stream")
    b = run("run", "--random", str(cfg), "--seed", "4", "--ids", "1,2,3", "-n", "5", "--no-stream")
    assert a.returncode == 0 and a.stdout == b.stdout and len(json.loads(a.stdout.strip().splitlines()[-1])) == 5
    r = run("run", str(tmp_path / "nothing"), "--ids", "1")
    assert r.returncode == 1 and r.stderr.startswith("moe:")


@pytest.mark.parametrize("dtype,kw", [("float32", dict(temp=0.0)), ("float32", dict(temp=0.9, seed=5, repeat_penalty=1.3)),
                                      ("bfloat16", dict(temp=0.0))])
def test_logprobs_of_generated_tokens_match_plain(model_dirs, dtype, kw):
    """What the model thought of each emitted token comes from the RAW logits (before the penalty and
    the temperature, src/generate.rs:78-82), the plain implementation's for the same history."""
    import moe_b200

    d, eng = G.engine_for(model_dirs, "B", dtype)
    prompts = [helpers.random_tokens(384, n, 60 + n) for n in (4, 11)]
    outs = moe_b200.generate(eng, prompts, max_tokens=7, eos=(), logprobs=3, **kw)
    cfg, w = plain.read_model(d)
    tol = 2e-4 if dtype == "float32" else 5e-2
    for p, o in zip(prompts, outs):
        assert len(o.logprobs) == len(o.tokens) == 7
        ref = torch.log_softmax(plain.forward(cfg, w, p + o.tokens)[len(p) - 1:-1].double(), -1)
        for j, (tok, (lp, top)) in enumerate(zip(o.tokens, o.logprobs)):
            assert abs(lp - float(ref[j, tok])) < tol, (j, lp, float(ref[j, tok]))
            assert len(top) == 3 and all(abs(l - float(ref[j, i])) < tol for i, l in top)
            assert [l for _, l in top] == sorted((l for _, l in top), reverse=True)
            if dtype == "float32":
                best = torch.topk(ref[j], 4).values
                if float(best[2] - best[3]) > 1e-3:
                    assert sorted(i for i, _ in top) == sorted(torch.topk(ref[j], 3).indices.tolist())
    plain_outs = moe_b200.generate(eng, prompts, max_tokens=7, eos=(), **kw)
    assert [o.tokens for o in plain_outs] == [o.tokens for o in outs] and plain_outs[0].logprobs is None

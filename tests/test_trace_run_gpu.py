"""bin/trace_run as a program: steps on standard input, logits files out, in both dtypes."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gpu_util as G
import helpers

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(model_dir, dtype, out_dir, steps, max_tokens):
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                          "--out", out_dir, "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    done = []
    for s in steps:                               # the next step is sent only after "done <step>"
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        line = p.stdout.readline().strip()
        assert line == f"done {s['step']}", (line, p.stderr.read() if p.poll() is not None else "")
        done.append(line)
    p.stdin.close()
    assert p.wait(timeout=600) == 0, p.stderr.read()
    return done


def as_trace(steps):
    """The steps of ``helpers.run_schedule`` in the program's own format, and where each wanted
    place lands: (request, position) -> (step, row)."""
    out, where, at = [], {}, {}
    for i, st in enumerate(steps):
        row = 0
        entries = []
        for rid, toks, want in st["entries"]:
            entries.append({"id": rid, "tokens": list(toks), "want": list(want)})
            for w in want:
                where[(rid, at.get(rid, 0) + w)] = (i, row)
                row += 1
            at[rid] = at.get(rid, 0) + len(toks)
        out.append({"step": i, "entries": entries, "end": list(st.get("end", []))})
    return out, where


def cut_steps(cut, reqs):
    if cut == "whole":
        return helpers.whole_schedule(reqs), 320
    if cut == "tail":
        return helpers.tail_schedule(reqs, 32), 320
    # batches of unequal lengths on room for 256 tokens: (64 + 64 + 128), then (64 + 64 + 128)
    ids = list(reqs)
    return (helpers.batches_schedule({r: reqs[r] for r in ids}, 3, lambda r: len(reqs[r]) // 2, want_all=True), 256)


@pytest.mark.parametrize("cut", ["whole", "tail", "batches"])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("D", "float32"), ("D", "bfloat16")])
def test_the_program_replays_every_cut_and_matches_plain(model_dirs, tmp_path, name, dtype, cut):
    """The program is driven as a user drives it (steps on standard input, files out) in the three
    cuts: each request alone and whole; all but the last 32 tokens, then one by one; batches of
    unequal lengths whose shorter requests end earlier, one batch after another on room for fewer
    requests than there are, so that slots are used again.  Its files equal, to rounding of the last
    bit, what the same schedule gives inside this process on an engine of the same size; and that
    result is compared with the plain implementation directly, run with the engine's picks."""
    import moe_b200

    d, shared = G.engine_for(model_dirs, name, dtype)
    V = helpers.CONFIGS[name]["vocab_size"]
    lengths = [40, 9, 70, 3, 21, 100] if cut == "batches" else [40, 9, 70, 3, 150]
    reqs = {f"q{i}": helpers.random_tokens(V, n, 200 + i) for i, n in enumerate(lengths)}
    steps, max_tokens = cut_steps(cut, reqs)
    trace, where = as_trace(steps)
    out = str(tmp_path / "out")
    run_trace(d, dtype, out, trace, max_tokens=max_tokens)
    eng = moe_b200.Engine(shared.model, max_tokens=max_tokens)
    logits, picks = helpers.run_schedule(eng, steps)
    helpers.check_schedule_against_plain(d, reqs, logits, picks, G.tol(dtype), G.flip(dtype))
    assert set(where) == set(logits)
    files = {}
    for (rid, pos), (st, row) in where.items():
        if st not in files:
            files[st] = torch.from_numpy(np.fromfile(os.path.join(out, f"{st}.f32"), dtype="<f4").reshape(-1, V))
        got, mine = files[st][row], logits[(rid, pos)]
        assert float((got - mine).abs().max()) <= 1e-6 * float(mine.abs().max()), (rid, pos, st, row)
    wanted_steps = {st for st, _ in where.values()}
    assert sorted(os.listdir(out)) == sorted(f"{st}.f32" for st in wanted_steps)


def test_steps_without_wanted_logits_write_nothing(model_dirs, tmp_path):
    d = model_dirs.get("A", "float32", seed=1, std=0.2)
    out = str(tmp_path / "o")
    run_trace(d, "float32", out, [
        {"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]},
        {"step": 2, "entries": [], "end": []},
    ], max_tokens=64)
    assert sorted(os.listdir(out)) == ["1.f32"]
    got = torch.from_numpy(np.fromfile(os.path.join(out, "1.f32"), dtype="<f4").astype(np.float64))
    ref = helpers.plain_logits(d, [1, 2, 3, 4])[3]
    assert float((got - ref).abs().max() / ref.abs().max()) < G.TOL_F32


@pytest.mark.parametrize("bad,needle", [
    ('{"step": 1, "entries": [{"id": "b", "tokens": [1] * 200, "want": []}]}'.replace("[1] * 200", str([1] * 200)), "CacheError"),
    ('{"entries": []}', "KeyError"),
    ('not a step', "JSONDecodeError"),
    ('{"step": 1, "entries": [{"id": "a", "tokens": [5], "want": [3]}]}', "wanted place"),
])
def test_a_bad_line_ends_the_program_with_one_message(model_dirs, tmp_path, bad, needle):
    """A line that is no step, a wanted place outside the step or a step the cache has no room for:
    exit code 1 and one line that names the input line, after the steps before it were done."""
    d = model_dirs.get("A", "float32", seed=1, std=0.2)
    first = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": []})
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "128"], input=first + "\n" + bad + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 1 and p.stdout.strip().splitlines() == ["done 0"]
    last = p.stderr.strip().splitlines()[-1]
    assert last.startswith("trace_run: input line 2:") and needle in last, p.stderr
    assert os.path.exists(tmp_path / "o" / "0.f32")

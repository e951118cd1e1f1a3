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


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_replay_in_unequal_batches_with_slots_reused(model_dirs, tmp_path, name, dtype):
    d = model_dirs.get(name, dtype, seed=1, std=G.STD[dtype][1])
    V = helpers.CONFIGS[name]["vocab_size"]
    reqs = {f"q{i}": helpers.random_tokens(V, n, 200 + i) for i, n in enumerate([40, 9, 70, 3, 21])}
    steps, where = [], {}                         # where[(request, position)] = (step, row)
    step = 0
    for batch in (["q0", "q1", "q2"], ["q3", "q4"]):     # 64 + 64 + 128 tokens held, then 64 + 64: max-tokens 256
        live = list(batch)
        done = {r: max(1, len(reqs[r]) // 2) for r in live}
        entries, row = [], 0
        for r in live:
            want = list(range(0, done[r], 2)) + ([done[r] - 1] if (done[r] - 1) % 2 else [])
            entries.append({"id": r, "tokens": reqs[r][:done[r]], "want": want})
            for w in want:
                where[(r, w)] = (step, row)
                row += 1
        ends = [r for r in live if done[r] >= len(reqs[r])]
        steps.append({"step": step, "entries": entries, "end": ends})
        live = [r for r in live if r not in ends]
        step += 1
        while live:
            entries = [{"id": r, "tokens": [reqs[r][done[r]]], "want": [0]} for r in live]
            for i, r in enumerate(live):
                where[(r, done[r])] = (step, i)
                done[r] += 1
            ends = [r for r in live if done[r] >= len(reqs[r])]
            steps.append({"step": step, "entries": entries, "end": ends})
            live = [r for r in live if r not in ends]
            step += 1
    out = str(tmp_path / "out")
    run_trace(d, dtype, out, steps, max_tokens=256)
    files = {}
    scale, worst = 0.0, 0.0
    _, eng = G.engine_for(model_dirs, name, dtype)
    for rid, toks in reqs.items():
        if dtype == "float32":
            ref = helpers.plain_logits(d, toks)
            limit = G.TOL_F32
        else:
            ref = helpers.replay_whole(eng, {rid: toks})[rid].double()      # in-process engine, whole request
            limit = G.TOL_CUT_BF16
        for (r, pos), (st, row) in where.items():
            if r != rid:
                continue
            if st not in files:
                files[st] = np.fromfile(os.path.join(out, f"{st}.f32"), dtype="<f4").reshape(-1, V)
            got = torch.from_numpy(files[st][row].astype(np.float64))
            worst = max(worst, float((got - ref[pos]).abs().max() / ref.abs().max()))
        assert worst < limit, f"{rid}: {worst:.3g}"
    # a step with nothing wanted writes no file
    assert not os.path.exists(os.path.join(out, f"{step}.f32"))


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

"""Command line in the reference's manner (src/main.rs:7-125, 127-196).

    moe run   <model> --ids 1,2,3 [-n N] [--temp F] [--top-p F] [--top-k N] [--repeat-penalty F] [--seed N]
    moe run   <model> --prompts FILE        one list of ids a line = one batch of unequal prompts
    moe bench <model> [--prompt-len N] [--tokens N] [--batch N]
    moe info  <model>
    moe run|bench|info --random CONFIG.json [--seed N]     random weights instead of a folder

Options keep the reference's names, meanings and defaults where it has them
(``--ids``, ``-n/--tokens`` [128], ``--ctx``, ``--temp`` [0], ``--top-p`` [0.95],
``--top-k`` [0], ``--repeat-penalty`` [1.0], ``--seed`` [0], ``--prompts``,
``--no-stream``, ``--stats``, ``--prompt-len`` [32], bench ``--tokens`` [16]).
Added here: ``--dtype bfloat16|float32`` [bfloat16], ``--batch N``,
``--max-tokens N`` (cache size), ``--random CONFIG.json`` (with ``--seed``),
``--peak-gbs F`` (bench: the bandwidth its roofline line is a percentage of).  Prompts are token ids; there is no tokenizer.
Arguments are parsed as the reference does: ``--k v``, ``--k=v``, short aliases
``-n -o -h -V``, and a fixed list of boolean flags.
"""
from __future__ import annotations

import json
import sys
import time
from typing import Dict, List, Tuple

USAGE = """\
moe - Qwen2 MoE generation on one B200

USAGE
  moe run   <model> [options]        generate tokens
  moe info  <model>                  show the architecture and its footprint
  moe bench <model> [options]        measure prefill and decode throughput

<model> is a folder with config.json and *.safetensors (or give --random CONFIG.json).

RUN OPTIONS
      --ids 1,2,3           prompt as token ids
      --prompts PATH        one prompt a line (ids separated by commas or spaces, or a JSON
                            list); the prompts form batches; one JSON result a line
  -n, --tokens N            tokens to generate            [128]
      --ctx N               context window per sequence   [min(model, 4096), at least prompt + n]
      --temp F              sampling temperature, 0 = greedy   [0]
      --top-p F             nucleus cutoff                [0.95]
      --top-k N             candidate cutoff, 0 = off     [0]
      --repeat-penalty F    penalty on recent tokens      [1.0]
      --seed N              sampler seed                  [0]
      --logprobs N          report each token's logprob and N alternatives, from the raw logits   [0]
      --trace PATH          with --ids: write every token's routing decisions (experts, weights) as JSON lines
      --batch N             requests per batch            [all]
      --no-stream           print only the finished list
      --stats               throughput detail
  -o, --out PATH            with --prompts: write results here instead of stdout

BENCH OPTIONS
      --prompt-len N        synthetic prompt length       [32]
      --tokens N            decode steps to time          [16]
      --batch N             sequences decoded together    [1]

      --peak-gbs F          memory bandwidth the roofline line is a percentage of   [7700]
      --kernels             then a table of a decode step's device time by kind of kernel

GLOBAL
      --random CONFIG.json  instead of <model>: random weights of this configuration, drawn on
                            the GPU from --seed (the sampler's seed and the weights' are one option)
      --dtype NAME          bfloat16 | float32            [bfloat16]
      --max-tokens N        tokens the cache can hold     [what the run needs]
  -h, --help                this message
  -V, --version             version
"""

FLAGS = {"help", "kernels", "no-stream", "stats", "version"}
ALIASES = {"n": "tokens", "o": "out", "h": "help", "V": "version"}


def parse_args(argv: List[str]) -> Tuple[str, List[str], Dict[str, str]]:
    pos: List[str] = []
    opt: Dict[str, str] = {}
    i = 0
    while i < len(argv):
        a = argv[i]
        name = None
        if a.startswith("--"):
            name = a[2:]
        elif a.startswith("-") and len(a) > 1 and not a[1].isdigit():
            name = a[1:]
        if name is not None:
            key, _, inline = name.partition("=")
            has_inline = "=" in name
            key = ALIASES.get(key, key)
            if has_inline:
                val = inline
            elif key in FLAGS:
                val = "1"
            else:
                i += 1
                val = argv[i] if i < len(argv) else ""
            opt[key] = val
        else:
            pos.append(a)
        i += 1
    cmd = pos.pop(0) if pos else ""
    return cmd, pos, opt


def fail(msg) -> "None":
    print(f"moe: {msg}", file=sys.stderr)
    raise SystemExit(1)


def _num(opt, key, default, typ):
    if key not in opt:
        return default
    try:
        return typ(opt[key])
    except ValueError:
        return default


def _ids(text: str) -> List[int]:
    text = text.strip()
    if text.startswith("["):
        return [int(x) for x in json.loads(text)]
    return [int(x) for x in text.replace(",", " ").split()]


def human(n: int) -> str:
    units = ["B", "KB", "MB", "GB", "TB"]
    v, i = float(n), 0
    while v >= 1024 and i < len(units) - 1:
        v /= 1024
        i += 1
    return f"{n} B" if i == 0 else f"{v:.2f} {units[i]}"


def _load(path: str, opt, device="cuda"):
    """The model of the command: a folder, or with ``--random CONFIG.json`` random weights of that
    configuration drawn on the device from ``--seed`` (nothing is written)."""
    import moe_b200

    dtype = opt.get("dtype", "bfloat16")
    try:
        if "random" in opt:
            with open(opt["random"], encoding="utf-8") as f:
                cfg = json.load(f)
            return moe_b200.random_model(cfg, seed=_num(opt, "seed", 0, int), dtype=dtype, device=device)
        return moe_b200.load_model(path, dtype=dtype, device=device)
    except (moe_b200.ConfigError, moe_b200.WeightError, ValueError, OSError) as e:
        fail(e)


def _grouped(descriptions: List[str], total: int, what: str) -> List[str]:
    """Equal descriptions once, with the number of parts that have them."""
    seen: Dict[str, int] = {}
    for d in descriptions:
        seen[d] = seen.get(d, 0) + 1
    return [f"  {what:<10} {d}" + ("" if n == total else f"   ({n} of {total})") for d, n in seen.items()]


def summary(model) -> str:
    """The reference's ``Spec::summary`` (src/spec.rs:341-376): what the model is made of, in the
    words of its own parts (``Part.describe``); nothing here knows a kind of part."""
    spec = model.spec
    n = len(model.blocks)
    lines = [spec.architecture, f"  layers {n}  hidden {spec.hidden_size}  vocab {spec.vocab_size}"]
    if len(spec.schedule) != n or any(e.layer != i for i, e in enumerate(spec.schedule)):
        lines.append("  schedule   " + " ".join(
            f"{e.layer}" + ("" if e.writes_cache and e.cache == e.layer else f"[cache {e.cache}{'' if e.writes_cache else ', read'}]")
            for e in spec.schedule))
    by_category: Dict[str, List[str]] = {}
    for b in model.blocks:
        for part in b.parts():
            by_category.setdefault(part.category, []).append(part.describe())
    for category, found in by_category.items():
        lines += _grouped(found, len(found), category)
    lines.append(f"  {'output':<10} {model.head.describe()}")
    return "\n".join(lines)


def step_bytes(model, live_lengths: List[int]) -> Tuple[float, float]:
    """Bytes that a step of one token for each of the live sequences has to read: every weight it
    uses once (``Part.step_elements``; a layer that the schedule runs twice is read twice), and
    the keys and values of the live sequences (a window bounds them).  -> (weights, cache)"""
    esize = 2 if model.rt.is_bf16 else 4
    B = len(live_lengths)
    weights = model.embedding.step_elements(B) + model.final_norm.step_elements(B) + model.head.step_elements(B)
    cache = 0.0
    for e in model.spec.schedule:
        blk = model.blocks[e.layer]
        weights += sum(p.step_elements(B) for p in blk.parts())
        req = blk.mixer.kv_request()
        if req is not None:
            per_pos = 2 * req.num_kv_heads * req.head_dim * esize
            cache += per_pos * sum(min(n, req.window) if req.window else n for n in live_lengths)
    return weights * esize, cache


def cmd_info(path: str, opt) -> None:
    model = _load(path, opt, device="cpu")
    from .models.decoder import expected_tensors

    exp = expected_tensors(model.spec)
    esize = 2 if model.rt.is_bf16 else 4
    total = sum(_numel(t.shape) for t in exp.values()) * esize
    experts = sum(_numel(t.shape) for t in exp.values() if t.sparse) * esize
    print(summary(model))
    print(f"\nweights    {len(exp)} tensors, {human(total)}")
    print(f"  dense    {human(total - experts)}")
    print(f"  experts  {human(experts)} ({100.0 * experts / max(total, 1):.0f}%)")
    kv = sum(2 * r.num_kv_heads * r.head_dim for r in model.kv_requests().values() if r) * esize * 1024
    print(f"kv cache   {human(kv)} per 1k tokens")
    state = sum(_numel(r.shape) * 4 for r in model.state_requests().values() if r)
    if state:
        print(f"state      {human(state)} per sequence")
    print(f"source     {'random weights of ' + opt['random'] if 'random' in opt else path + ' (safetensors)'}")


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def tracing_parts(model):
    """(layer index, feed-forward part) for every run of a layer, in the order of the schedule.  A part
    that routes records its decisions in its ``trace`` list when that is set (``Part.trace``); one that
    does not leaves the list empty."""
    return [(e.layer, model.blocks[e.layer].ffn) for e in model.spec.schedule]


def write_trace(path: str, model, runs, tokens) -> int:
    """One JSON object per (token, routed layer): which experts it chose and with what weight, after a
    header line that explains the file (src/main.rs:771-799).  ``runs``: what ``tracing_parts`` gave,
    their ``trace`` lists filled by a run of ONE request fed in order (prompt, then token by token)."""
    runs = [(layer, p) for layer, p in runs if p.trace]
    times = {id(p): sum(1 for _, q in runs if q is p) for _, p in runs}
    taken = {}
    per_run = []                    # per run of a layer: [(experts, weights)] by position
    for layer, part in runs:
        i = taken.get(id(part), 0)
        taken[id(part)] = i + 1
        rows = []
        for idx, w in part.trace[i::times[id(part)]]:
            for e_row, w_row in zip(idx.tolist(), w.tolist()):
                if e_row and e_row[0] >= 0:             # (rows of no sequence, from a padded step, carry -1)
                    rows.append((e_row, w_row))
        per_run.append((layer, rows))
    spec = model.spec
    first = runs[0][1] if runs else None
    n = 0
    with open(path, "w") as f:
        f.write(json.dumps({"model": spec.architecture, "layers": len(spec.layers),
                            "experts": getattr(first, "E", 0), "top_k": getattr(first, "k", 0)}) + "\n")
        positions = min((len(r) for _, r in per_run), default=0)
        for pos in range(positions):
            for layer, rows in per_run:
                e_row, w_row = rows[pos]
                f.write(json.dumps({"pos": pos, "layer": layer, "token": tokens[pos] if pos < len(tokens) else None,
                                    "experts": [[e, round(w, 6)] for e, w in zip(e_row, w_row)]}) + "\n")
                n += 1
    return n


def cmd_run(path: str, opt) -> None:
    import moe_b200
    from moe_b200.engine.generate import GenerationStats

    if "prompts" in opt:
        src = sys.stdin.read() if opt["prompts"] == "-" else open(opt["prompts"]).read()
        prompts = [_ids(l) for l in src.splitlines() if l.strip()]
        if not prompts:
            fail(f"{opt['prompts']}: no prompts")
    elif "ids" in opt:
        prompts = [_ids(opt["ids"])]
    else:
        fail("give one of --ids or --prompts")
    if any(not p for p in prompts):
        fail("empty prompt")
    n_gen = _num(opt, "tokens", 128, int)
    t_load = time.perf_counter()
    model = _load(path, opt)
    batch = _num(opt, "batch", len(prompts), int)
    longest = max(len(p) for p in prompts)
    max_ctx = model.spec.max_position_embeddings or 4096
    ctx = max(_num(opt, "ctx", min(max_ctx, 4096), int), longest + n_gen)
    need = sum(sorted((-(-(len(p) + n_gen) // 64) * 64 for p in prompts), reverse=True)[:batch])
    engine = moe_b200.Engine(model, max_tokens=_num(opt, "max-tokens", need, int), max_slots=batch)
    load_s = time.perf_counter() - t_load
    stream = "no-stream" not in opt and len(prompts) == 1

    def on_token(i, tok):
        if stream:
            print(tok, end=" ", flush=True)
        return True

    runs = []
    if "trace" in opt:
        if len(prompts) != 1:
            fail("--trace records one request: give --ids")
        runs = tracing_parts(model)
        for _, part in runs:
            part.trace = []
    stats = GenerationStats()
    outs = moe_b200.generate(
        engine, prompts, max_tokens=n_gen, temp=_num(opt, "temp", 0.0, float), top_p=_num(opt, "top-p", 0.95, float),
        top_k=_num(opt, "top-k", 0, int), repeat_penalty=_num(opt, "repeat-penalty", 1.0, float),
        seed=_num(opt, "seed", 0, int), batch_size=batch, ctx=ctx, on_token=on_token, stats=stats,
        logprobs=_num(opt, "logprobs", 0, int), lookahead=False if runs else None)
    if runs:
        n = write_trace(opt["trace"], model, runs, prompts[0] + outs[0].tokens)
        for _, part in runs:
            part.trace = None
        print(f"wrote {n} routing records to {opt['trace']}", file=sys.stderr)

    def probes(o):
        return [{"token": t, "logprob": round(lp, 6), "top": [[i, round(l, 6)] for i, l in top]}
                for t, (lp, top) in zip(o.tokens, o.logprobs)]

    if "prompts" in opt:
        lines = [json.dumps({"index": i, "prompt": prompts[i], "tokens": o.tokens, "generated": len(o.tokens),
                             "prompt_tokens": o.prompt_tokens, "finish": o.finish_reason,
                             **({"logprobs": probes(o)} if o.logprobs is not None else {})})
                 for i, o in enumerate(outs)]
        if "out" in opt:
            with open(opt["out"], "w") as f:
                f.write("\n".join(lines) + "\n")
            print(f"wrote {len(lines)} results to {opt['out']}", file=sys.stderr)
        else:
            print("\n".join(lines))
    elif stream:
        print()
    else:
        print(outs[0].tokens)
    if "prompts" not in opt and outs[0].logprobs is not None:
        print(json.dumps(probes(outs[0])))
    gen = sum(len(o.tokens) for o in outs)
    print(f"\nload {load_s:.2f}s | prefill {stats.prefill_tokens} tok in {stats.prefill_seconds:.2f}s "
          f"({stats.prefill_tokens / max(stats.prefill_seconds, 1e-6):.1f} tok/s) | decode {gen} tok in "
          f"{stats.decode_seconds:.2f}s ({stats.decode_tokens / max(stats.decode_seconds, 1e-6):.2f} tok/s)",
          file=sys.stderr)
    if "stats" in opt:
        print(f"decode steps {stats.decode_steps} | kv cache {human(engine.cache.bytes())} | "
              f"finish {[o.stop for o in outs]}", file=sys.stderr)


def cmd_bench(path: str, opt) -> None:
    """``moe bench`` (src/main.rs:1221-1253): ids (i*7+13) % vocab, timed prefill, then timed
    single-token steps with fixed tokens i % vocab; logits are computed every step."""
    import torch

    import moe_b200

    model = _load(path, opt)
    plen, n, B = _num(opt, "prompt-len", 32, int), _num(opt, "tokens", 16, int), _num(opt, "batch", 1, int)
    V = model.spec.vocab_size
    ids = [(i * 7 + 13) % V for i in range(plen)]
    engine = moe_b200.Engine(model, max_tokens=B * (-(-(plen + n + 8) // 64) * 64), max_slots=B)
    slots = [engine.new_sequence() for _ in range(B)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.step(slots, [ids] * B)
    torch.cuda.synchronize()
    pf = time.perf_counter() - t0
    t1 = time.perf_counter()
    for i in range(n):
        engine.step(slots, [[i % V]] * B, check=False)
    torch.cuda.synchronize()
    dc = time.perf_counter() - t1
    engine.rt.check()
    print(summary(model))
    print(f"\nprefill  {plen * B} tok in {pf:.3f}s   {plen * B / max(pf, 1e-9):.1f} tok/s")
    print(f"decode   {n * B} tok in {dc:.3f}s   {n * B / max(dc, 1e-9):.2f} tok/s   {1000.0 * dc / max(n, 1):.2f} ms/step")
    print(f"batch    {B}   dtype {opt.get('dtype', 'bfloat16')}   kv cache {human(engine.cache.bytes())}")
    # what a decode step has to read, against the memory bandwidth given (B200 HBM3e nominal by default)
    wb, cb = step_bytes(model, [plen + n // 2] * B)
    peak = _num(opt, "peak-gbs", 7700.0, float)
    gbs = (wb + cb) / max(dc / max(n, 1), 1e-12) / 1e9
    print(f"roofline {human(int(wb))} weights + {human(int(cb))} cache a step   {gbs:.0f} GB/s   "
          f"{100.0 * gbs / peak:.1f}% of {peak:.0f} GB/s")
    if "kernels" in opt:
        print()
        print(kernel_table(lambda i: engine.step(slots, [[i % V]] * B, check=False), steps=4))


def kernel_table(step, steps: int = 4) -> str:
    """Device time of a decode step by kind of kernel: ``steps`` more steps under the CUDA activity
    tracer, each kernel's time summed by its name without template arguments.  (Kernels that overlap,
    on two streams or through programmatic dependent launch, are each counted in full, so the sum
    can exceed the step's time.)"""
    import re

    import torch
    from torch.profiler import ProfilerActivity, profile

    import warnings

    torch.cuda.synchronize()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(steps):
                step(i)
            torch.cuda.synchronize()
    kinds: Dict[str, List[float]] = {}
    for e in prof.events():
        if e.device_type != torch.autograd.DeviceType.CUDA:
            continue
        name = re.sub(r"\(anonymous namespace\)::|^void ", "", e.name)
        name = re.sub(r"<.*", "", name.split("(")[0]).strip() or e.name
        k = kinds.setdefault(name, [0.0, 0])
        k[0] += e.time_range.end - e.time_range.start
        k[1] += 1
    total = sum(v[0] for v in kinds.values()) or 1.0
    lines = [f"{'kernel':<34}{'us/step':>10}{'share':>8}{'launches/step':>15}"]
    for name, (us, n) in sorted(kinds.items(), key=lambda kv: -kv[1][0]):
        lines.append(f"{name[:33]:<34}{us / steps:>10.1f}{100.0 * us / total:>7.1f}%{n / steps:>15.1f}")
    return "\n".join(lines)


def main(argv=None) -> int:
    import moe_b200

    cmd, pos, opt = parse_args(list(sys.argv[1:] if argv is None else argv))
    if "version" in opt:
        print(f"moe {moe_b200.__version__}")
        return 0
    if "help" in opt or not cmd:
        print(USAGE)
        return 0
    if cmd not in ("run", "info", "bench"):
        fail(f"unknown command '{cmd}' (try --help)")
    if not pos and "random" not in opt:
        fail(f"{cmd}: name a model folder (or --random CONFIG.json)")
    {"run": cmd_run, "info": cmd_info, "bench": cmd_bench}[cmd](pos[0] if pos else "", opt)
    return 0

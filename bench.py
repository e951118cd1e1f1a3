#!/usr/bin/env python3
"""Decode and prefill throughput of moe_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of Qwen1.5-MoE-A2.7B with random bfloat16 weights,
8 sequences with 512-token prompts inside a 4096-token context, K decode steps.
A "step" is one decode step (inputs copied from pinned memory, every layer, the
output projection and a greedy pick).  Prints ONE JSON line.

  value    decoded tokens a second, timed on the device with CUDA events
  e2e      the same through moe_b200.generate(): host token lists in and out
  prefill  one 2,048-token prompt: tokens a second and fraction of the bf16 peak
  roofline bytes a decode step must read (every weight it uses once, and the
           cache of the live requests) / its time, against the measured copy bandwidth
  points   decode at batch 1 and 64

The reference (JGalego/Moe) is a Rust CPU engine; it installs only with a Rust
toolchain, which this image lacks, so ``--impl reference`` reports that.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

A27B = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=24, hidden_size=2048, num_attention_heads=16, num_key_value_heads=16, head_dim=128,
    num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
    intermediate_size=5632, norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[],
    vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, use_sliding_window=False, tie_word_embeddings=False,
    max_position_embeddings=8192,
)
FULL_LAYERS = 24
# the larger shape of the same architecture (Qwen2-57B-A14B): only with --sweep, to see other sizes
A57B = dict(A27B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
            num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560, shared_expert_intermediate_size=20480,
            intermediate_size=18944)
CONTEXT, PROMPT_LEN, PREFILL_TOKENS = 4096, 512, 2048


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        self.rows = []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def model_numbers(cfg, layers):
    """Parameter counts and per-token work of the configuration."""
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, mi, si = cfg["num_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"]
    attn = (nh + 2 * nkv) * hd * H + H * nh * hd
    expert = 3 * mi * H
    shared = 3 * si * H + H
    router = E * H
    return dict(attn=attn, expert=expert, shared=shared, router=router, head=V * H,
                kv_bytes_per_token_layer=2 * nkv * hd * 2,
                active_per_token=layers * (attn + k * expert + shared + router))


def run_ours(args):
    import torch

    import moe_b200
    from moe_b200.engine.generate import GenerationStats
    from moe_b200.ops import core
    from moe_b200.sampling.params import SamplingParams
    from moe_b200.sampling.sampler import DeviceSampler

    pk = peaks()
    cfg = dict(A57B if (args.sweep and args.shape == "57b") else A27B)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    torch.cuda.set_device(0)
    model = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    V = cfg["vocab_size"]
    nums = model_numbers(cfg, layers)
    clocks = ClockSampler()

    def decode_run(B, steps, warmup, sample_clocks=False, prompt_len=PROMPT_LEN):
        """``prompt_len``: one length for all sequences, or (lo, hi) for unequal lengths drawn from a
        seeded generator.  -> (ms per step, launches per step, h2d bytes per step, mean cache tokens a
        sequence, unique experts per layer, clocks)"""
        if isinstance(prompt_len, tuple):
            import random

            rng = random.Random(B)
            lens = [rng.randint(*prompt_len) for _ in range(B)]
        else:
            lens = [prompt_len] * B
        room = sum(-(-(n + steps + warmup + 8) // 64) * 64 for n in lens)
        eng = moe_b200.Engine(model, max_tokens=room, max_slots=B)
        sampler = DeviceSampler(eng.cache.rng_states, eng.rt.device)
        greedy = SamplingParams()
        slots = [eng.new_sequence() for _ in range(B)]
        prompts = [[(i * 7 + 13 + 31 * b) % V for i in range(lens[b])] for b in range(B)]
        b0 = 0
        while b0 < B:                                   # prompts in groups of at most 4,096 tokens, to bound the workspace
            b1, held = b0, 0
            while b1 < B and (b1 == b0 or held + lens[b1] <= 4096) and b1 - b0 < 8:
                held += lens[b1]
                b1 += 1
            eng.step(slots[b0:b1], prompts[b0:b1], [[] for _ in slots[b0:b1]])
            b0 = b1

        def one(i):
            logits = eng.step(slots, [[(i * 13 + 7 * b) % V] for b in range(B)], check=False)
            return sampler.sample(logits, eng.last_batch.slots, greedy)

        for i in range(warmup):
            one(i)
        # which experts a step touches (for the byte count), measured on one extra untimed step
        routed = [b.ffn for b in model.blocks if b.ffn.kind == "routed_experts"]
        for r in routed:
            r.trace = []
        one(warmup)
        uniq = sum(len(torch.unique(r.trace[0][0][:B])) for r in routed) / max(len(routed), 1)   # (rows past B: padding)
        for r in routed:
            r.trace = None
        torch.cuda.synchronize()
        if sample_clocks:
            clocks.start()
        l0 = core.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for i in range(steps):
            one(warmup + 1 + i)
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        clk = clocks.stop() if sample_clocks else None
        eng.rt.check()
        launches = (core.launches - l0) / steps
        mean_len = sum(lens) / B + warmup + 1 + steps / 2
        h2d = (3 * B + 4 * B + 2 + B) * 4
        for s in slots:
            eng.release(s)
        del eng
        torch.cuda.empty_cache()
        return ms, launches, h2d, mean_len, uniq, clk

    def decode_bytes(B, mean_len, uniq):
        per_layer = nums["attn"] + nums["shared"] + nums["router"] + uniq * nums["expert"]
        weights = 2 * (layers * per_layer + nums["head"]) + 2 * B * cfg["hidden_size"]   # bf16, + embedding rows
        kv = B * mean_len * nums["kv_bytes_per_token_layer"] * layers
        return weights + kv

    if args.sweep:
        # decode only, one line per batch size (not the benchmark record)
        for b in [int(v) for v in args.sweep.split(",")]:
            plen = (256, 2048) if args.unequal else (args.prompt_len or PROMPT_LEN)
            m, _, _, mean_len, uniq, _ = decode_run(b, max(8, args.steps // 2), args.warmup, prompt_len=plen)
            nb = decode_bytes(b, mean_len, uniq)
            gbs = nb / (m / 1e3) / 1e9
            print(json.dumps({"shape": args.shape, "layers": layers, "batch": b, "cache_tokens": int(mean_len),
                              "experts_per_layer": round(uniq, 1), "bytes_per_step": int(nb), "ms_per_step": round(m, 4),
                              "tokens_per_s": round(b / (m / 1e3), 1), "hbm_gbs": round(gbs, 1),
                              "hbm_frac": round(gbs / pk["hbm_gbs"], 4)}), flush=True)
        return 0

    # ---- headline: batch 8 ---------------------------------------------------------------
    B = 8
    ms, launches, h2d, mean_len, uniq, clk = decode_run(B, args.steps, args.warmup, sample_clocks=True)
    value = B / (ms / 1e3)
    nbytes = decode_bytes(B, mean_len, uniq)
    achieved = nbytes / (ms / 1e3) / 1e9

    # ---- other batch sizes: at least 64 steps each, with clocks and roofline of their own --------
    points, points_detail = {}, {}
    for b in (1, 64):
        n_steps = max(64, args.steps)
        m, _, _, ml, uq, ck = decode_run(b, n_steps, args.warmup, sample_clocks=True)
        points[f"decode_b{b}"] = round(b / (m / 1e3), 1)
        gbs = decode_bytes(b, ml, uq) / (m / 1e3) / 1e9
        points_detail[f"decode_b{b}"] = {"ms_per_step": round(m, 4), "steps": n_steps, "hbm_gbs": round(gbs, 1),
                                         "hbm_frac": round(gbs / pk["hbm_gbs"], 4), "experts_per_layer": round(uq, 1),
                                         "sm_mhz": ck["sm_mhz"], "reasons": ck["reasons"]}

    # ---- prefill of 2,048 tokens ------------------------------------------------------------
    eng = moe_b200.Engine(model, max_tokens=PREFILL_TOKENS + 64, max_slots=1)
    ids = [(i * 7 + 13) % V for i in range(PREFILL_TOKENS)]
    times = []
    for it in range(args.warmup + 5):
        s = eng.new_sequence()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([s], [ids], check=False)
        b_.record()
        torch.cuda.synchronize()
        eng.release(s)
        if it >= args.warmup:
            times.append(a.elapsed_time(b_))
    eng.rt.check()
    pf_ms = sorted(times)[len(times) // 2]
    T = PREFILL_TOKENS
    flops = 2 * T * nums["active_per_token"] + 2 * nums["head"] \
        + layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * T * (T + 1) // 2
    # frac: of the burst peak (a cuBLAS product timed alone); frac_sustained: of the peak of a seconds-long
    # loop under the power cap, which is the state this step is measured in, after the decode runs
    prefill = {"value": round(T / (pf_ms / 1e3), 1), "tokens": T, "ms": round(pf_ms, 3),
               "frac": round(flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               "frac_sustained": round(flops / (pf_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}
    del eng
    torch.cuda.empty_cache()

    # ---- end to end through the Python entry point ----------------------------------------
    eng = moe_b200.Engine(model, max_tokens=8 * (-(-(PROMPT_LEN + args.steps + 8) // 64) * 64), max_slots=8)
    prompts = [[(i * 7 + 13 + 31 * b) % V for i in range(PROMPT_LEN)] for b in range(8)]
    moe_b200.generate(eng, prompts, max_tokens=4, eos=())                       # warm-up
    st = GenerationStats()
    moe_b200.generate(eng, prompts, max_tokens=args.steps + 1, eos=(), stats=st)
    e2e = {"value": round(st.decode_tokens / max(st.decode_seconds, 1e-9), 1), "unit": "tokens/s",
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": (8 + 1) * 4,
           "prefill_tokens_per_s": round(st.prefill_tokens / max(st.prefill_seconds, 1e-9), 1)}

    out = {
        "metric": "decode tokens/s (batch 8, Qwen1.5-MoE-A2.7B shape, bf16)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random weights N(0, 0.02)",
        "config": {
            "model": "Qwen1.5-MoE-A2.7B shape", "layers": layers, "layers_of_model": FULL_LAYERS, "hidden": 2048,
            "heads": 16, "kv_heads": 16, "head_dim": 128, "experts": 60, "top_k": 4, "moe_intermediate": 1408,
            "shared_intermediate": 5632, "vocab": V, "global_batch": B, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights read per step >> 126 MB)",
            "peaks": pk["source"],
        },
        "clocks": clk,
        "e2e": e2e,
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(nbytes),
                     "experts_per_layer": round(uniq, 1), "of": pk["source"]},
        "points": points,
        "points_detail": points_detail,
    }
    print(json.dumps(out))
    return 0


def run_fp32_long(args):
    """The true 32-bit path at the model's layer sizes and a long context: 8 sequences of unequal
    prompts (4,096 to 24,576 tokens, seeded) inside 32,768 positions, a window of 4,096 on the last
    three layers, then 64 decode steps; and the logits of two of the prompts against the bfloat16
    path on the same (bfloat16-representable) weights.  Prints one JSON line; not the benchmark record."""
    import random

    import torch

    import moe_b200

    pk = peaks()
    cfg = dict(A27B, use_sliding_window=True, sliding_window=4096, max_window_layers=21, max_position_embeddings=32768)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    cfg["max_window_layers"] = max(0, layers - 3)
    V = cfg["vocab_size"]
    rng = random.Random(5)
    lens = [rng.randint(4096, 24576) for _ in range(8)] if not args.prompt_len else [args.prompt_len] * 8
    steps = 64
    model = moe_b200.random_model(cfg, seed=0, dtype="float32", device="cuda:0", stored_dtype="bfloat16")
    room = sum(-(-(n + steps + 8) // 64) * 64 for n in lens)
    eng = moe_b200.Engine(model, max_tokens=room, max_slots=8)
    prompts = [[(i * 7 + 13 + 31 * b) % V for i in range(n)] for b, n in enumerate(lens)]
    slots = [eng.new_sequence() for _ in lens]
    last = {}
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for b in range(8):
        last[b] = eng.step([slots[b]], [prompts[b]]).float().clone()     # (the engine runs it in pieces)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    nums = model_numbers(cfg, layers)
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(3):
        eng.step(slots, [[(i * 13 + 7 * b) % V] for b in range(8)], check=False)
    a.record()
    for i in range(steps):
        eng.step(slots, [[(i * 13 + 7 * b + 3) % V] for b in range(8)], check=False)
    z.record()
    torch.cuda.synchronize()
    eng.rt.check()
    ms = a.elapsed_time(z) / steps
    full, win = cfg["max_window_layers"], layers - cfg["max_window_layers"]
    kv_tok = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 4
    mean = [n + 3 + steps / 2 for n in lens]
    kv = kv_tok * (full * sum(mean) + win * sum(min(m, 4096) for m in mean))
    uniq = cfg["num_experts"] * (1 - (1 - cfg["num_experts_per_tok"] / cfg["num_experts"]) ** 8)
    weights = 4 * (layers * (nums["attn"] + nums["shared"] + nums["router"] + uniq * nums["expert"]) + nums["head"])
    gbs = (weights + kv) / (ms / 1e3) / 1e9
    out = {"workload": "float32, context 32768, 8 unequal prompts, 64 decode steps", "layers": layers, "prompt_tokens": lens,
           "prefill_tokens_per_s": round(sum(lens) / prefill_s, 1), "prefill_s": round(prefill_s, 2),
           "decode_ms_per_step": round(ms, 3), "decode_tokens_per_s": round(8 / (ms / 1e3), 1),
           "decode_bytes_per_step": int(weights + kv), "decode_hbm_gbs": round(gbs, 1),
           "decode_hbm_frac": round(gbs / pk["hbm_gbs"], 4)}
    # ---- the bfloat16 path on the same weights: the two shortest prompts' last logits --------------
    for s_ in slots:
        eng.release(s_)
    short = sorted(range(8), key=lambda b: lens[b])[:2]
    del eng
    torch.cuda.empty_cache()
    m16 = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    e16 = moe_b200.Engine(m16, max_tokens=sum(-(-(lens[b] + 8) // 64) * 64 for b in short), max_slots=2)
    worst = []
    for n, b in enumerate(short):
        # the first whole, the second in pieces of 2,048 tokens that go on from the cache (the windowed
        # layers' rings wrap on the way)
        e16.max_step_tokens = 8192 if n == 0 else 2048
        s_ = e16.new_sequence()
        lg = e16.step([s_], [prompts[b]]).float()
        e16.release(s_)
        worst.append(round(float((lg - last[b]).abs().max() / last[b].abs().max()), 5))
    out["bf16_vs_fp32_last_logits_rel"] = max(worst)
    out["bf16_vs_fp32_prompts"] = [lens[b] for b in short]
    out["bf16_vs_fp32_each"] = {"whole": worst[0], "pieces_of_2048": worst[1]}
    print(json.dumps(out))
    return 0


def run_long_prompt(args):
    """One prompt of ``--prompt-len`` tokens (32,768 unless given) in bfloat16 through the engine's
    step, which runs it in pieces of at most 8,192 tokens that go on from the cache.  Prints one JSON
    line; not the benchmark record."""
    import torch

    import moe_b200

    pk = peaks()
    cfg = dict(A27B, max_position_embeddings=131072)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    V = cfg["vocab_size"]
    T = args.prompt_len or 32768
    model = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    eng = moe_b200.Engine(model, max_tokens=-(-T // 64) * 64 + 64, max_slots=1)
    ids = [(i * 7 + 13) % V for i in range(T)]
    times = []
    for it in range(3):
        s = eng.new_sequence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([s], [ids], check=False)
        b.record()
        torch.cuda.synchronize()
        eng.rt.check()
        eng.release(s)
        times.append(a.elapsed_time(b))
    ms = sorted(times)[1]
    nums = model_numbers(cfg, layers)
    flops = 2 * T * nums["active_per_token"] + 2 * nums["head"] \
        + layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * T * (T + 1) // 2
    print(json.dumps({"workload": "bfloat16, one prompt, pieces of %d tokens" % eng.max_step_tokens, "layers": layers,
                      "prompt_tokens": T, "ms": round(ms, 2), "tokens_per_s": round(T / (ms / 1e3), 1),
                      "tflops": round(flops / (ms / 1e3) / 1e12, 1),
                      "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
    return 0


def profile_step(args):
    """A small case for a profiler: the model's layer sizes, few layers, graphs off (every kernel is
    a launch of its own); only the steps between cudaProfilerStart and cudaProfilerStop matter."""
    import torch

    import moe_b200

    cfg = dict(A27B)
    V = cfg["vocab_size"]
    if args.profile_step == "sample":
        # the sampling kernels alone, on random logits of the model's vocabulary: greedy, then a
        # temperature with top-p, then with top-k too
        from moe_b200.ops import core

        B = args.batch
        logits = torch.randn(B, V, device="cuda:0") * 2
        slots = torch.arange(B, dtype=torch.int32, device="cuda:0")
        rng = torch.arange(1, B + 2, dtype=torch.int64, device="cuda:0") * 0x9E3779B97F4A7C15 % (1 << 62) | 1
        out = torch.zeros(B, dtype=torch.int32, device="cuda:0")
        last = torch.zeros(B + 1, dtype=torch.int32, device="cuda:0")

        def run(i):
            core.sample(logits, slots, rng, out, last_token=last)
            core.sample(logits, slots, rng, out, temp=0.8, top_p=0.95, last_token=last)
            core.sample(logits, slots, rng, out, temp=0.8, top_k=40, top_p=0.95, last_token=last)
        model = None
    else:
        cfg["num_hidden_layers"] = args.layers or 2
        model = moe_b200.random_model(cfg, seed=0, dtype=args.dtype, device="cuda:0")
    if args.profile_step == "sample":
        pass
    elif args.profile_step == "decode":
        B = args.batch
        eng = moe_b200.Engine(model, max_tokens=B * 1024, max_slots=B, use_graphs=False)
        slots = [eng.new_sequence() for _ in range(B)]
        eng.step(slots, [[(i * 7 + 31 * b) % V for i in range(PROMPT_LEN)] for b in range(B)], [[] for _ in slots])
        run = lambda i: eng.step(slots, [[(i * 13 + 7 * b) % V] for b in range(B)])
    elif args.profile_step == "chunk":
        # a piece of a long prompt: --prompt-len tokens [2048] that go on from 6,144 tokens in the cache
        n, past = args.prompt_len or PREFILL_TOKENS, 6144
        eng = moe_b200.Engine(model, max_tokens=past + n + 64, max_slots=1, use_graphs=False)
        s = eng.new_sequence()
        eng.step([s], [[(i * 7 + 13) % V for i in range(past)]], [[]])
        ids = [(i * 11 + 5) % V for i in range(n)]

        def run(i):
            eng.step([s], [ids])
            eng.truncate(s, past)
    else:
        eng = moe_b200.Engine(model, max_tokens=PREFILL_TOKENS + 64, max_slots=1, use_graphs=False)
        ids = [(i * 7 + 13) % V for i in range(PREFILL_TOKENS)]

        def run(i):
            s = eng.new_sequence()
            eng.step([s], [ids])
            eng.release(s)
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for i in range(max(1, min(args.steps, 2))):
        run(3 + i)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    print(f"profiled {args.profile_step} step(s)")
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (reported in config)")
    ap.add_argument("--profile-step", choices=["decode", "prefill", "chunk", "sample"], default=None,
                    help="run a few steps of one kind between cudaProfilerStart/Stop (for ncu "
                         "--profile-from-start off) and print no benchmark line")
    ap.add_argument("--batch", type=int, default=8, help="with --profile-step decode: sequences in the batch")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="with --profile-step: the path whose kernels are wanted")
    ap.add_argument("--shape", choices=["a2.7b", "57b"], default="a2.7b", help="with --sweep: the layer sizes")
    ap.add_argument("--prompt-len", type=int, default=0, help="with --sweep: tokens in each prompt (default 512)")
    ap.add_argument("--workload", choices=["fp32-32k", "long-prompt"], default=None,
                    help="fp32-32k: the true 32-bit path at a context of 32,768; long-prompt: one bfloat16 prompt of "
                         "--prompt-len tokens [32768] run in pieces (each prints its own line, no benchmark record)")
    ap.add_argument("--unequal", action="store_true", help="with --sweep: prompts of unequal lengths, 256 to 2,048 tokens")
    ap.add_argument("--sweep", default=None, help="comma-separated batch sizes: print decode throughput for each "
                                                  "and no benchmark line")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "JGalego/Moe is a Rust crate (no Python package, "
                          "no setup.py/pyproject); cargo and rustc are absent from this image and there is no network"}))
        return 0
    if args.gpus != 1:
        print("bench.py: moe_b200 is a single-GPU library; --gpus must be 1")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.profile_step:
        return profile_step(args)
    if args.workload == "long-prompt":
        return run_long_prompt(args)
    if args.workload == "fp32-32k":
        return run_fp32_long(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())

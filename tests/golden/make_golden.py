#!/usr/bin/env python3
"""Write tests/golden/qwen2moe_oracle from the reference's own scripts/oracle.py.

    python tests/golden/make_golden.py /path/to/JGalego-Moe/scripts/oracle.py

The oracle (pure standard library, Python doubles) is imported, a tiny random
model is built with its generator, and its ``forward`` gives logits after every
prefix of a token list.  The model uses only what the oracle can express of
Qwen2 MoE: grouped-query attention without q/k norm, half-split rotary, the
Qwen window convention, softmax top-k routing without renormalisation, routed
SwiGLU experts, a dense first layer, an (ungated) shared expert, tied output.

The folder is written in Qwen2 MoE's own conventions so that any loader of that
architecture reads it: ``mlp.shared_experts.*`` becomes ``mlp.shared_expert.*``
with ``down_proj`` doubled and a zero ``shared_expert_gate`` (sigmoid(0) * 2 = 1
exactly), and ``lm_head`` is dropped because the embedding is tied.
"""
import importlib.util
import json
import os
import sys


def main():
    oracle_path = sys.argv[1]
    spec = importlib.util.spec_from_file_location("moe_oracle", oracle_path)
    oracle = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(oracle)

    rng = oracle.Rand(0x51DE)
    H, V, NH, NKV, HD, E, MI, DI, SI, L = 32, 48, 4, 2, 16, 4, 16, 24, 16, 2
    cfg = dict(
        architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
        hidden_size=H, num_hidden_layers=L, num_attention_heads=NH, num_key_value_heads=NKV, head_dim=HD,
        vocab_size=V, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=128,
        num_experts=E, num_experts_per_tok=2, moe_intermediate_size=MI, intermediate_size=DI,
        shared_expert_intermediate_size=SI, norm_topk_prob=False, tie_word_embeddings=True,
        sliding_window=3, use_sliding_window=True, max_window_layers=1,
        decoder_sparse_step=2, mlp_only_layers=[], qkv_bias=False,
    )
    w = {"model.embed_tokens.weight": rng.mat(V, H), "model.norm.weight": rng.vec(H, 0.2, 1.0)}
    w["lm_head.weight"] = w["model.embed_tokens.weight"]
    for l in range(L):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = rng.vec(H, 0.2, 1.0)
        w[p + "post_attention_layernorm.weight"] = rng.vec(H, 0.2, 1.0)
        w[p + "self_attn.q_proj.weight"] = rng.mat(NH * HD, H)
        w[p + "self_attn.k_proj.weight"] = rng.mat(NKV * HD, H)
        w[p + "self_attn.v_proj.weight"] = rng.mat(NKV * HD, H)
        w[p + "self_attn.o_proj.weight"] = rng.mat(H, NH * HD)
        if l == 0:
            w[p + "mlp.gate_proj.weight"] = rng.mat(DI, H)
            w[p + "mlp.up_proj.weight"] = rng.mat(DI, H)
            w[p + "mlp.down_proj.weight"] = rng.mat(H, DI)
            continue
        w[p + "mlp.gate.weight"] = rng.mat(E, H)
        for e in range(E):
            q = p + f"mlp.experts.{e}."
            w[q + "gate_proj.weight"] = rng.mat(MI, H)
            w[q + "up_proj.weight"] = rng.mat(MI, H)
            w[q + "down_proj.weight"] = rng.mat(H, MI)
        s = p + "mlp.shared_experts."
        w[s + "gate_proj.weight"] = rng.mat(SI, H)
        w[s + "up_proj.weight"] = rng.mat(SI, H)
        w[s + "down_proj.weight"] = rng.mat(H, SI)

    assert oracle.windows(cfg, L) == [None, 3]
    tokens = [3, 11, 5, 40, 7, 1, 22, 9, 30, 2]
    logits = oracle.forward(cfg, w, tokens)

    # the same weights under Qwen2 MoE's names
    out = {}
    for name, t in w.items():
        if name == "lm_head.weight":
            continue
        if ".mlp.shared_experts." in name:
            new = name.replace(".mlp.shared_experts.", ".mlp.shared_expert.")
            out[new] = [[2.0 * v for v in row] for row in t] if new.endswith("down_proj.weight") else t
        else:
            out[name] = t
    for l in range(1, L):
        out[f"model.layers.{l}.mlp.shared_expert_gate.weight"] = [[0.0] * H]

    d = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qwen2moe_oracle")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    oracle.write_safetensors(os.path.join(d, "model.safetensors"), out)
    with open(os.path.join(d, "expected.json"), "w") as f:
        json.dump({"tokens": tokens, "logits": logits}, f)
    print(f"{d}: {len(out)} tensors, {len(tokens)} positions")


if __name__ == "__main__":
    main()

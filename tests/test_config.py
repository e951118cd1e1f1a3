"""Configuration and registry (CPU)."""
import copy
import json

import pytest

import helpers
from moe_b200.config import ConfigError, Qwen2MoeConfig, parse_config, read_config_json, registered_architectures


def test_both_tiny_configurations_parse_and_differ_in_every_size():
    a = Qwen2MoeConfig.from_dict(helpers.CONFIG_A)
    b = Qwen2MoeConfig.from_dict(helpers.CONFIG_B)
    for f in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
              "num_experts", "num_experts_per_tok", "moe_intermediate_size", "shared_expert_intermediate_size",
              "norm_topk_prob", "vocab_size", "rope_theta", "rms_norm_eps", "tie_word_embeddings",
              "decoder_sparse_step", "intermediate_size"):
        assert getattr(a, f) != getattr(b, f), f
    assert a.eos_token_ids == (255,) and b.eos_token_ids == (7, 383)


def test_sparse_and_dense_layers_follow_step_and_mlp_only():
    b = Qwen2MoeConfig.from_dict(helpers.CONFIG_B)
    # decoder_sparse_step 2 and mlp_only_layers [2]: layers 0 and 2 are dense, layer 1 routed
    assert [b.layer_is_sparse(l) for l in range(3)] == [False, True, False]
    a = Qwen2MoeConfig.from_dict(helpers.CONFIG_A)
    assert all(a.layer_is_sparse(l) for l in range(2))


def test_window_conventions():
    """The cases of the reference's own unit test (src/spec.rs:580-609)."""
    base = dict(helpers.CONFIG_A, num_hidden_layers=4)
    w = lambda **kw: Qwen2MoeConfig.from_dict(dict(base, **kw)).layer_windows()
    assert w() == [None] * 4
    assert w(sliding_window=0, use_sliding_window=True) == [None] * 4
    assert w(sliding_window=32, use_sliding_window=True, max_window_layers=2) == [None, None, 32, 32]
    assert w(sliding_window=32, use_sliding_window=False) == [None] * 4
    assert w(sliding_window=128, layer_types=["sliding_attention", "full_attention", "sliding_attention",
                                              "full_attention"]) == [128, None, 128, None]
    assert Qwen2MoeConfig.from_dict(helpers.CONFIG_B).layer_windows() == [None, 8, 8]


def test_defaults_follow_the_reference():
    c = Qwen2MoeConfig.from_dict(dict(hidden_size=64, num_attention_heads=4, num_hidden_layers=1, vocab_size=10,
                                      intermediate_size=8))
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.head_dim == 16
    assert c.num_key_value_heads == 4 and c.norm_topk_prob is False and c.eos_token_ids == ()


@pytest.mark.parametrize("bad, needle", [
    (dict(hidden_size=None), "hidden_size"),
    (dict(num_attention_heads=None), "num_attention_heads"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(num_experts_per_tok=9), "num_experts_per_tok"),
    (dict(moe_intermediate_size=None), "moe_intermediate_size"),
    (dict(vocab_size="big"), "integer"),
    (dict(mlp_only_layers=[7]), "mlp_only_layers"),
    (dict(eos_token_id=9999), "eos_token_id"),
    (dict(decoder_sparse_step=0), "decoder_sparse_step"),
])
def test_bad_configs_are_refused_with_the_key_named(bad, needle):
    cfg = copy.deepcopy(helpers.CONFIG_A)
    for k, v in bad.items():
        if v is None:
            cfg.pop(k)
        else:
            cfg[k] = v
    with pytest.raises(ConfigError) as e:
        Qwen2MoeConfig.from_dict(cfg)
    assert needle in str(e.value)


def test_dense_layers_need_intermediate_size():
    cfg = copy.deepcopy(helpers.CONFIG_B)
    cfg.pop("intermediate_size")
    with pytest.raises(ConfigError):
        Qwen2MoeConfig.from_dict(cfg)


def test_registry_picks_the_architecture_and_lists_known_names():
    arch, typed = parse_config(helpers.CONFIG_A)
    assert arch.name == "Qwen2MoeForCausalLM" and isinstance(typed, Qwen2MoeConfig)
    arch2, _ = parse_config({k: v for k, v in helpers.CONFIG_A.items() if k != "architectures"})
    assert arch2.name == arch.name      # by model_type
    with pytest.raises(ConfigError) as e:
        parse_config(dict(helpers.CONFIG_A, architectures=["LlamaForCausalLM"]))
    assert "Qwen2MoeForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    assert "Qwen2MoeForCausalLM" in registered_architectures()


def test_config_json_errors(tmp_path):
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(helpers.CONFIG_A))
    assert read_config_json(str(tmp_path))["hidden_size"] == 64


def test_round_trip_through_config_json():
    for cfg in helpers.CONFIGS.values():
        c = Qwen2MoeConfig.from_dict(cfg)
        assert Qwen2MoeConfig.from_dict(c.to_dict()) == c


def test_model_spec_is_data_layer_by_layer():
    arch, typed = parse_config(helpers.CONFIG_B)
    spec = arch.model_spec(typed)
    assert [l.ffn.kind for l in spec.layers] == ["dense_swiglu", "routed_experts", "dense_swiglu"]
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 8, 8]
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True)]
    assert spec.head.params["tied"] is True

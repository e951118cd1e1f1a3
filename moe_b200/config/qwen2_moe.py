"""Typed configuration of Qwen2 MoE (``Qwen2MoeForCausalLM``), read from the
architecture's own config.json keys.

Every size and constant comes from config.json; the defaults below are the ones
the reference engine applies when a key is absent (src/spec.rs:255-337), except
``norm_topk_prob``, whose default for this architecture is false
(src/gguf.rs:326-333).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import Architecture, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Qwen2MoeForCausalLM"


def _need(cfg: Dict[str, Any], key: str, typ=int):
    if key not in cfg or cfg[key] is None:
        raise ConfigError(f"{ARCHITECTURE}: config.json lacks '{key}'")
    return _typed(cfg, key, typ)


def _typed(cfg, key, typ):
    v = cfg[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"{ARCHITECTURE}: '{key}' must be an integer, got {v!r}")
        return int(v)
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{ARCHITECTURE}: '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"{ARCHITECTURE}: '{key}' must be true or false, got {v!r}")
        return v
    raise AssertionError(typ)


def _opt(cfg, key, typ, default):
    if key not in cfg or cfg[key] is None:
        return default
    return _typed(cfg, key, typ)


def _ids(cfg, key) -> Tuple[int, ...]:
    # a number or an array of numbers (src/spec.rs:222-228)
    v = cfg.get(key)
    if isinstance(v, bool):
        return ()
    if isinstance(v, int):
        return (v,)
    if isinstance(v, list):
        return tuple(int(x) for x in v if isinstance(x, int) and not isinstance(x, bool))
    return ()


@dataclass(frozen=True)
class Qwen2MoeConfig:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    qkv_bias: bool
    # feed-forward
    intermediate_size: Optional[int]
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: Optional[int]
    shared_expert_intermediate_size: int
    norm_topk_prob: bool
    routed_scaling_factor: float
    decoder_sparse_step: int
    mlp_only_layers: Tuple[int, ...]
    # attention window
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    layer_types: Optional[Tuple[str, ...]]
    # output
    tie_word_embeddings: bool
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    # ---- derived, layer by layer -------------------------------------------------
    def layer_is_sparse(self, layer: int) -> bool:
        """A layer is routed iff the model has experts, the layer is not listed
        in ``mlp_only_layers`` and ``(layer + 1) % decoder_sparse_step == 0``."""
        if self.num_experts <= 0 or layer in self.mlp_only_layers:
            return False
        return (layer + 1) % self.decoder_sparse_step == 0

    def layer_windows(self) -> List[Optional[int]]:
        """Attention window per layer, ``None`` where a layer sees everything.

        Precedence as in src/spec.rs:422-444: no (or zero) ``sliding_window`` ->
        none; an explicit ``layer_types`` list; ``use_sliding_window`` false ->
        none; else layers ``l >= max_window_layers`` get the window."""
        n = self.num_hidden_layers
        w = self.sliding_window
        if not w or w <= 0:
            return [None] * n
        if self.layer_types is not None:
            local = ("sliding_attention", "local_attention")
            return [w if (l < len(self.layer_types) and self.layer_types[l] in local) else None for l in range(n)]
        if not self.use_sliding_window:
            return [None] * n
        return [w if l >= self.max_window_layers else None for l in range(n)]

    # ---- parsing -----------------------------------------------------------------
    @staticmethod
    def from_dict(cfg: Dict[str, Any]) -> "Qwen2MoeConfig":
        hidden = _need(cfg, "hidden_size")
        heads = _need(cfg, "num_attention_heads")
        layers = _need(cfg, "num_hidden_layers")
        vocab = _need(cfg, "vocab_size")
        kv_heads = _opt(cfg, "num_key_value_heads", int, heads)
        if heads <= 0 or kv_heads <= 0 or layers <= 0 or vocab <= 0 or hidden <= 0:
            raise ConfigError(f"{ARCHITECTURE}: sizes must be positive")
        if "head_dim" in cfg and cfg["head_dim"] is not None:
            head_dim = _typed(cfg, "head_dim", int)
        else:
            if hidden % heads:
                raise ConfigError(
                    f"{ARCHITECTURE}: hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                    "and no head_dim is given"
                )
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(
                f"{ARCHITECTURE}: num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}"
            )
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"{ARCHITECTURE}: head_dim {head_dim} must be even (rotary pairs)")

        num_experts = _opt(cfg, "num_experts", int, 0)
        top_k = _opt(cfg, "num_experts_per_tok", int, 2)
        sparse_step = _opt(cfg, "decoder_sparse_step", int, 1)
        if sparse_step <= 0:
            raise ConfigError(f"{ARCHITECTURE}: decoder_sparse_step must be >= 1")
        mlp_only = cfg.get("mlp_only_layers") or []
        if not isinstance(mlp_only, list) or any(isinstance(x, bool) or not isinstance(x, int) for x in mlp_only):
            raise ConfigError(f"{ARCHITECTURE}: mlp_only_layers must be a list of layer indices")
        for x in mlp_only:
            if not 0 <= x < layers:
                raise ConfigError(f"{ARCHITECTURE}: mlp_only_layers names layer {x} of {layers}")

        layer_types = cfg.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, list) or any(not isinstance(t, str) for t in layer_types):
                raise ConfigError(f"{ARCHITECTURE}: layer_types must be a list of strings")
            layer_types = tuple(layer_types)

        c = Qwen2MoeConfig(
            vocab_size=vocab,
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=_opt(cfg, "rms_norm_eps", float, 1e-6),
            rope_theta=_opt(cfg, "rope_theta", float, 10000.0),
            max_position_embeddings=_opt(cfg, "max_position_embeddings", int, 8192),
            qkv_bias=_opt(cfg, "qkv_bias", bool, True),
            intermediate_size=_opt(cfg, "intermediate_size", int, None),
            num_experts=num_experts,
            num_experts_per_tok=top_k,
            moe_intermediate_size=_opt(cfg, "moe_intermediate_size", int, None),
            shared_expert_intermediate_size=_opt(cfg, "shared_expert_intermediate_size", int, 0),
            norm_topk_prob=_opt(cfg, "norm_topk_prob", bool, False),
            routed_scaling_factor=_opt(cfg, "routed_scaling_factor", float, 1.0),
            decoder_sparse_step=sparse_step,
            mlp_only_layers=tuple(sorted(set(mlp_only))),
            use_sliding_window=_opt(cfg, "use_sliding_window", bool, False),
            sliding_window=_opt(cfg, "sliding_window", int, None),
            max_window_layers=_opt(cfg, "max_window_layers", int, 0),
            layer_types=layer_types,
            tie_word_embeddings=_opt(cfg, "tie_word_embeddings", bool, False),
            eos_token_ids=_ids(cfg, "eos_token_id"),
            bos_token_id=(_ids(cfg, "bos_token_id") or (None,))[0],
        )
        any_sparse = any(c.layer_is_sparse(l) for l in range(layers))
        any_dense = any(not c.layer_is_sparse(l) for l in range(layers))
        if any_sparse:
            if c.moe_intermediate_size is None or c.moe_intermediate_size <= 0:
                raise ConfigError(f"{ARCHITECTURE}: routed layers need 'moe_intermediate_size'")
            if not 0 < top_k <= num_experts:
                raise ConfigError(
                    f"{ARCHITECTURE}: num_experts_per_tok {top_k} must lie in 1..num_experts ({num_experts})"
                )
            if c.shared_expert_intermediate_size < 0:
                raise ConfigError(f"{ARCHITECTURE}: shared_expert_intermediate_size must be >= 0")
        if any_dense and (c.intermediate_size is None or c.intermediate_size <= 0):
            raise ConfigError(f"{ARCHITECTURE}: dense layers need 'intermediate_size'")
        if c.rms_norm_eps <= 0 or c.rope_theta <= 0:
            raise ConfigError(f"{ARCHITECTURE}: rms_norm_eps and rope_theta must be positive")
        for e in c.eos_token_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"{ARCHITECTURE}: eos_token_id {e} outside the vocabulary of {vocab}")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen2_moe",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "qkv_bias": self.qkv_bias,
            "num_experts": self.num_experts,
            "num_experts_per_tok": self.num_experts_per_tok,
            "shared_expert_intermediate_size": self.shared_expert_intermediate_size,
            "norm_topk_prob": self.norm_topk_prob,
            "routed_scaling_factor": self.routed_scaling_factor,
            "decoder_sparse_step": self.decoder_sparse_step,
            "mlp_only_layers": list(self.mlp_only_layers),
            "use_sliding_window": self.use_sliding_window,
            "max_window_layers": self.max_window_layers,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.intermediate_size is not None:
            d["intermediate_size"] = self.intermediate_size
        if self.moe_intermediate_size is not None:
            d["moe_intermediate_size"] = self.moe_intermediate_size
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d


def model_spec(c: Qwen2MoeConfig) -> ModelSpec:
    """Translate the configuration into parts, layer by layer.

    Tensor names are the checkpoint's (src/model.rs:343-350, 370-379, 416-463)."""
    windows = c.layer_windows()
    rope = {"kind": "rotary", "theta": c.rope_theta, "rotary_dim": c.head_dim}
    layers = []
    for l in range(c.num_hidden_layers):
        p = f"model.layers.{l}."
        norm = lambda name: PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.rms_norm_eps}, p + name + ".")
        mixer = PartSpec(
            "gqa_attention",
            {
                "hidden_size": c.hidden_size,
                "num_heads": c.num_attention_heads,
                "num_kv_heads": c.num_key_value_heads,
                "head_dim": c.head_dim,
                "qkv_bias": c.qkv_bias,
                "window": windows[l],
                "position": dict(rope),
            },
            p + "self_attn.",
        )
        if c.layer_is_sparse(l):
            ffn = PartSpec(
                "routed_experts",
                {
                    "hidden_size": c.hidden_size,
                    "num_experts": c.num_experts,
                    "top_k": c.num_experts_per_tok,
                    "expert_size": c.moe_intermediate_size,
                    "norm_topk_prob": c.norm_topk_prob,
                    "routed_scaling_factor": c.routed_scaling_factor,
                    "shared_size": c.shared_expert_intermediate_size,
                    "shared_gate": c.shared_expert_intermediate_size > 0,
                },
                p + "mlp.",
            )
        else:
            ffn = PartSpec("dense_swiglu", {"hidden_size": c.hidden_size, "size": c.intermediate_size}, p + "mlp.")
        layers.append(
            LayerSpec("prenorm", norm("input_layernorm"), mixer, norm("post_attention_layernorm"), ffn)
        )
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size},
                           "model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(l, l, True) for l in range(c.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.rms_norm_eps}, "model.norm."),
        head=PartSpec(
            "lm_head",
            {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size, "tied": c.tie_word_embeddings},
            "lm_head.",
        ),
        eos_token_ids=c.eos_token_ids,
        bos_token_id=c.bos_token_id,
        max_position_embeddings=c.max_position_embeddings,
        ignorable=("*.rotary_emb.inv_freq",) + (("lm_head.weight",) if c.tie_word_embeddings else ()),
    )


register_architecture(
    Architecture(ARCHITECTURE, Qwen2MoeConfig.from_dict, model_spec, Qwen2MoeConfig.to_dict),
    model_types=("qwen2_moe",),
)

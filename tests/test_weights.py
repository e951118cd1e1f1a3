"""Weights by tensor name, the dtype policy and the one error message (CPU)."""
import json
import os
import struct

import pytest
import torch

import helpers
import plain_qwen2moe as plain
from moe_b200.config import parse_config
from moe_b200.models import expected_tensors
from moe_b200.weights import SafetensorsError, SafetensorsStore, WeightError, write_safetensors
from moe_b200.weights.store import convert_for_compute


def _expected(cfg):
    arch, typed = parse_config(cfg)
    spec = arch.model_spec(typed)
    return spec, {n: t.shape for n, t in expected_tensors(spec).items()}


def test_random_model_folder_has_every_tensor_with_its_shape(model_dirs):
    for name, cfg in helpers.CONFIGS.items():
        d = model_dirs.get(name, "bfloat16", seed=3)
        assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
        spec, exp = _expected(cfg)
        store = SafetensorsStore(d)
        store.check(exp, spec.ignorable)
        assert set(store.names()) == set(exp)
        assert all(store.stored_dtype(n) == torch.bfloat16 for n in exp)
    # tied: no lm_head tensor; untied: one
    assert "lm_head.weight" not in _expected(helpers.CONFIG_B)[1]
    assert "lm_head.weight" in _expected(helpers.CONFIG_A)[1]


def test_seed_decides_the_weights(model_dirs):
    a = SafetensorsStore(model_dirs.get("A", "float32", seed=0))
    b = SafetensorsStore(model_dirs.get("A", "float32", seed=0, overrides={"max_position_embeddings": 4097}))
    c = SafetensorsStore(model_dirs.get("A", "float32", seed=1))
    n = "model.layers.1.mlp.experts.2.up_proj.weight"
    assert torch.equal(a.raw(n), b.raw(n)) and not torch.equal(a.raw(n), c.raw(n))
    assert torch.all(a.raw("model.norm.weight") == 1)
    assert 0.015 < float(a.raw("model.embed_tokens.weight").std()) < 0.025


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, model_dirs):
    src = SafetensorsStore(model_dirs.get("A", "float32", seed=0))
    tensors = {n: src.raw(n).clone() for n in src.names()}
    del tensors["model.layers.0.self_attn.k_proj.bias"]
    del tensors["model.layers.1.mlp.shared_expert_gate.weight"]
    tensors["model.layers.0.mlp.experts.9.up_proj.weight"] = torch.zeros(2, 2)
    tensors["model.layers.1.self_attn.o_proj.weight"] = torch.zeros(64, 32)
    d = tmp_path / "broken"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(helpers.CONFIG_A))
    write_safetensors(str(d / "model.safetensors"), tensors)
    spec, exp = _expected(helpers.CONFIG_A)
    with pytest.raises(WeightError) as e:
        SafetensorsStore(str(d)).check(exp, spec.ignorable)
    err = e.value
    assert err.missing == ["model.layers.0.self_attn.k_proj.bias", "model.layers.1.mlp.shared_expert_gate.weight"]
    assert err.unexpected == ["model.layers.0.mlp.experts.9.up_proj.weight"]
    assert err.wrong_shape == [("model.layers.1.self_attn.o_proj.weight", (64, 32), (64, 64))]
    msg = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "k_proj.bias", "experts.9", "[64, 32]"):
        assert needle in msg


def test_ignorable_names_and_integer_weights(tmp_path, model_dirs):
    src = SafetensorsStore(model_dirs.get("B", "float32", seed=0))
    tensors = {n: src.raw(n).clone() for n in src.names()}
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()   # tied model that stores both
    d = tmp_path / "extra"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors)
    spec, exp = _expected(helpers.CONFIG_B)
    SafetensorsStore(str(d)).check(exp, spec.ignorable)
    tensors["model.norm.weight"] = torch.ones(96, dtype=torch.int32)
    write_safetensors(str(d / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        SafetensorsStore(str(d)).check(exp, spec.ignorable)
    assert e.value.wrong_dtype


def test_dtype_policy():
    bf, f32, f16 = torch.ones(2, dtype=torch.bfloat16), torch.ones(2), torch.ones(2, dtype=torch.float16)
    i64 = torch.ones(2, dtype=torch.int64)
    # bfloat16 compute: bf16 stays, 32-bit stays, f16 widens exactly, integers become int32
    assert convert_for_compute(bf, torch.bfloat16).dtype == torch.bfloat16
    assert convert_for_compute(f32, torch.bfloat16).dtype == torch.float32
    assert convert_for_compute(f16, torch.bfloat16).dtype == torch.float32
    assert convert_for_compute(i64, torch.bfloat16).dtype == torch.int32
    # float32 compute: everything floating widens
    assert convert_for_compute(bf, torch.float32).dtype == torch.float32
    x = torch.randn(64).to(torch.bfloat16)
    assert torch.equal(convert_for_compute(x, torch.float32), x.float())


def test_malformed_files_are_refused(tmp_path):
    """Header length and byte ranges are checked before anything is sliced (src/store.rs:80-119)."""
    d = tmp_path / "m"
    d.mkdir()
    with pytest.raises(SafetensorsError):
        SafetensorsStore(str(d))                       # no .safetensors files
    p = d / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        SafetensorsStore(str(d))                       # truncated
    p.write_bytes(struct.pack("<Q", 1 << 60) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsStore(str(d))                       # header longer than the file
    head = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsStore(str(d))                       # data runs past the file
    head = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsStore(str(d))                       # offsets disagree with the shape
    p.write_bytes(struct.pack("<Q", 5) + b"[1,2]")
    with pytest.raises(SafetensorsError):
        SafetensorsStore(str(d))                       # header not an object


def test_writer_and_plain_reader_agree(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "z.w": torch.randn(2, 2, 2)}
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    got = plain.read_safetensors(str(tmp_path / "model.safetensors"))
    for n in t:
        assert torch.equal(got[n], t[n].double())
    s = SafetensorsStore(str(tmp_path))
    assert torch.equal(s.raw("a"), t["a"]) and s.shape("z.w") == (2, 2, 2)


def _restacked(src: SafetensorsStore, cfg, form: str):
    """The same weights with every routed layer's experts in another checkpoint layout
    (src/model.rs:396-420): "fused" gate_up_proj [E, 2 size, hidden] + down_proj [E, hidden, size];
    "stacked" three tensors of three dimensions."""
    out = {}
    E = cfg["num_experts"]
    per_expert = {}
    for n in src.names():
        parts = n.split(".")
        if ".mlp.experts." in n:
            layer = ".".join(parts[:3])
            per_expert.setdefault(layer, {})[(int(parts[5]), parts[6])] = src.raw(n)
        else:
            out[n] = src.raw(n).clone()
    for layer, t in per_expert.items():
        g = torch.stack([t[(e, "gate_proj")] for e in range(E)])
        u = torch.stack([t[(e, "up_proj")] for e in range(E)])
        dn = torch.stack([t[(e, "down_proj")] for e in range(E)])
        if form == "fused":
            out[f"{layer}.mlp.experts.gate_up_proj"] = torch.cat([g, u], dim=1)
        else:
            out[f"{layer}.mlp.experts.gate_proj"], out[f"{layer}.mlp.experts.up_proj"] = g, u
        out[f"{layer}.mlp.experts.down_proj"] = dn
    return out


@pytest.mark.parametrize("form", ["fused", "stacked"])
def test_fused_and_stacked_expert_layouts_load_to_the_same_model(tmp_path, model_dirs, form):
    import moe_b200

    base = model_dirs.get("B", "float32", seed=2)
    d = tmp_path / form
    d.mkdir()
    (d / "config.json").write_text(json.dumps(helpers.CONFIG_B))
    write_safetensors(str(d / "model.safetensors"), _restacked(SafetensorsStore(base), helpers.CONFIG_B, form))
    a = moe_b200.load_model(base, dtype="float32", device="cpu")
    b = moe_b200.load_model(str(d), dtype="float32", device="cpu")
    fa, fb = a.blocks[1].ffn, b.blocks[1].ffn
    assert fa.w_gu.shape == (8, 96, 96) and torch.equal(fa.w_gu, fb.w_gu) and torch.equal(fa.w_down, fb.w_down)
    assert torch.equal(fa.ws_gu, fb.ws_gu) and torch.equal(fa.w_router, fb.w_router)
    # a wrong shape in that layout is reported by its own name
    broken = _restacked(SafetensorsStore(base), helpers.CONFIG_B, form)
    broken["model.layers.1.mlp.experts.down_proj"] = torch.zeros(8, 96, 47)
    write_safetensors(str(d / "model.safetensors"), broken)
    with pytest.raises(WeightError) as e:
        moe_b200.load_model(str(d), dtype="float32", device="cpu")
    assert "model.layers.1.mlp.experts.down_proj is [8, 96, 47], expected [8, 96, 48]" in str(e.value)


def test_weights_drawn_when_asked_for_equal_those_drawn_at_once():
    import moe_b200
    from moe_b200.weights import RandomStore, random_tensors

    arch, typed = parse_config(helpers.CONFIG_B)
    spec = arch.model_spec(typed)
    at_once = random_tensors(spec, 5, 0.05, "bfloat16", "cpu")
    store = RandomStore(spec, 5, 0.05, "bfloat16", "cpu")
    assert set(store.names()) == set(at_once)
    for n in list(at_once)[::7] + list(at_once)[:3]:          # in another order than they were drawn at once
        assert torch.equal(store.raw(n), at_once[n]) and store.shape(n) == tuple(at_once[n].shape)
    m = moe_b200.random_model(helpers.CONFIG_B, seed=5, dtype="bfloat16", device="cpu", std=0.05)
    assert torch.equal(m.blocks[1].ffn.w_gu[3, 48:], at_once["model.layers.1.mlp.experts.3.up_proj.weight"])
    assert torch.equal(m.blocks[0].mixer.wqkv[96:128], at_once["model.layers.0.self_attn.k_proj.weight"])


def test_mutated_files_load_or_are_refused_never_anything_else(tmp_path):
    """A sweep in the manner of the reference's malformed-input tests (tests/malformed.rs, fuzz/):
    bytes of a valid file's length word and header are flipped, cut or repeated; every result is
    either a store whose tensors can all be read or ONE of the loader's own errors."""
    import random

    tensors = {"a.weight": torch.arange(12, dtype=torch.float32).reshape(3, 4),
               "b.weight": torch.ones(5, dtype=torch.bfloat16), "c": torch.zeros(2, 2, dtype=torch.float16)}
    src = tmp_path / "src"
    src.mkdir()
    write_safetensors(str(src / "model.safetensors"), tensors)
    good = (src / "model.safetensors").read_bytes()
    head_len = struct.unpack("<Q", good[:8])[0]
    rng = random.Random(7)
    d = tmp_path / "mut"
    d.mkdir()
    loaded = refused = 0
    for trial in range(400):
        b = bytearray(good)
        kind = trial % 4
        if kind == 0:                                   # flip bytes in the length word or the header
            for _ in range(rng.randint(1, 4)):
                i = rng.randrange(0, 8 + head_len)
                b[i] = rng.randrange(256)
        elif kind == 1:                                 # cut the file somewhere
            b = b[:rng.randrange(0, len(b))]
        elif kind == 2:                                 # a digit of the header becomes another digit
            digits = [i for i in range(8, 8 + head_len) if chr(b[i]).isdigit()]
            b[rng.choice(digits)] = ord(str(rng.randrange(10)))
        else:                                           # a stretch of the header is repeated or dropped
            i, j = sorted(rng.sample(range(8, 8 + head_len), 2))
            b = b[:i] + (b[i:j] * 2 if trial % 8 == 3 else b"") + b[j:]
        (d / "model.safetensors").write_bytes(bytes(b))
        try:
            st = SafetensorsStore(str(d))
            for name in st.names():
                st.get(name, torch.float32)
            loaded += 1
        except (SafetensorsError, WeightError):
            refused += 1
    assert loaded + refused == 400 and refused > 200 and loaded > 0

"""Each part of a layer alone, built from its PartSpec with random tensors, against the plain
function of the same part.  Sizes differ from both tiny configurations."""
import pytest
import torch

import gpu_util as G
import plain_qwen2moe as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def build(category, kind, params, dtype, std=0.3, seed=0):
    """(bound part, its tensors as float64 CPU tensors under their local names, runtime)."""
    from moe_b200.config.spec import PartSpec
    from moe_b200.parts import Runtime, make_part

    rt = Runtime(DEV, dtype)
    part = make_part(category, PartSpec(kind, params, "x."))
    g = torch.Generator().manual_seed(seed)
    store_dt = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    tensors, ref = {}, {}
    for name, ts in part.tensors().items():
        t = torch.randn(ts.shape, generator=g) * std + (1.0 if ts.init == "ones" else 0.0)
        t = t.to(store_dt)
        tensors[name] = t.to(DEV)
        ref[name] = t.double()
    part.bind(dict(tensors), rt)
    return part, ref, rt


def acts(rt, x):
    from moe_b200.parts import Activations

    x = x.to(DEV)
    if rt.is_bf16:
        return Activations(act=x.to(torch.bfloat16).contiguous(), f32=x.float().contiguous())
    return Activations(act=x.float().contiguous(), f32=x.float().contiguous())


DTYPES = [torch.float32, torch.bfloat16]


def tol(dt):
    return 2e-5 if dt == torch.float32 else 2e-2


def rel(got, ref):
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max())


@pytest.mark.parametrize("dt", DTYPES)
def test_rmsnorm_part(dt):
    part, ref, rt = build("norm", "rmsnorm", {"size": 120, "eps": 1e-5}, dt)
    x = torch.randn(9, 120)
    h = part.forward(rt, x.to(DEV).contiguous(), want32=True)
    want = plain.rmsnorm(x.double(), ref["weight"], 1e-5)
    assert rel(h.f32, want) < 2e-6
    assert h.act.dtype == dt and rel(h.act, want) < tol(dt)


def test_rotary_part_table():
    part, _, rt = build("position", "rotary", {"theta": 1e6, "rotary_dim": 48}, torch.float32)
    table, rot = part.rotary_table()
    assert rot == 48 and torch.equal(table.cpu(), plain.rope_inv_freq(1e6, 48))
    assert part.attention_scale() == 1.0


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window,bias", [(6, 2, 48, None, True), (5, 1, 16, 5, False), (2, 2, 64, 70, True)])
def test_attention_part_prefill_then_decode(dt, nh, nkv, hd, window, bias):
    from moe_b200.cache import KVCache

    H = 88
    params = {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qkv_bias": bias,
              "window": window, "position": {"kind": "rotary", "theta": 1e4, "rotary_dim": hd}}
    part, ref, rt = build("mixer", "gqa_attention", params, dt)
    cache = KVCache({0: part.kv_request()}, {0: None}, 1024, 2, dt, DEV)
    slot = cache.acquire()
    T, D = 90, 6
    x = torch.randn(T + D, H)
    if dt == torch.bfloat16:
        x = x.to(torch.bfloat16).float()
    cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, rope_theta=1e4)
    w = {"p.self_attn." + k: v for k, v in ref.items()}
    want = plain.attention_block(cfg, w, "p.", x.double(), torch.arange(T + D), window)
    G.give_pages(cache, slot, T)
    got = [part.forward(rt, acts(rt, x[:T]), G.make_batch(DEV, [slot], [0], [T]), cache.view(0))]
    for i in range(D):
        G.give_pages(cache, slot, T + i + 1)
        got.append(part.forward(rt, acts(rt, x[T + i:T + i + 1]), G.make_batch(DEV, [slot], [T + i], [1]),
                                cache.view(0)))
    got = torch.cat(got)
    assert got.dtype == torch.float32 and rel(got, want) < tol(dt)
    assert int(rt.status[0]) == 0


@pytest.mark.parametrize("dt", DTYPES)
def test_dense_swiglu_part(dt):
    part, ref, rt = build("ffn", "dense_swiglu", {"hidden_size": 72, "size": 200}, dt)
    x = torch.randn(13, 72)
    if dt == torch.bfloat16:
        x = x.to(torch.bfloat16).float()
    got = part.forward(rt, acts(rt, x), None)
    want = plain.swiglu_mlp({"m." + k: v for k, v in ref.items()}, "m.", x.double())
    assert rel(got, want) < tol(dt)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("E,k,norm,shared,scale", [(6, 2, False, 40, 1.0), (12, 5, True, 0, 2.0), (3, 3, True, 24, 1.0)])
def test_routed_experts_part(dt, E, k, norm, shared, scale):
    H, I, T = 56, 24, 41
    params = {"hidden_size": H, "num_experts": E, "top_k": k, "expert_size": I, "norm_topk_prob": norm,
              "routed_scaling_factor": scale, "shared_size": shared, "shared_gate": shared > 0}
    part, ref, rt = build("ffn", "routed_experts", params, dt)
    x = torch.randn(T, H)
    if dt == torch.bfloat16:
        x = x.to(torch.bfloat16).float()
    part.trace = []
    got = part.forward(rt, acts(rt, x), G.make_batch(DEV, [0], [0], [T]))
    picks = part.trace[0][0].cpu().tolist()
    cfg = dict(num_experts_per_tok=k, norm_topk_prob=norm, routed_scaling_factor=scale)
    w = {"p.mlp." + n: v for n, v in ref.items()}
    free = []
    plain.moe_block(cfg, w, "p.", x.double(), trace=free)
    want = plain.moe_block(cfg, w, "p.", x.double(), forced=picks)
    assert rel(got, want) < tol(dt)
    same = sum(sorted(a) == sorted(b) for a, b in zip(picks, free[0][0]))
    assert same >= T - (0 if dt == torch.float32 else 1)      # the router reads the 32-bit state in both paths
    assert int(rt.status[0]) == 0


@pytest.mark.parametrize("dt", DTYPES)
def test_embedding_and_head_parts(dt):
    emb, ref, rt = build("embedding", "token_embedding", {"vocab_size": 77, "hidden_size": 40}, dt)
    ids = torch.tensor([0, 76, 5, 5], dtype=torch.int32, device=DEV)
    x = emb.forward(rt, ids, 4)
    assert x.dtype == torch.float32 and torch.equal(x.cpu().double(), ref["weight"][ids.cpu().long()])
    from moe_b200.config.spec import PartSpec
    from moe_b200.parts import make_part

    tied = make_part("head", PartSpec("lm_head", {"vocab_size": 77, "hidden_size": 40, "tied": True}, "lm_head."))
    assert tied.tensors() == {}
    tied.bind({}, rt, embedding=emb)
    h = torch.randn(3, 40)
    if dt == torch.bfloat16:
        h = h.to(torch.bfloat16).float()
    got = tied.forward(rt, acts(rt, h))
    assert got.shape == (3, 77) and rel(got, h.double() @ ref["weight"].T) < tol(dt)
    untied, ref2, _ = build("head", "lm_head", {"vocab_size": 77, "hidden_size": 40, "tied": False}, dt)
    assert rel(untied.forward(rt, acts(rt, h)), h.double() @ ref2["weight"].T) < tol(dt)


@pytest.mark.parametrize("dt", DTYPES)
def test_prenorm_block(dt):
    """norm -> mixer -> residual -> norm -> feed-forward, the second sum left pending."""
    from moe_b200.cache import KVCache
    from moe_b200.config.spec import LayerSpec, PartSpec
    from moe_b200.parts import Runtime, make_block

    H, nh, nkv, hd, I, T = 64, 2, 1, 32, 96, 17
    layer = LayerSpec(
        "prenorm",
        PartSpec("rmsnorm", {"size": H, "eps": 1e-6}, "n1."),
        PartSpec("gqa_attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
                                   "qkv_bias": True, "window": None,
                                   "position": {"kind": "rotary", "theta": 1e4, "rotary_dim": hd}}, "a."),
        PartSpec("rmsnorm", {"size": H, "eps": 1e-6}, "n2."),
        PartSpec("dense_swiglu", {"hidden_size": H, "size": I}, "f."),
    )
    rt = Runtime(DEV, dt)
    blk = make_block(layer)
    g = torch.Generator().manual_seed(3)
    w = {}
    for part in blk.parts():
        tensors = {}
        for name, ts in part.tensors().items():
            t = (torch.randn(ts.shape, generator=g) * 0.2 + (1.0 if ts.init == "ones" else 0.0))
            t = t.to(torch.bfloat16 if dt == torch.bfloat16 else torch.float32)
            tensors[name] = t.to(DEV)
            w[part.spec.prefix + name] = t.double()
        part.bind(tensors, rt)
    cache = KVCache({0: blk.mixer.kv_request()}, {0: None}, 256, 1, dt, DEV)
    slot = cache.acquire()
    G.give_pages(cache, slot, T)
    x0 = torch.randn(T, H)
    pend0 = torch.randn(T, H) * 0.1
    x = x0.to(DEV).contiguous()
    x, pending = blk.forward(rt, x, pend0.to(DEV).contiguous(), G.make_batch(DEV, [slot], [0], [T]), cache.view(0), None)
    # plain
    xs = x0.double() + pend0.double()
    pw = {"p.self_attn." + k[2:]: v for k, v in w.items() if k.startswith("a.")}
    n = plain.rmsnorm(xs, w["n1.weight"], 1e-6)
    xs = xs + plain.attention_block(dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd,
                                         rope_theta=1e4), pw, "p.", n, torch.arange(T), None)
    n = plain.rmsnorm(xs, w["n2.weight"], 1e-6)
    want_pending = plain.swiglu_mlp({"m." + k[2:]: v for k, v in w.items() if k.startswith("f.")}, "m.", n)
    assert rel(x, xs) < tol(dt) and rel(pending, want_pending) < tol(dt)

"""The command line's pieces that need no GPU: ``moe info`` for a folder, for ``--random`` and for
architectures registered from outside, and the byte count of a decode step."""
import json

import pytest

import helpers


def run_info(capsys, *argv):
    from moe_b200 import cli

    assert cli.main(["info", *argv]) == 0
    return capsys.readouterr().out


def test_info_describes_the_model_in_the_words_of_its_parts(model_dirs, capsys):
    out = run_info(capsys, model_dirs.get("B", "float32", seed=1, std=0.2), "--dtype", "float32")
    assert "Qwen2MoeForCausalLM" in out and "layers 3  hidden 96  vocab 384" in out
    assert "GQA(3 q / 1 kv heads, head_dim=32, bias), rope theta 1000000, window 8   (2 of 3)" in out
    assert "dense SwiGLU 160   (2 of 3)" in out
    assert "8 experts of 48, top-3, softmax gate, renormalised, shared expert 128 (gated)   (1 of 3)" in out
    assert "output projection (the embedding)" in out
    # layers 1 (the only routed one): 8 experts x 3 x 48 x 96 values of 4 bytes
    assert "experts  432.00 KB" in out and "kv cache   768.00 KB per 1k tokens" in out


def test_info_with_random_weights_needs_no_folder(tmp_path, capsys):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(helpers.CONFIG_A))
    out = run_info(capsys, "--random", str(cfg), "--seed", "3")
    assert "4 experts of 32, top-2" in out and "random weights of" in out


def test_info_on_architectures_registered_from_outside(tmp_path, capsys):
    """Nothing in the summary knows a kind of part: a model whose mixers are not attention prints too."""
    import moe_b200
    import test_extend_gpu as X

    X.register_toy()
    X.register_toy_switch()
    d = str(tmp_path / "toy")
    moe_b200.write_random_model(d, X.TOY, seed=3, dtype="float32")
    out = run_info(capsys, d, "--dtype", "float32")
    assert "ToyDecayForCausalLM" in out and "toy_decay" in out and "reads another layer's cache" in out
    assert "schedule   0 1 2[cache 0, read] 1[cache 2]" in out
    assert "state      384 B per sequence" in out          # 48 floats for each of the stateful layer's two runs
    d2 = str(tmp_path / "switch")
    moe_b200.write_random_model(d2, X.SWITCH, seed=3, dtype="float32")
    out = run_info(capsys, d2, "--dtype", "float32")
    assert "toy_switch" in out and "window 6" in out and "on 16 dims" not in out


def test_bytes_of_a_decode_step(model_dirs):
    import moe_b200
    from moe_b200 import cli

    m = moe_b200.load_model(model_dirs.get("A", "float32", seed=1, std=0.2), dtype="float32", device="cpu")
    c = helpers.CONFIG_A
    H, mi, si, E, k = 64, 32, 64, 4, 2
    attn = (4 + 2 * 2) * 16 * H + (4 + 2 * 2) * 16 + H * 4 * 16
    for B in (1, 3):
        touched = E * (1 - (1 - k / E) ** B)
        layer = attn + 2 * H + E * H + 3 * si * H + H + touched * 3 * mi * H
        want = 4 * (2 * layer + B * H + H + 256 * H)
        w, kv = cli.step_bytes(m, [10] * B)
        assert w == pytest.approx(want)
        assert kv == 2 * B * 10 * 2 * 2 * 16 * 4
    # a window bounds what is read from the cache
    mb = moe_b200.load_model(model_dirs.get("B", "float32", seed=1, std=0.2), dtype="float32", device="cpu")
    _, kv = cli.step_bytes(mb, [100])
    assert kv == (100 + 8 + 8) * 2 * 1 * 32 * 4

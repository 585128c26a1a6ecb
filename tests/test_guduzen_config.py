"""The Guduzen configuration without a GPU: reading config.json, what it refuses, the model it describes (parts,
schedule, cache needs, checkpoint names), and the plain implementation's own pieces."""
import copy
import json

import pytest
import torch

import plain_guduzen as plain
from gpullama3.java_b200.cache.sequence_cache import KVCacheNeed, StateNeed
from gpullama3.java_b200.config import ConfigError, config_from_dict, load_config
from gpullama3.java_b200.engine.model import CausalLM
from guduzen_helpers import CONFIGS, GUDUZEN_A, GUDUZEN_B, make_guduzen_dir, plain_inputs


def test_the_architecture_is_found_under_either_key():
    a = config_from_dict(GUDUZEN_A)
    d = dict(GUDUZEN_A)
    d["architectures"] = [d.pop("architecture")]
    assert config_from_dict(d) == a
    assert config_from_dict(a.to_dict()) == a


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_model_structure(name):
    cfg = config_from_dict(CONFIGS[name])
    model = CausalLM(cfg, torch.float32, "cpu")
    assert set(model.parameter_specs()) == set(cfg.tensor_names())
    assert model.streams == CONFIGS[name].get("streams")
    assert not model.pad_safe and model.graph_safe      # a recurrent state takes no padding; every launch is replayable
    for i, L in enumerate(CONFIGS[name]["layers"]):
        block = model.blocks[i]
        assert (block.feed_forward is None) == (L["mlp"] is None)
        need = block.cache_need()
        assert isinstance(need, StateNeed if L["type"] == "channel_delta" else KVCacheNeed)


def test_shared_caches_and_windows():
    cfg = config_from_dict(GUDUZEN_A)
    sched = cfg.schedule()
    assert [(e.cache, e.writes_cache) for e in sched] == [(0, True), (1, True), (2, True), (1, False), (4, True)]
    model = CausalLM(cfg, torch.float32, "cpu")
    writer, reader = model.blocks[1].mixer, model.blocks[3].mixer
    assert (writer.window, reader.window) == (20, 33)
    assert writer.cache_need() == reader.cache_need() and writer.cache_need().window == 33   # the longer of the two
    assert "k" not in reader.parameters() and "q_bias" in reader.parameters()
    # heads of 24 and values of 16 are widened to one size the kernels take; the latent of 40 to 64
    assert writer.head_dim == 32 and model.blocks[2].mixer.cache_need() == KVCacheNeed(1, 64, None)
    b = CausalLM(config_from_dict(GUDUZEN_B), torch.float32, "cpu")
    assert b.blocks[1].mixer.cache_need().window is None and b.blocks[4].mixer.window == 9


@pytest.mark.parametrize("change, match", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "unknown mixer type"),
    (lambda d: d["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("heads", 8), "differ"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda d: d["layers"][2].__setitem__("mlp", {"kind": "routed", "ff": 8}), "mlp"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.__setitem__("streams", 0), "streams"),
])
def test_what_the_configuration_refuses(change, match):
    d = copy.deepcopy(GUDUZEN_A)
    change(d)
    with pytest.raises(ConfigError, match=match):
        CausalLM(config_from_dict(d), torch.float32, "cpu")


def test_ranks_come_from_the_checkpoint(tmp_path):
    """A folder whose config.json does not give the low-rank sizes of the delta mixer loads all the same."""
    from gpullama3.java_b200.weights.loader import load_checkpoint_tensors
    from gpullama3.java_b200.weights.safetensors_io import WeightError

    d = make_guduzen_dir(tmp_path, GUDUZEN_A, seed=1)
    raw = json.loads((d / "config.json").read_text())
    for L in raw["layers"]:
        L["mixer"].pop("a_rank", None)
        L["mixer"].pop("g_rank", None)
    (d / "config.json").write_text(json.dumps(raw))
    cfg = load_config(d)
    model = CausalLM(cfg, torch.float32, "cpu")
    expected = {n: s.shape for n, s in model.checkpoint_specs().items()}
    assert expected["l0.mix.a1"] == (-1, 64) and expected["l0.mix.g2"] == (4 * 24, -1)
    tensors = load_checkpoint_tensors(d, expected, torch.float32)
    assert tensors["l0.mix.a1"].shape == (8, 64) and tensors["l0.mix.g2"].shape == (96, 16)
    expected["l0.mix.a1"] = (-1, 65)
    with pytest.raises(WeightError, match="wrong shape"):
        load_checkpoint_tensors(d, expected, torch.float32)


def test_plain_pieces():
    g = torch.Generator().manual_seed(0)
    # the convolution is causal: changing a later input leaves earlier outputs alone; taps = 1 is a plain scaling
    x = torch.randn(9, 5, generator=g, dtype=torch.float64)
    w = torch.randn(5, 3, generator=g, dtype=torch.float64)
    y = plain.short_convolution(x, w)
    x2 = x.clone()
    x2[6] += 1.0
    y2 = plain.short_convolution(x2, w)
    assert torch.equal(y[:6], y2[:6]) and not torch.equal(y[6], y2[6])
    z = x * w[:, :1].T
    assert torch.allclose(plain.short_convolution(x, w[:, :1]), z * torch.sigmoid(z))
    # the delta rule with g = 1, beta = 1 and orthonormal keys stores each value under its key exactly
    k = torch.eye(4, dtype=torch.float64)
    v = torch.randn(4, 3, generator=g, dtype=torch.float64)
    o = plain.delta_rule(k, k, v, torch.ones(4, dtype=torch.float64), torch.ones(4, 4, dtype=torch.float64))
    assert torch.allclose(o, v)
    # ... and writing a second value under the same key replaces the first
    o = plain.delta_rule(k[[0, 0]], k[[0, 0]], v[:2], torch.ones(2, dtype=torch.float64), torch.ones(2, 4, dtype=torch.float64))
    assert torch.allclose(o[1], v[1])
    # windows: itself and the size - 1 tokens before it
    m = plain.visible(6, 2)
    assert m[4].tolist() == [False, False, False, True, True, False] and plain.visible(3, None)[2].all()
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12


def test_one_stream_with_identity_weights_is_the_plain_residual(tmp_path):
    """streams = 1 with read = mix = write = 1 computes what a model without streams computes."""
    d = make_guduzen_dir(tmp_path, GUDUZEN_B, seed=2)
    cfg, weights = plain_inputs(d)
    with_streams = dict(cfg, streams=1)
    w2 = dict(weights)
    for i, L in enumerate(cfg["layers"]):
        for hc in ("hc1", "hc2") if L["mlp"] else ("hc1",):
            w2[f"l{i}.{hc}.in"] = torch.ones(1)
            w2[f"l{i}.{hc}.out"] = torch.ones(1)
            w2[f"l{i}.{hc}.mix"] = torch.ones(1, 1)
    tokens = list(range(3, 40))
    assert torch.allclose(plain.forward(cfg, weights, tokens), plain.forward(with_streams, w2, tokens), rtol=1e-12, atol=1e-12)

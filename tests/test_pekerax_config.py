"""The Pekerax configuration without a GPU: keys read and written back, layers turned into parts, checkpoint names and
shapes, what is refused, and the cache bookkeeping of kept first positions."""
import copy

import pytest

from gpullama3.java_b200.cache.sequence_cache import CacheSizes, KVCacheNeed, KVGroup
from gpullama3.java_b200.config import ConfigError, config_from_dict
from gpullama3.java_b200.engine.model import parameter_specs_by_checkpoint_name
from pekerax_helpers import CONFIGS, PEKERAX_A


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_parts(name):
    cfg = config_from_dict(CONFIGS[name])
    assert config_from_dict(cfg.to_dict()) == cfg
    specs = cfg.layer_specs()
    assert len(specs) == len(CONFIGS[name]["layers"])
    for spec, L in zip(specs, CONFIGS[name]["layers"]):
        assert spec.parts["mixer"].kind == {"attention": "attention", "delta": "head_delta"}[L["type"]]
        assert ("feed_forward" in spec.parts) == (L["mlp"] is not None)
        if L["mlp"] is not None:
            assert spec.parts["feed_forward"].kind == {"dense": "gated", "moe": "routed"}[L["mlp"]["kind"]]
            assert spec.parts["feed_forward"].args["activation"] == "clamped_sigmoid"
        assert spec.parts["mixer_norm"].kind == "layernorm"
    assert cfg.embedding_scale() == CONFIGS[name].get("embedding", {}).get("scale", 1.0)


def test_no_mask_means_no_window():
    d = copy.deepcopy(PEKERAX_A)
    del d["layers"][2]["mixer"]["mask"]
    args = config_from_dict(d).layer_specs()[2].parts["mixer"].args
    assert args["window"] is None and args["keep_first"] == 0


def test_value_mixing_roles():
    cfg = config_from_dict(PEKERAX_A)
    roles = [s.parts["mixer"].args.get("value_mix") for s in cfg.layer_specs()]
    assert roles == ["source", None, "mixed", "mixed", None]
    one = copy.deepcopy(PEKERAX_A)
    del one["layers"][2]["mixer"]["v_mix"], one["layers"][3]["mixer"]["v_mix"]
    assert [s.parts["mixer"].args.get("value_mix") for s in config_from_dict(one).layer_specs()][0] == "source"


def test_checkpoint_names_and_shapes():
    specs = parameter_specs_by_checkpoint_name(config_from_dict(PEKERAX_A))
    assert specs["embed"].shape == (160, 64) and specs["final.norm.b"].shape == (64,)
    assert specs["l0.mix.q.norm"].shape == (64,) and specs["l0.mix.k.norm"].shape == (32,)
    assert specs["l0.mix.sink"].shape == (4,) and specs["l0.mix.g"].shape == (4, 64) and specs["l0.mix.vmix"].shape == ()
    assert specs["l0.mix.o"].shape == (64, 96) and specs["l0.mlp.gate"].shape == (96, 64)
    assert specs["l1.mix.a"].shape == (4, 64) and specs["l1.mix.dt_bias"].shape == (4,) and specs["l1.mix.g"].shape == (96, 64)
    assert specs["l1.mix.v.conv"].shape == (96, 3) and specs["l1.mix.norm"].shape == (24,)
    assert specs["l1.mlp.router"].shape == (6, 64) and specs["l1.mlp.e5.down"].shape == (64, 32)
    assert "l2.norm2" not in specs and "l2.mlp.gate" not in specs and "l4.mix.vmix" not in specs
    assert not any(n.startswith("l1.mix.vmix") for n in specs)


@pytest.mark.parametrize("change, message", [
    (lambda d: d["layers"][0].update(type="recurrent"), "unknown mixer type"),
    (lambda d: d["layers"][0]["mixer"]["mask"].pop("size"), "missing key"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=5), "experts"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda d: d["layers"][0]["mlp"].update(limit=0.0), "positive"),
    (lambda d: d["layers"][2]["mixer"].update(vdim=16), "agree"),
    (lambda d: d["norm"].pop("eps"), "missing key"),
])
def test_refused(change, message):
    d = copy.deepcopy(PEKERAX_A)
    change(d)
    with pytest.raises(ConfigError, match=message):
        cfg = config_from_dict(d)
        parameter_specs_by_checkpoint_name(cfg)


def test_kept_first_pages_are_never_let_go():
    """A windowed group with kept first positions frees the pages behind the window except those of the kept positions,
    hands them all back at the end, and is sized for them."""
    import torch

    sizes = CacheSizes(n_pages=64, max_slots=2, dtype=torch.float32, device=torch.device("cpu"), window_slack=1024)
    for keep, kept_pages in ((0, 0), (3, 1), (64, 1), (65, 2)):
        g = KVGroup(KVCacheNeed(1, 16, window=100, keep_first=keep), [0], sizes)
        g.acquire(0)
        length = 0
        for step in (700, 1, 1, 130, 1):
            g.reserve(0, length + step)
            length += step
            g.commit(0, length)
            row = g.rows[0]
            first_needed = (length - 100 + 1) // 64
            assert all(p >= 0 for p in row[:kept_pages]) and all(p >= 0 for p in row[first_needed:])
            assert all(p < 0 for p in row[kept_pages:first_needed])
            g.check()
        g.release(0)
        assert g.pool.n_held == 0

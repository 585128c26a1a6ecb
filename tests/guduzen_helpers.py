"""Small Guduzen configurations for the tests, and model folders with random weights made so that faults show.

The three configurations differ from one another in every size and option: number of streams (2, none, 1), soft cap
or none, layer order, heads and groups, key size against value size (smaller, equal, larger), sizes that the
tensor-core kernels take (64, 128) and sizes that are widened (24 -> 32, 40 -> 64), windows shorter and longer than a
page and none at all, a reader of another layer's cache with a longer window than the writer's own, convolutions of 2
to 4 taps, delta heads that share query/key heads, more latent-attention heads than one decode launch takes, layers without
feed-forward.  Score scales are large, so attention
is peaked and one key that is wrongly seen or missed moves the logits."""
from __future__ import annotations

import json
from pathlib import Path

import torch

GUDUZEN_A = {
    "architecture": "Guduzen", "vocab": 160, "width": 64, "streams": 2, "logit_softcap": 20.0, "norm": {"eps": 1e-5},
    "initializer_range": 0.08,
    "layers": [
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 3, "a_rank": 8, "g_rank": 16}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 4, "kv_heads": 4, "dim": 24, "vdim": 16, "scale": 0.9, "mask": {"size": 20}}},
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 2, "dim": 16, "vdim": 24, "kv_rank": 40, "q_rank": 24, "scale": 1.1}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 80},
         "mixer": {"heads": 4, "kv_heads": 4, "dim": 24, "vdim": 16, "scale": 0.7, "mask": {"size": 33}, "kv_from": 1}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 96},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.4, "mask": {"size": 70}}},
    ],
}
GUDUZEN_B = {
    "architecture": "Guduzen", "vocab": 200, "width": 96, "norm": {"eps": 1e-6}, "initializer_range": 0.06,
    "layers": [
        {"type": "latent_attention", "mlp": None,
         "mixer": {"heads": 20, "dim": 32, "vdim": 16, "kv_rank": 64, "q_rank": 20, "scale": 0.6}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 128},
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.25}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "conv": 2, "a_rank": 4, "g_rank": 4}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 40, "scale": 1.0, "mask": {"size": 64}}},
        {"type": "attention", "mlp": {"kind": "dense", "ff": 128},
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.2, "mask": {"size": 9}, "kv_from": 1}},
    ],
}
GUDUZEN_C = {
    "architecture": "Guduzen", "vocab": 96, "width": 48, "streams": 1, "logit_softcap": 8.0, "norm": {"eps": 1e-6},
    "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.8, "mask": {"size": 1}}},
        {"type": "channel_delta", "mlp": None,
         "mixer": {"heads": 3, "kv_heads": 1, "dim": 40, "vdim": 8, "conv": 4, "a_rank": 6, "g_rank": 2}},
        {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 64},
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 72, "conv": 1, "a_rank": 3, "g_rank": 5}},
    ],
}
CONFIGS = {"A": GUDUZEN_A, "B": GUDUZEN_B, "C": GUDUZEN_C}


def make_guduzen_dir(tmp_path: Path, config_json: dict, seed: int = 0, slow_decay: float = 3.0) -> Path:
    """A model folder with random bfloat16 weights.  Norm weights (stored around zero) and biases get a visible
    spread; the delta layers' step biases are lowered by ``slow_decay`` so that their state remembers hundreds of
    tokens instead of a handful; stream weights are spread around the values of a plain residual sum."""
    from gpullama3.java_b200.config import config_from_dict
    from gpullama3.java_b200.weights import random_checkpoint, write_safetensors

    cfg = config_from_dict(config_json)
    tag = abs(hash(json.dumps([config_json, seed, slow_decay], sort_keys=True))) % 10 ** 10
    out = Path(tmp_path) / f"guduzen_{tag}"
    if (out / "model.safetensors").is_file():
        return out
    out.mkdir(parents=True, exist_ok=True)
    where = "cuda" if torch.cuda.is_available() else "cpu"
    tensors = {n: t.cpu().to(torch.float32) for n, t in random_checkpoint(cfg, seed, dtype=torch.float32, norm_std=0.2,
                                                                          device=where)}
    for name in tensors:
        if name.endswith(".dt_bias"):
            tensors[name] = tensors[name] - slow_decay
        if name.endswith(".b") and tensors[name].dim() == 1:
            tensors[name] = tensors[name] * 4.0    # biases that matter next to the projections
    (out / "config.json").write_text(json.dumps(cfg.to_dict(), indent=2))
    write_safetensors(out / "model.safetensors", {n: t.to(torch.bfloat16) for n, t in tensors.items()})
    return out


def plain_inputs(model_dir: Path):
    """config.json as a dict and the weights as float32 tensors by checkpoint name, read with the safetensors package
    (not with the product's reader)."""
    from safetensors.torch import load_file

    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    weights = {k: v.to(torch.float32) for k, v in load_file(str(Path(model_dir) / "model.safetensors")).items()}
    return cfg, weights


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype, what: str = "") -> None:
    """float32: accumulation-order noise only.  bfloat16: the engine rounds activations between its kernels, the plain
    implementation does not round at all; what is allowed is a few roundings' worth relative to the largest logit."""
    got = got.detach().to("cpu", torch.float64)
    ref = ref.detach().to("cpu", torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(ref.abs().max()) + 1e-30
    err = (got - ref).abs()
    if dtype == torch.float32:
        assert float(err.max()) <= 5e-5 * scale, f"{what}: max err {float(err.max()):.3e} vs scale {scale:.3e}"
    else:
        assert float(err.max()) <= 0.08 * scale, f"{what}: max err {float(err.max()):.3e} vs scale {scale:.3e}"
        assert float(err.mean()) <= 0.012 * scale, f"{what}: mean err {float(err.mean()):.3e} vs scale {scale:.3e}"

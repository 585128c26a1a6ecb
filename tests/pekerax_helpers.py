"""Small Pekerax configurations for the tests, and model folders with random weights made so that faults show.

The three configurations differ from one another in every size and option: layer order, heads against key/value heads
(grouped, equal, one), key size against value size (smaller, equal, larger), sizes the tensor-core attention kernels take
and sizes that are widened, windows shorter and longer than a page, kept first positions (none, a few, more than a
page), value mixing (several layers, a single one, none), convolutions of 1 to 4 taps, layers without feed-forward, dense
and routed feed-forwards, one expert of many and several, one group and several, an embedding scale that is not a power
of two and none at all."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _moe(ff, limit, experts, top, count=1, keep=1):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def _attn(heads, kv, dim, vdim, scale, size, keep=None, mix=False):
    mask = {"size": size} if keep is None else {"size": size, "keep_first": keep}
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": mask}
    if mix:
        m["v_mix"] = True
    return m


PEKERAX_A = {
    "architecture": "Pekerax", "vocab": 160, "width": 64, "embedding": {"scale": 5.5}, "norm": {"eps": 1e-5},
    "initializer_range": 0.08,
    "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 16, 24, 0.4, 20, keep=3, mix=True), "mlp": {"kind": "dense", "ff": 96, "limit": 0.8}},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 3}, "mlp": _moe(32, 0.6, 6, 2, 3, 2)},
        {"type": "attention", "mixer": _attn(6, 2, 32, 24, 0.3, 70, keep=0, mix=True), "mlp": None},
        {"type": "attention", "mixer": _attn(2, 2, 64, 24, 0.2, 33, keep=70, mix=True), "mlp": _moe(48, 2.0, 4, 1)},
        {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "conv": 1}, "mlp": None},
    ],
}
PEKERAX_B = {
    "architecture": "Pekerax", "vocab": 200, "width": 96, "norm": {"eps": 1e-6}, "initializer_range": 0.06,
    "layers": [
        {"type": "delta", "mixer": {"heads": 3, "kv_heads": 1, "dim": 40, "vdim": 16, "conv": 4}, "mlp": {"kind": "dense", "ff": 64, "limit": 3.0}},
        {"type": "attention", "mixer": _attn(2, 1, 128, 128, 0.09, 64, keep=1, mix=True), "mlp": _moe(24, 1.2, 8, 3, 4, 2)},
        {"type": "attention", "mixer": _attn(3, 3, 16, 40, 0.5, 9), "mlp": {"kind": "dense", "ff": 128, "limit": 0.5}},
    ],
}
PEKERAX_C = {
    "architecture": "Pekerax", "vocab": 96, "width": 48, "embedding": {"scale": 0.75}, "norm": {"eps": 1e-6},
    "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mixer": _attn(1, 1, 32, 32, 0.3, 1, keep=2), "mlp": _moe(16, 1.0, 2, 2)},
        {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 72, "conv": 2}, "mlp": _moe(40, 1.5, 9, 4, 3, 3)},
        {"type": "attention", "mixer": _attn(8, 2, 16, 8, 0.6, 300, keep=5), "mlp": None},
    ],
}
CONFIGS = {"A": PEKERAX_A, "B": PEKERAX_B, "C": PEKERAX_C}


def make_pekerax_dir(tmp_path: Path, config_json: dict, seed: int = 0, slow_decay: float = 3.0, edit=None) -> Path:
    """A model folder with random bfloat16 weights.  Norm weights and biases get a visible spread; the delta layers'
    step biases are lowered by ``slow_decay`` so that their state remembers hundreds of tokens instead of a handful;
    sinks are spread over a few units and the mixing weights lie around one half.  ``edit(tensors)`` may change the
    float32 tensors before they are rounded and written."""
    from gpullama3.java_b200.config import config_from_dict
    from gpullama3.java_b200.weights import random_checkpoint, write_safetensors

    cfg = config_from_dict(config_json)
    tag = abs(hash(json.dumps([config_json, seed, slow_decay, getattr(edit, "__name__", None)], sort_keys=True))) % 10 ** 10
    out = Path(tmp_path) / f"pekerax_{tag}"
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
            tensors[name] = tensors[name] * 10.0    # norm biases that matter next to the normalised values
    if edit is not None:
        edit(tensors)
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


def has_routing(cfg: dict) -> bool:
    return any((L.get("mlp") or {}).get("kind") == "moe" for L in cfg["layers"])


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype, what: str = "", routed: bool = False) -> None:
    """float32: accumulation-order noise only, at every position.  bfloat16: the engine rounds activations between its
    kernels, the plain implementation does not round at all; what is allowed is a few roundings' worth relative to the
    largest logit.  With a routed feed-forward a bfloat16 run may choose another expert than the plain implementation
    where two scores lie within rounding of each other, which moves that token's logits: up to one position in six (two
    of a short run) may then lie outside (never in float32, where the scores agree to six digits)."""
    got = got.detach().to("cpu", torch.float64)
    ref = ref.detach().to("cpu", torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(ref.abs().max()) + 1e-30
    err = (got - ref).abs()
    if dtype == torch.float32:
        assert float(err.max()) <= 5e-5 * scale, f"{what}: max err {float(err.max()):.3e} vs scale {scale:.3e}"
        return
    worst, mean = err.amax(dim=-1), err.mean(dim=-1)
    bad = (worst > 0.08 * scale) | (mean > 0.012 * scale)
    allowed = max(2, bad.numel() // 6) if routed else 0
    assert int(bad.sum()) <= allowed, (f"{what}: {int(bad.sum())} of {bad.numel()} positions outside "
                                       f"(max err {float(err.max()):.3e}, scale {scale:.3e})")

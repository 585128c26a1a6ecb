"""Keys at the edges of Pekerax's attention and far back in its delta rule: just inside and just outside a window, the
last kept first position and the first one that is not kept (fewer than a page of them and more), the sink, keys far
back over many pages, the first tokens of a sequence, and long decoding.  Each test first shows on the plain
implementation that the thing it probes moves the logits by far more than the tolerance (a window or a kept run one
token shorter or longer, the sink gone, the far keys hidden, the early tokens dropped), so that an engine that got it
wrong could not pass.  The window model's score scale is small: its attention is nearly flat, so every visible key
carries weight and the edge key cannot hide behind a peak (its second layer has one head, whose distance penalty is the
smallest there is, so that kept positions a hundred tokens back still count); the far-key model's is large, so that single far keys carry
the result."""
import copy

import pytest
import torch

import plain_pekerax
from conftest import random_prompts
from pekerax_helpers import assert_logits, make_pekerax_dir, plain_inputs

pytestmark = pytest.mark.gpu
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])

WINDOWS = {
    "architecture": "Pekerax", "vocab": 64, "width": 32, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
    "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 48, "limit": 2.0},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.02, "mask": {"size": 17, "keep_first": 3}, "v_mix": True}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.02, "mask": {"size": 40, "keep_first": 67}, "v_mix": True}},
    ],
}
FAR = {
    "architecture": "Pekerax", "vocab": 64, "width": 32, "norm": {"eps": 1e-6}, "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 48, "limit": 2.0},
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 1.5, "mask": {"size": 690, "keep_first": 0}}},
        {"type": "delta", "mlp": None, "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "conv": 3}},
    ],
}


def flat_and_sunk(tensors):
    """Nearly flat attention (no distance penalty to speak of is left to the scale alone: the norm weights are small)
    and sinks that take a visible share."""
    for n in tensors:
        if n.endswith(".sink"):
            tensors[n] = tensors[n].abs() + 1.5


def _run(model_dir, dtype, tokens, prompt_len, chunk=None):
    """Logits at every position: the first ``prompt_len`` tokens as a prompt (in portions of ``chunk``), the rest one
    token a step."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    model = load_model(model_dir, dtype)
    cache = model.new_cache(64 * (len(tokens) // 64 + 2))
    step = StepFunction(model, cache)
    slot = cache.acquire()
    out, at = [], 0
    while at < len(tokens):
        n = 1 if at >= prompt_len else min(chunk or prompt_len, prompt_len - at)
        out.append(step([SequenceInput(slot, tokens[at:at + n], list(range(n)))]).cpu().clone())
        at += n
    cache.release(slot)
    cache.check_invariants()
    return torch.cat(out)


def _moved(a, b, scale):
    """Per position: how far two sets of logits are apart, in units of the float32 tolerance."""
    return (a - b).abs().amax(dim=1) / (5e-5 * scale)


@DTYPES
@pytest.mark.parametrize("prompt_len, chunk", [(180, None), (100, None), (100, 7), (3, None)])
def test_window_kept_positions_and_sink_in_prompts_and_in_decoding(session_tmp, dtype, prompt_len, chunk):
    d = make_pekerax_dir(session_tmp, WINDOWS, seed=2, edit=flat_and_sunk)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [180], seed=3)[0]
    ref = plain_pekerax.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    for layer, size, keep in ((0, 17, 3), (1, 40, 67)):
        for key, other in (("size", size - 1), ("size", size + 1), ("keep_first", keep - 1), ("keep_first", keep + 1)):
            c2 = copy.deepcopy(cfg)
            c2["layers"][layer]["mixer"]["mask"][key] = other
            moved = _moved(plain_pekerax.forward(c2, weights, tokens), ref, scale)[size + keep + 2:]
            # (the second layer spreads its weight over a hundred keys: one of them moves the logits less, still
            # several times what the float32 comparison allows)
            assert float((moved > (20 if layer == 0 else 5)).float().mean()) > 0.9, (layer, key, other, moved.median())
    gone = {n: (t - 40.0 if n.endswith(".sink") else t) for n, t in weights.items()}
    moved = _moved(plain_pekerax.forward(cfg, gone, tokens), ref, scale)
    assert float((moved > 20).float().mean()) > 0.9, moved.median()
    assert_logits(_run(d, dtype, tokens, prompt_len, chunk), ref, dtype, f"windows, prompt of {prompt_len}")


@DTYPES
@pytest.mark.parametrize("prompt_len, chunk", [(700, None), (520, 130), (64, None)])
def test_far_keys_and_long_memory(session_tmp, dtype, prompt_len, chunk):
    """700 tokens: eleven pages of keys with peaked scores, and a delta-rule state that still holds the first tokens at
    the end."""
    d = make_pekerax_dir(session_tmp, FAR, seed=4, slow_decay=6.0)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [700], seed=5)[0]
    ref = plain_pekerax.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    hidden = copy.deepcopy(cfg)
    hidden["layers"][0]["mixer"]["mask"]["size"] = 400            # attention that cannot see far back
    moved = _moved(plain_pekerax.forward(hidden, weights, tokens), ref, scale)[450:]
    assert float((moved > 20).float().mean()) > 0.9, moved.median()
    only_delta = copy.deepcopy(cfg)
    only_delta["layers"][0]["mixer"]["mask"]["size"] = 1          # so that only the delta rule carries the past
    full = plain_pekerax.forward(only_delta, weights, tokens)
    late = plain_pekerax.forward(only_delta, weights, tokens[300:])   # the same tokens without the first 300
    moved = _moved(late[250:], full[550:], float(full.abs().max()))
    assert float((moved > 20).float().mean()) > 0.9, moved.median()
    got = _run(d, dtype, tokens, prompt_len, chunk)
    assert_logits(got, ref, dtype, f"far keys, prompt of {prompt_len}")
    assert_logits(got[:4], ref[:4], dtype, "the first tokens")

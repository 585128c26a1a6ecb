"""Keys at the edges: just inside and just outside a window (of the layer that writes a cache and of a layer that reads
it with a longer window), far back in a latent-attention cache that spans many pages, far back in the delta rule's
state, the first tokens of a sequence, and long decoding.  Each test first shows on the plain implementation that the
thing it probes moves the logits by far more than the tolerance (a window one token shorter or longer, the far keys
hidden, the early tokens dropped), so that an engine that got it wrong could not pass.  The window model's score
scale is small: its attention is nearly flat, so every key of a window carries weight and the edge key cannot hide
behind a peak; the far-key model's is large, so that single far keys carry the result."""
import copy

import pytest
import torch

import plain_guduzen
from conftest import random_prompts
from guduzen_helpers import assert_logits, make_guduzen_dir, plain_inputs

pytestmark = pytest.mark.gpu
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])

WINDOWS = {
    "architecture": "Guduzen", "vocab": 64, "width": 32, "streams": 2, "norm": {"eps": 1e-6}, "initializer_range": 0.1,
    "layers": [
        {"type": "attention", "mlp": {"kind": "dense", "ff": 48},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.05, "mask": {"size": 17}}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.05, "mask": {"size": 70}, "kv_from": 0}},
    ],
}
FAR = {
    "architecture": "Guduzen", "vocab": 64, "width": 32, "streams": 3, "logit_softcap": 15.0, "norm": {"eps": 1e-6},
    "initializer_range": 0.1,
    "layers": [
        {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 48},
         "mixer": {"heads": 2, "dim": 16, "vdim": 16, "kv_rank": 32, "q_rank": 16, "scale": 2.0}},
        {"type": "channel_delta", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "conv": 3, "a_rank": 4, "g_rank": 4}},
    ],
}


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
def test_window_edges_in_prompts_and_in_decoding(session_tmp, dtype, prompt_len, chunk):
    d = make_guduzen_dir(session_tmp, WINDOWS, seed=2)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [180], seed=3)[0]
    ref = plain_guduzen.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    for layer, size in ((0, 17), (1, 70)):
        for other in (size - 1, size + 1):      # the key just inside dropped, the key just outside let in
            c2 = copy.deepcopy(cfg)
            c2["layers"][layer]["mixer"]["mask"]["size"] = other
            moved = _moved(plain_guduzen.forward(c2, weights, tokens), ref, scale)[size + 2:]
            assert float((moved > 20).float().mean()) > 0.9, (layer, other, moved.median())
    assert_logits(_run(d, dtype, tokens, prompt_len, chunk), ref, dtype, f"windows, prompt of {prompt_len}")


@DTYPES
@pytest.mark.parametrize("prompt_len, chunk", [(700, None), (520, 130), (64, None)])
def test_far_keys_and_long_memory(session_tmp, dtype, prompt_len, chunk):
    """700 tokens: eleven pages of latents, and a delta-rule state that still holds the first tokens at the end."""
    d = make_guduzen_dir(session_tmp, FAR, seed=4, slow_decay=6.0)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [700], seed=5)[0]
    ref = plain_guduzen.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    hidden = copy.deepcopy(cfg)
    hidden["layers"][0]["mixer"]["mask"] = {"size": 400}             # latent attention that cannot see far back
    moved = _moved(plain_guduzen.forward(hidden, weights, tokens), ref, scale)[450:]
    assert float((moved > 20).float().mean()) > 0.9, moved.median()
    only_delta = copy.deepcopy(cfg)
    only_delta["layers"][0]["mixer"]["mask"] = {"size": 1}           # so that only the delta rule carries the past
    full = plain_guduzen.forward(only_delta, weights, tokens)
    late = plain_guduzen.forward(only_delta, weights, tokens[300:])   # the same tokens without the first 300
    moved = _moved(late[250:], full[550:], float(full.abs().max()))
    assert float((moved > 20).float().mean()) > 0.9, moved.median()
    got = _run(d, dtype, tokens, prompt_len, chunk)
    assert_logits(got, ref, dtype, f"far keys, prompt of {prompt_len}")
    assert_logits(got[:4], ref[:4], dtype, "the first tokens")

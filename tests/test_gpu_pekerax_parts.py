"""Pekerax's mechanisms one at a time, each against its function of the plain implementation: the layer norm, the
clamped gated unit in the products' epilogues, the router (scores, groups, choice, weights), the experts streamed and as
dense products, and one-layer models that hold nothing but an attention mixer or a delta mixer."""
import types

import pytest
import torch

import plain_pekerax as P
from conftest import random_prompts
from pekerax_helpers import assert_logits, make_pekerax_dir, plain_inputs

pytestmark = pytest.mark.gpu
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
F = torch.float64


def _close(got, ref, dtype, what, f32=2e-5, bf16=2e-2):
    got, ref = got.detach().cpu().to(F), ref.detach().cpu().to(F)
    scale = float(ref.abs().max()) + 1e-30
    err = float((got - ref).abs().max())
    assert err <= (f32 if dtype == torch.float32 else bf16) * scale, f"{what}: {err:.3e} vs scale {scale:.3e}"


@DTYPES
@pytest.mark.parametrize("rows, dim", [(5, 48), (3, 50), (1300, 1024), (7, 5000), (2, 1)])
def test_layer_norm(dtype, rows, dim):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(rows + dim)
    x = torch.randn(rows, dim, generator=g) * 3 + 50.0          # a large mean: E[x^2] - mean^2 would lose the variance
    w, b = torch.randn(dim, generator=g), torch.randn(dim, generator=g)
    out = torch.empty((rows, dim), dtype=dtype, device="cuda")
    ops.layernorm(x.cuda(), w.cuda(), b.cuda(), out, 1e-5)
    _close(out, P.layer_norm(x.to(F), w.to(F), b.to(F), 1e-5), dtype, "layer norm", f32=1e-4, bf16=1e-2)
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32)
    out2 = torch.empty((2, dim), dtype=dtype, device="cuda")
    ops.layernorm(x.cuda(), w.cuda(), b.cuda(), out2, 1e-5, pick.cuda())
    assert torch.equal(out2.cpu(), out.cpu()[pick.long()])


@DTYPES
@pytest.mark.parametrize("tokens", [1, 9, 40, 300])
@pytest.mark.parametrize("limit", [0.4, 7.0])
def test_clamped_gated_unit(dtype, tokens, limit):
    """The gated feed-forward with the clamped unit: every product kernel that has the epilogue, by number of rows."""
    from gpullama3.java_b200.parts.feed_forward import SwiGLUFeedForward

    g = torch.Generator().manual_seed(tokens)
    width, ff = 64, 96
    ws = {n: (torch.randn(s, generator=g) * 0.3).to(torch.bfloat16).float() for n, s in
          (("gate", (ff, width)), ("up", (ff, width)), ("down", (width, ff)))}
    x = torch.randn(tokens, width, generator=g).to(torch.bfloat16).float()
    part = SwiGLUFeedForward(width, ff, "clamped_sigmoid", limit=limit, slope=1.702)
    part.load(ws, dtype, torch.device("cuda"))
    ctx = types.SimpleNamespace(dtype=dtype, all_decode=False, n_tokens=tokens,
                                empty=lambda shape, dt: torch.empty(tuple(shape), dtype=dt, device="cuda"))
    residual = torch.zeros(tokens, width, device="cuda")
    part.forward(x.to(dtype).cuda(), ctx, residual)
    ref = P.clamped_gated_unit(x.to(F), ws["gate"].to(F), ws["up"].to(F), ws["down"].to(F), limit)
    assert float(((x @ ws["gate"].T) > limit).float().mean()) > 0.02 or limit > 5     # the clamp is at work
    _close(residual, ref, dtype, f"clamped unit, {tokens} rows")


@pytest.mark.parametrize("experts, groups, keep, top", [(10, 2, 1, 3), (6, 3, 2, 2), (9, 3, 3, 4), (4, 1, 1, 1), (2, 1, 1, 2),
                                                         (64, 8, 3, 6), (40, 1, 1, 8)])
def test_router(experts, groups, keep, top):
    from gpullama3.java_b200.kernels import ops

    g = torch.Generator().manual_seed(experts * 7 + top)
    T, width = 77, 48
    h = torch.randn(T, width, generator=g)
    router = torch.randn(experts, width, generator=g) * 0.3
    chosen = torch.empty((T, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((T, top), dtype=torch.float32, device="cuda")
    scores = torch.empty((T, experts), dtype=torch.float32, device="cuda")
    ops.moe_route(h.cuda(), router.cuda(), chosen, weights, groups, keep, 1e-20, scores)
    idx, w = P.route(h.to(F), router.to(F), groups, keep, top)
    _close(scores, torch.softmax(h.to(F) @ router.to(F).T, dim=-1), torch.float32, "scores")
    assert torch.equal(chosen.cpu().long(), idx), "chosen experts (in the order of their scores)"
    _close(weights, w, torch.float32, "weights")
    # a group that holds the single best expert is among the kept ones; barred groups are never chosen from
    per = experts // groups
    if keep < groups:
        s = scores.cpu()
        best = s.view(T, groups, per).amax(dim=-1)
        kept = best.topk(keep, dim=-1).indices
        assert all(int(c) // per in kept[t].tolist() for t in range(T) for c in chosen[t].cpu())


@DTYPES
@pytest.mark.parametrize("tokens, decode", [(1, True), (7, True), (50, False), (400, False)])
def test_routed_feed_forward(dtype, tokens, decode):
    """Rows streamed past the experts' weights (few tokens, decode steps) and gathered into dense products (prompts)
    against the plain mixture; the two ways agree with each other far closer than the precision's tolerance."""
    from gpullama3.java_b200.parts.routed_feed_forward import RoutedFeedForward

    g = torch.Generator().manual_seed(tokens)
    width, ff, E, top = 64, 40, 6, 2
    ws = {"router": (torch.randn(E, width, generator=g) * 0.5).to(torch.bfloat16).float()}
    for e in range(E):
        for n, s in (("gate", (ff, width)), ("up", (ff, width)), ("down", (width, ff))):
            ws[f"e{e}.{n}"] = (torch.randn(s, generator=g) * 0.3).to(torch.bfloat16).float()
    x = torch.randn(tokens, width, generator=g).to(torch.bfloat16).float()
    part = RoutedFeedForward(width, ff, E, top, groups=3, keep_groups=2, activation="clamped_sigmoid", limit=0.7, slope=1.702)
    part.load(ws, dtype, torch.device("cuda"))
    ctx = types.SimpleNamespace(dtype=dtype, all_decode=decode, n_tokens=tokens,
                                empty=lambda shape, dt: torch.empty(tuple(shape), dtype=dt, device="cuda"))
    assert part.as_prompt(ctx, tokens) == (tokens == 400)
    residual = torch.full((tokens, width), 0.5, device="cuda")
    part.forward(x.to(dtype).cuda(), ctx, residual)
    W = {"p." + k: v.to(F) for k, v in ws.items()}
    ref = 0.5 + P.mixture_of_experts(x.to(F), W, "p.", E, 3, 2, top, 0.7)
    _close(residual, ref, dtype, f"routed feed-forward, {tokens} tokens")
    if tokens == 400:   # the same step through the kernels that read the counts themselves
        other = torch.full((tokens, width), 0.5, device="cuda")
        part.as_prompt = lambda ctx, n: False
        part.forward(x.to(dtype).cuda(), ctx, other)
        _close(other, residual, dtype, "streamed against gathered", f32=2e-6, bf16=4e-3)


@DTYPES
def test_routed_feed_forward_with_rows_too_long_to_stage(dtype, monkeypatch):
    """When the streaming kernel cannot stage the rows, a step of few tokens goes the prompts' way: the grouped product
    in bfloat16, one product per expert in float32 (which is then no longer safe to record)."""
    from gpullama3.java_b200.kernels import ops
    from gpullama3.java_b200.parts.routed_feed_forward import RoutedFeedForward

    monkeypatch.setattr(ops, "moe_rows_takes", lambda k, dt: False)
    g = torch.Generator().manual_seed(5)
    width, ff, E, top, tokens = 64, 48, 5, 3, 6
    ws = {"router": (torch.randn(E, width, generator=g) * 0.5).to(torch.bfloat16).float()}
    for e in range(E):
        for n, s in (("gate", (ff, width)), ("up", (ff, width)), ("down", (width, ff))):
            ws[f"e{e}.{n}"] = (torch.randn(s, generator=g) * 0.3).to(torch.bfloat16).float()
    x = torch.randn(tokens, width, generator=g).to(torch.bfloat16).float()
    part = RoutedFeedForward(width, ff, E, top, activation="clamped_sigmoid", limit=0.9, slope=1.702)
    part.load(ws, dtype, torch.device("cuda"))
    assert part.graph_safe == (dtype == torch.bfloat16)
    ctx = types.SimpleNamespace(dtype=dtype, all_decode=True, n_tokens=tokens,
                                empty=lambda shape, dt: torch.empty(tuple(shape), dtype=dt, device="cuda"))
    assert part.as_prompt(ctx, tokens)
    residual = torch.zeros(tokens, width, device="cuda")
    part.forward(x.to(dtype).cuda(), ctx, residual)
    W = {"p." + k: v.to(F) for k, v in ws.items()}
    _close(residual, P.mixture_of_experts(x.to(F), W, "p.", E, 1, 1, top, 0.9), dtype, "rows too long to stage")


def _one_layer(kind):
    if kind == "attention of 12 heads on one, 96 wide":   # the decode kernel's upper tile rows, the flash kernel's third size
        layer = {"type": "attention", "mlp": None,
                 "mixer": {"heads": 12, "kv_heads": 1, "dim": 80, "vdim": 96, "scale": 0.3, "mask": {"size": 37, "keep_first": 33}}}
    elif kind == "attention without a mask":
        layer = {"type": "attention", "mlp": None,
                 "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.4}}
    elif kind == "attention":
        layer = {"type": "attention", "mlp": None,
                 "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.5, "mask": {"size": 50, "keep_first": 2},
                           "v_mix": True}}
    else:
        layer = {"type": "delta", "mlp": None, "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 3}}
    return {"architecture": "Pekerax", "vocab": 64, "width": 32, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6},
            "initializer_range": 0.1, "layers": [layer]}


@DTYPES
@pytest.mark.parametrize("kind", ["attention", "attention of 12 heads on one, 96 wide", "attention without a mask", "delta"])
def test_one_mixer_alone(session_tmp, dtype, kind):
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d = make_pekerax_dir(session_tmp, _one_layer(kind), seed=3)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [150], seed=1)[0]
    ref = P.forward(cfg, weights, tokens)
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 4)
    step = StepFunction(model, cache)
    slot = cache.acquire()
    got = [step([SequenceInput(slot, tokens[:90], list(range(90)))]).cpu()]
    got += [step([SequenceInput(slot, [t], [0])]).cpu() for t in tokens[90:]]
    cache.release(slot)
    assert_logits(torch.cat(got), ref, dtype, kind + " alone")

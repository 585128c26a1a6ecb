"""A plain, slow implementation of the Pekerax decoder: one function per mechanism, whole sequences at once,
float64 on the CPU, no cache and no state carried between calls.  It shares no code with the package; the tests
compare the engine with it.

Notation: T tokens, x [T, width]; weights are a dict of float tensors by checkpoint name, a linear weight is
[out, in] and is applied as x @ W.T."""
from __future__ import annotations

import math

import torch

F = torch.float64


# ---------------------------------------------------------------- norms and small functions
def layer_norm(x, w, b, eps):
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_normalise(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ---------------------------------------------------------------- feed-forward
def clamped_gated_unit(h, gate, up, down, limit):
    """g = min(gate h, limit), u = clamp(up h, +-limit); down( g sigmoid(1.702 g) (u + 1) )."""
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, n_groups, keep_groups, top):
    """Per token: chosen expert indices [T, top] and their weights [T, top].  Scores are a softmax over all experts;
    experts outside the ``keep_groups`` groups with the largest best score are barred; weights are the chosen scores
    over their sum."""
    s = torch.softmax(h @ router.T, dim=-1)                       # [T, E]
    T, E = s.shape
    per = E // n_groups
    best = s.view(T, n_groups, per).max(dim=-1).values            # [T, groups]
    kept = torch.zeros(T, n_groups, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep_groups, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(T, n_groups, per).reshape(T, E)
    masked = s.masked_fill(~allowed, -1.0)
    idx = masked.topk(top, dim=-1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(dim=-1, keepdim=True) + 1e-20)


def mixture_of_experts(h, W, prefix, n_experts, n_groups, keep_groups, top, limit):
    idx, w = route(h, W[prefix + "router"], n_groups, keep_groups, top)
    out = torch.zeros(h.shape[0], W[prefix + "e0.down"].shape[0], dtype=F)
    for e in range(n_experts):
        y = clamped_gated_unit(h, W[f"{prefix}e{e}.gate"], W[f"{prefix}e{e}.up"], W[f"{prefix}e{e}.down"], limit)
        share = (w * (idx == e)).sum(dim=-1, keepdim=True)
        out += share * y
    return out


# ---------------------------------------------------------------- attention
def kept_window_mask(T, size, keep_first):
    """[T, T]: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def head_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F)


def sink_attention(q, k, v, scale, mask, slopes, sinks):
    """q [T, H, d], k [T, G, d], v [T, G, dv].  Scores lose slope_h * (i - j); the softmax's denominator also holds
    exp(sink_h), which has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(F)
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale - slopes[h] * dist
        s = s.masked_fill(~mask, float("-inf"))
        s = torch.cat([s, sinks[h].expand(T, 1)], dim=1)
        p = torch.softmax(s, dim=-1)[:, :T]
        out[:, h] = p @ v[:, g]
    return out


def attention_mixer(h, W, p, m, eps, v_first):
    """``m``: the layer's mixer record.  ``v_first``: the values of the first value-mixing layer (None when this is
    that layer or the layer does not mix).  Returns (output, this layer's own unmixed values)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_normalise(h @ W[p + "q"].T, eps) * W[p + "q.norm"]
    k = rms_normalise(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    v = h @ W[p + "v"].T
    own_v = v
    if v_first is not None:
        lam = W[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    rule = m.get("mask") or {"size": T}       # (no mask: every earlier position is visible)
    mask = kept_window_mask(T, rule["size"], rule.get("keep_first") or 0)
    o = sink_attention(q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv), m["scale"], mask, head_slopes(H), W[p + "sink"])
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T, own_v


# ---------------------------------------------------------------- gated delta rule
def causal_conv(x, w):
    """x [T, C], w [C, taps]: y[t, c] = sum_j w[c, j] x[t - (taps - 1) + j, c], zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], dim=0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def delta_recurrence(q, k, v, beta, g):
    """One head: q, k [T, dk], v [T, dv], beta, g [T].  S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, dk = q.shape
    S = torch.zeros(dk, v.shape[1], dtype=F)
    out = torch.zeros(T, v.shape[1], dtype=F)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, dk)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, dk)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                                   # [T, H]
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))   # [T, H]
    gate = silu(h @ W[p + "g"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        kv = hh // (H // G)
        o[:, hh] = delta_recurrence(q[:, kv], k[:, kv], v[:, hh], beta[:, hh], g[:, hh])
    o = rms_normalise(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * dv) @ W[p + "o"].T


# ---------------------------------------------------------------- the model
def feed_forward(h, W, p, mlp):
    if mlp["kind"] == "dense":
        return clamped_gated_unit(h, W[p + "gate"], W[p + "up"], W[p + "down"], mlp["limit"])
    r = mlp["router"]
    return mixture_of_experts(h, W, p, r["experts"], r["groups"]["count"], r["groups"]["keep"], r["top"],
                              mlp["expert"]["limit"])


def forward(cfg: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (float64); with ``return_layers`` also the residual after every layer."""
    W = {n: t.to(F) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    v_first = None
    after = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        if L["type"] == "attention":
            mixes = bool(L["mixer"].get("v_mix"))
            y, own_v = attention_mixer(h, W, p + "mix.", L["mixer"], eps, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = own_v
        elif L["type"] == "delta":
            y = delta_mixer(h, W, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp") is not None:
            h = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            x = x + feed_forward(h, W, p + "mlp.", L["mlp"])
        after.append(x)
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits

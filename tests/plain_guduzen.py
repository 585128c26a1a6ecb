"""A plain, slow implementation of the Guduzen decoder: one function per mechanism, whole sequences at once,
float64 on the CPU, no cache and no state carried between calls.  It shares no code with the package; the tests
compare the engine with it.

Notation: T tokens, x [T, width]; weights are a dict of float tensors by checkpoint name, a linear weight is
[out, in] and is applied as x @ W.T."""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_normalise(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """The layer norms: weights are stored around zero."""
    return rms_normalise(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_feed_forward(x, gate, up, down):
    return (gelu_tanh(x @ gate.T) * (x @ up.T)) @ down.T


def softcap(logits, cap):
    return cap * torch.tanh(logits / cap)


def visible(T, window):
    """[T, T] mask: query i sees key j when 0 <= i - j (< window, if there is one)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window is not None:
        m = m & (i - j < window)
    return m


def softmax_attention(q, k, v, scale, mask):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def windowed_attention(x, W, p, m, eps, shared=None):
    """The 'attention' mixer.  Returns its output and the (keys, values) it used, for layers that share them."""
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_normalise((x @ W[p + "q"].T + W[p + "q.b"]).view(T, H, d), eps)
    if shared is None:
        k = rms_normalise((x @ W[p + "k"].T + W[p + "k.b"]).view(T, G, d), eps)
        v = (x @ W[p + "v"].T + W[p + "v.b"]).view(T, G, dv)
    else:
        k, v = shared
    window = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(q, k, v, m["scale"], visible(T, window))
    return o.reshape(T, H * dv) @ W[p + "o"].T, (k, v)


def latent_attention(x, W, p, m, eps):
    T = x.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    c_q = rms_normalise(x @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    c = rms_normalise(x @ W[p + "dkv"].T, eps) * W[p + "dkv.norm"]
    q = (c_q @ W[p + "uq"].T).view(T, H, d)
    k = (c @ W[p + "uk"].T).view(T, H, d)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    window = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(q, k, v, m["scale"], visible(T, window))
    return o.reshape(T, H * dv) @ W[p + "o"].T


def short_convolution(x, w):
    """x [T, C], w [C, taps] (last column: the current token); zeros before the start; then SiLU."""
    T, taps = x.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F), x], dim=0)
    y = sum(padded[j:j + T] * w[:, j] for j in range(taps))
    return y * torch.sigmoid(y)


def delta_rule(q, k, v, beta, g):
    """One head: q, k, g [T, d], v [T, dv], beta [T].  S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=F)
    out = torch.zeros(T, v.shape[1], dtype=F)
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def channel_delta(x, W, p, m, eps):
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_convolution(x @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, d)
    k = short_convolution(x @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, d)
    v = short_convolution(x @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(x @ W[p + "b"].T)
    rate = torch.exp(W[p + "A_log"])[None, :, None]
    step = torch.nn.functional.softplus(((x @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).view(T, H, d))
    g = torch.exp(-rate * step)
    gate = torch.sigmoid((x @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, dv)
    o = torch.stack([delta_rule(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], beta[:, h], g[:, h]) for h in range(H)], dim=1)
    o = rms_normalise(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * dv) @ W[p + "o"].T


def connect(streams, W, prefix, y):
    """x_j <- sum_a mix[a, j] x_a + write[j] y, all j from the old streams."""
    s = len(streams)
    return [sum(W[prefix + "mix"][a, j] * streams[a] for a in range(s)) + W[prefix + "out"][j] * y for j in range(s)]


def forward(cfg: dict, weights: dict, tokens, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence."""
    W = {n: (t.to(F) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    s = cfg.get("streams")
    streams = [x.clone() for _ in range(s or 1)]
    kept = {}

    def sublayer(streams, i, which, norm_w, fn):
        if s is None:
            return [streams[0] + fn(offset_norm(streams[0], norm_w, eps))]
        prefix = f"l{i}.hc{which}."
        u = sum(W[prefix + "in"][a] * streams[a] for a in range(s))
        return connect(streams, W, prefix, fn(offset_norm(u, norm_w, eps)))

    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]

        def mixer(h, i=i, L=L, p=p, m=m):
            if L["type"] == "attention":
                src = m.get("kv_from")
                y, kv = windowed_attention(h, W, p, m, eps, kept[src] if src is not None else None)
                if src is None:
                    kept[i] = kv
                return y
            if L["type"] == "latent_attention":
                return latent_attention(h, W, p, m, eps)
            return channel_delta(h, W, p, m, eps)

        streams = sublayer(streams, i, 1, W[f"l{i}.norm1"], mixer)
        if L.get("mlp"):
            q = f"l{i}.mlp."
            streams = sublayer(streams, i, 2, W[f"l{i}.norm2"],
                               lambda h, q=q: gated_feed_forward(h, W[q + "gate"], W[q + "up"], W[q + "down"]))
        if layers_out is not None:
            layers_out.append(sum(streams))
    x = offset_norm(sum(streams), W["final.norm"], eps)
    logits = x @ W["embed"].T
    return softcap(logits, cfg["logit_softcap"]) if cfg.get("logit_softcap") else logits


def argmax_first(row) -> int:
    return int(torch.argmax(row))

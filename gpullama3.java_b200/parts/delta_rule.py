"""The gated delta rule with a decay per key channel: a recurrent mixer whose memory is one matrix per head.

For every token, with x the mixer's input:

    q, k = W_q x, W_k x  [kv_heads, d_k] ;  v = W_v x  [heads, d_v]      (head h reads q/k head h / (heads / kv_heads))
    each channel of q, k, v passes a short causal convolution over time, then SiLU
    q <- q / sqrt(sum q^2 + 1e-6) * d_k^(-1/2) ;  k <- k / sqrt(sum k^2 + 1e-6)                  per head
    beta = sigmoid(W_b x)  [heads] ;  g = exp(-exp(A_log[h]) * softplus(W_a2 W_a1 x + dt_bias))  [heads, d_k]
    S <- diag(g) S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q                        per head, S [d_k, d_v]
    y = W_o ( o / rms(o) * norm_weight * sigmoid(W_g2 W_g1 x) )                                  rms over d_v

What a sequence keeps is of fixed size: S of every head (float32) and the last ``taps - 1`` inputs of the convolution,
one float32 row per cache slot.  Norms, beta, g and the recurrence are 32-bit in both precisions; the projections and
the convolution are computed in the run's precision.  One product makes q, k, v, beta's and the two low-rank inputs
(its rows are the six weights one after the other, each group padded to a multiple of 8 rows)."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import StateNeed, StateView
from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import Mixer, StepContext, register_mixer
from .linear import Linear


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class ChannelDeltaRule(Mixer):
    graph_safe = True   # slots, lengths and tokens reach the kernels through the step's device tensors
    pad_safe = False    # every token it sees enters the state: a padded pass would leave its padding there

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: int, conv_taps: int,
                 norm_eps: float, decay_rank: int | None = None, gate_rank: int | None = None, unit_eps: float = 1e-6):
        """``decay_rank`` / ``gate_rank``: inner sizes of the two low-rank products; None reads them from the
        checkpoint's shapes (they are needed to make random weights)."""
        if n_heads % n_kv_heads:
            raise ConfigError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")
        if not (1 <= conv_taps <= ops.MAX_CONV_TAPS):
            raise ConfigError(f"conv taps {conv_taps}: the convolution kernel takes 1 to {ops.MAX_CONV_TAPS}")
        if min(head_dim, value_dim) < 1 or head_dim > 512:
            raise ConfigError(f"delta rule: key size {head_dim} must be between 1 and 512, value size positive")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.key_dim, self.value_dim, self.taps = int(head_dim), int(value_dim), int(conv_taps)
        self.norm_eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        G, H, dk, dv = n_kv_heads, n_heads, self.key_dim, self.value_dim
        self.channels = 2 * G * dk + H * dv            # what the convolution runs over: q, k, v side by side
        self.state_floats = H * dk * dv
        self.conv_floats = (self.taps - 1) * self.channels

    def parameters(self):
        G, H, dk, dv, h = self.n_kv_heads, self.n_heads, self.key_dim, self.value_dim, self.hidden_size
        ra = self.decay_rank if self.decay_rank is not None else -1
        rg = self.gate_rank if self.gate_rank is not None else -1
        taps_std = 1.0 / self.taps ** 0.5
        return {"q": ParamSpec((G * dk, h)), "k": ParamSpec((G * dk, h)), "v": ParamSpec((H * dv, h)),
                "q_conv": ParamSpec((G * dk, self.taps), "normal", 0.0, taps_std),
                "k_conv": ParamSpec((G * dk, self.taps), "normal", 0.0, taps_std),
                "v_conv": ParamSpec((H * dv, self.taps), "normal", 0.0, taps_std),
                "b": ParamSpec((H, h)), "A_log": ParamSpec((H,), "normal", -1.0, 0.5), "norm": ParamSpec((dv,), "norm"),
                "a1": ParamSpec((ra, h)), "a2": ParamSpec((H * dk, ra)), "dt_bias": ParamSpec((H * dk,), "normal", 0.0, 1.0),
                "g1": ParamSpec((rg, h)), "g2": ParamSpec((H * dv, rg)), "o": ParamSpec((h, H * dv))}

    def cache_need(self):
        return StateNeed((self.state_floats + self.conv_floats,), torch.float32)

    def load(self, tensors, dtype, device):
        run = lambda t: t.to(device).to(torch.float32 if dtype == torch.float32 else t.dtype)
        f32 = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        groups = [torch.cat([run(tensors["q"]), run(tensors["k"]), run(tensors["v"])], dim=0), run(tensors["b"]),
                  run(tensors["a1"]), run(tensors["g1"])]
        common = torch.float32 if any(g.dtype == torch.float32 for g in groups) else groups[0].dtype
        rows, offsets = [], []
        for g in groups:
            offsets.append(sum(r.shape[0] for r in rows))
            rows.append(g.to(common))
            pad = _pad8(g.shape[0]) - g.shape[0]
            if pad:
                rows.append(torch.zeros((pad, g.shape[1]), dtype=common, device=device))
        self.inputs = Linear(torch.cat(rows, dim=0).contiguous())
        _, self.beta_off, self.a1_off, self.g1_off = offsets
        self.decay_rank, self.gate_rank = tensors["a1"].shape[0], tensors["g1"].shape[0]
        self.a2 = Linear(run(tensors["a2"]).contiguous())
        self.g2 = Linear(run(tensors["g2"]).contiguous())
        self.o = Linear(run(tensors["o"]).contiguous())
        self.conv_weight = torch.cat([f32("q_conv"), f32("k_conv"), f32("v_conv")], dim=0).contiguous()
        self.dt_bias, self.a_log, self.norm_weight = f32("dt_bias"), f32("A_log"), f32("norm")
        if device.type == "cuda" and not ops.delta_rule_supported(self.key_dim):
            raise ConfigError(f"delta rule: no kernel holds a state column of {self.key_dim} rows")

    def forward(self, x, ctx: StepContext, cache: StateView, residual, writes_cache=True, then_norm=None):
        H, G, dk, dv, T = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim, x.shape[0]
        state = cache.data                                                    # [slots, S of every head | convolution inputs]
        proj = self.inputs.store(x, ctx.dtype, ctx.empty)
        qkv = ctx.empty((T, self.channels), ctx.dtype)
        ops.causal_conv_silu(proj, self.conv_weight, state[:, self.state_floats:], ctx.slots_dev, ctx.seq_ids,
                             ctx.cu_seqlens, qkv, self.channels, update_state=writes_cache)
        decay = self.a2.store(proj[:, self.a1_off:self.a1_off + self.decay_rank], ctx.dtype, ctx.empty)   # [T, H dk]
        gate = self.g2.store(proj[:, self.g1_off:self.g1_off + self.gate_rank], ctx.dtype, ctx.empty)     # [T, H dv]
        o = ctx.empty((T, H * dv), torch.float32)
        ops.delta_rule_scan(qkv, proj[:, self.beta_off:], decay, self.dt_bias, self.a_log, state, ctx.slots_dev,
                            ctx.cu_seqlens, o, H, G, dk, dv, dk ** -0.5, self.unit_eps, alloc=ctx.empty)
        gated = ctx.empty((T, H * dv), ctx.dtype)
        ops.gated_rmsnorm(o, self.norm_weight, gate, gated, H, dv, self.norm_eps)
        return self.o.add_to(gated, residual, then_norm)


class HeadDeltaRule(Mixer):
    """The gated delta rule with one decay per head, a gate of full rank and SiLU on it:

        q, k, v, the convolution, the unit vectors and beta as in ``ChannelDeltaRule``
        g = exp(-exp(A_log[h]) * softplus(W_a x + dt_bias))  [heads]             (one number per head and token)
        S <- g S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q          per head, S [d_k, d_v]
        y = W_o ( o / rms(o) * norm_weight * silu(W_g x) )                       rms over d_v, W_g x laid out heads x d_v

    One product makes q, k, v, beta's, the decays' and the gate's inputs.  State and precisions as in
    ``ChannelDeltaRule``; the scan is the same kernel, told that all key channels of a head decay alike."""
    graph_safe = True
    pad_safe = False

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: int, conv_taps: int,
                 norm_eps: float, unit_eps: float = 1e-6, gate_activation: str = "silu"):
        if n_heads % n_kv_heads:
            raise ConfigError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")
        if not (1 <= conv_taps <= ops.MAX_CONV_TAPS):
            raise ConfigError(f"conv taps {conv_taps}: the convolution kernel takes 1 to {ops.MAX_CONV_TAPS}")
        if min(head_dim, value_dim) < 1 or head_dim > 512:
            raise ConfigError(f"delta rule: key size {head_dim} must be between 1 and 512, value size positive")
        if gate_activation not in ops.GATE_ACTIVATIONS:
            raise ConfigError(f"delta rule: gate activation {gate_activation!r}; known: {', '.join(sorted(ops.GATE_ACTIVATIONS))}")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.key_dim, self.value_dim, self.taps = int(head_dim), int(value_dim), int(conv_taps)
        self.norm_eps, self.unit_eps, self.gate_activation = float(norm_eps), float(unit_eps), gate_activation
        G, H, dk, dv = n_kv_heads, n_heads, self.key_dim, self.value_dim
        self.channels = 2 * G * dk + H * dv
        self.state_floats = H * dk * dv
        self.conv_floats = (self.taps - 1) * self.channels

    def parameters(self):
        G, H, dk, dv, h = self.n_kv_heads, self.n_heads, self.key_dim, self.value_dim, self.hidden_size
        taps_std = 1.0 / self.taps ** 0.5
        return {"q": ParamSpec((G * dk, h)), "k": ParamSpec((G * dk, h)), "v": ParamSpec((H * dv, h)),
                "q_conv": ParamSpec((G * dk, self.taps), "normal", 0.0, taps_std),
                "k_conv": ParamSpec((G * dk, self.taps), "normal", 0.0, taps_std),
                "v_conv": ParamSpec((H * dv, self.taps), "normal", 0.0, taps_std),
                "b": ParamSpec((H, h)), "A_log": ParamSpec((H,), "normal", -1.0, 0.5), "norm": ParamSpec((dv,), "norm"),
                "a": ParamSpec((H, h)), "dt_bias": ParamSpec((H,), "normal", 0.0, 1.0),
                "g": ParamSpec((H * dv, h)), "o": ParamSpec((h, H * dv))}

    def cache_need(self):
        return StateNeed((self.state_floats + self.conv_floats,), torch.float32)

    def load(self, tensors, dtype, device):
        run = lambda t: t.to(device).to(torch.float32 if dtype == torch.float32 else t.dtype)
        f32 = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        groups = [torch.cat([run(tensors["q"]), run(tensors["k"]), run(tensors["v"])], dim=0), run(tensors["b"]),
                  run(tensors["a"]), run(tensors["g"])]
        common = torch.float32 if any(g.dtype == torch.float32 for g in groups) else groups[0].dtype
        rows, offsets = [], []
        for g in groups:
            offsets.append(sum(r.shape[0] for r in rows))
            rows.append(g.to(common))
            pad = _pad8(g.shape[0]) - g.shape[0]
            if pad:
                rows.append(torch.zeros((pad, g.shape[1]), dtype=common, device=device))
        self.inputs = Linear(torch.cat(rows, dim=0).contiguous())
        _, self.beta_off, self.decay_off, self.gate_off = offsets
        self.o = Linear(run(tensors["o"]).contiguous())
        self.conv_weight = torch.cat([f32("q_conv"), f32("k_conv"), f32("v_conv")], dim=0).contiguous()
        self.dt_bias, self.a_log, self.norm_weight = f32("dt_bias"), f32("A_log"), f32("norm")
        if device.type == "cuda" and not ops.delta_rule_supported(self.key_dim):
            raise ConfigError(f"delta rule: no kernel holds a state column of {self.key_dim} rows")

    def forward(self, x, ctx: StepContext, cache: StateView, residual, writes_cache=True, then_norm=None):
        H, G, dk, dv, T = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim, x.shape[0]
        state = cache.data
        proj = self.inputs.store(x, ctx.dtype, ctx.empty)
        qkv = ctx.empty((T, self.channels), ctx.dtype)
        ops.causal_conv_silu(proj, self.conv_weight, state[:, self.state_floats:], ctx.slots_dev, ctx.seq_ids,
                             ctx.cu_seqlens, qkv, self.channels, update_state=writes_cache)
        o = ctx.empty((T, H * dv), torch.float32)
        ops.delta_rule_scan(qkv, proj[:, self.beta_off:], proj[:, self.decay_off:], self.dt_bias, self.a_log, state,
                            ctx.slots_dev, ctx.cu_seqlens, o, H, G, dk, dv, dk ** -0.5, self.unit_eps, alloc=ctx.empty,
                            decay_per_head=True)
        gated = ctx.empty((T, H * dv), ctx.dtype)
        ops.gated_rmsnorm(o, self.norm_weight, proj[:, self.gate_off:], gated, H, dv, self.norm_eps, self.gate_activation)
        return self.o.add_to(gated, residual, then_norm)


register_mixer("channel_delta", ChannelDeltaRule)
register_mixer("head_delta", HeadDeltaRule)

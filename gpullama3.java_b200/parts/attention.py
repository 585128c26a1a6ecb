"""Grouped-query causal attention over the paged cache: the mixer of the Llama 3 decoder.

One run: project the normalised input to queries, keys and values with one fused weight
(inference/InferenceCore.java:78-80 of the reference project computes the three separately),
rotate queries and keys and store keys and values at each token's position (:83-101), attend over
everything the sequence has cached up to each token (:106-145), project back and add to the
residual stream (:148-151).  Sizes, the position encoding and an optional window are parameters.

Further parameters, all off for Llama 3: biases of the three projections; an RMS norm without weight over every
query and key head; a score scale other than 1/sqrt(head size); a value size other than the key size; keys and values
taken from the cache another layer writes (the mixer then has no key and value projections).  With any of them on, a
kernel between the projection and the rotation finishes the heads (bias, norm, the scale folded into the queries) and
widens them with zeros to one size the attention kernels take; the output product's columns are widened to match."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import KVCacheNeed, KVView
from ..config.base import ConfigError
from ..kernels import fast, ops
from ..weights.loader import ParamSpec
from .base import Mixer, PositionEncoding, StepContext, register_mixer
from .linear import Linear


class GroupedQueryAttention(Mixer):
    graph_safe = True
    pad_safe = True

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, position: PositionEncoding,
                 window: int | None = None, *, value_dim: int | None = None, bias: bool = False,
                 qk_norm_eps: float | None = None, scale: float | None = None, shares_cache: bool = False,
                 cache_window="own"):
        """``cache_window``: how many of the latest positions the cache entry keeps (``"own"``: this mixer's window);
        a layer whose cache other layers read with a longer window, or with none, is told so here."""
        if n_heads % n_kv_heads:
            raise ConfigError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")
        self.key_dim, self.value_dim = int(head_dim), int(value_dim if value_dim is not None else head_dim)
        self.bias, self.qk_norm_eps, self.shares_cache = bool(bias), qk_norm_eps, bool(shares_cache)
        self.scale = float(scale) if scale is not None else None
        self.finishes_heads = bool(self.bias or qk_norm_eps is not None or scale is not None or shares_cache
                                   or self.value_dim != self.key_dim
                                   or (self.key_dim % ops.HEAD_DIM_STEP != 0 and not position.rotary_dim))
        if self.finishes_heads:
            if min(self.key_dim, self.value_dim) < 1:
                raise ConfigError(f"head sizes must be positive, got {self.key_dim} and {self.value_dim}")
            head_dim = kernel_head_dim(max(self.key_dim, self.value_dim))
            if position.rotary_dim and head_dim != self.key_dim:
                raise ConfigError(f"a rotated head of {self.key_dim} cannot be widened to {head_dim}")
        # what no kernel takes is refused here, when the model is built, not at the first step
        if head_dim % ops.HEAD_DIM_STEP or not (0 < head_dim <= ops.MAX_HEAD_DIM):
            raise ConfigError(f"head_dim {head_dim}: the attention kernels take head sizes in steps of "
                              f"{ops.HEAD_DIM_STEP} up to {ops.MAX_HEAD_DIM}")
        if position.rotary_dim > min(head_dim, ops.MAX_ROTARY_DIM) or position.rotary_dim % 2:
            raise ConfigError(f"rotary_dim {position.rotary_dim} must be even and at most "
                              f"{min(head_dim, ops.MAX_ROTARY_DIM)} (head_dim {head_dim})")
        if window is not None and window < 1:
            raise ConfigError(f"window {window} must be at least 1 (or None for no window)")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = hidden_size, n_heads, n_kv_heads, head_dim
        self.position, self.window = position, window
        self.cache_window = window if cache_window == "own" else cache_window
        if self.cache_window is not None and (window is None or self.cache_window < window):
            raise ConfigError(f"a cache that keeps {self.cache_window} positions cannot serve a window of {window}")
        self.q_dim, self.kv_dim = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv: Linear | None = None
        self.o: Linear | None = None
        self.head_bias = None
        self.segments = None

    def parameters(self):
        H, G, dk, dv = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim
        p = {"q": ParamSpec((H * dk, self.hidden_size)), "o": ParamSpec((self.hidden_size, H * dv))}
        if not self.shares_cache:
            p["k"] = ParamSpec((G * dk, self.hidden_size))
            p["v"] = ParamSpec((G * dv, self.hidden_size))
        if self.bias:
            for n in ("q", "k", "v") if not self.shares_cache else ("q",):
                p[n + "_bias"] = ParamSpec(p[n].shape[:1], "matrix")
        return p

    def children(self):
        return {"position": self.position}

    def cache_need(self):
        return KVCacheNeed(self.n_kv_heads, self.head_dim, self.cache_window)

    def plan_decode(self, ctx: StepContext, cache: KVView) -> tuple[int, bool]:
        """How a decode step's attention is launched: into how many spans each sequence's keys are cut, and
        whether the kernel may be scheduled while its predecessor still runs.  Both follow from the number of
        sequences, this mixer's own kv heads and the longest sequence the step must be right for (its cache
        group's ``kv_capacity``: a recorded step is replayed until its page tables are outgrown)."""
        capacity = ctx.capacity(cache.group)
        if self.window:
            capacity = min(capacity, self.window)
        resident = ops.resident_ctas(ctx.device, self.head_dim, self.n_heads // self.n_kv_heads)
        splits = ops.attention_decode_splits(ctx.n_seqs, self.n_kv_heads, capacity, resident)
        return splits, ops.attention_decode_early_start(ctx.n_seqs, self.n_kv_heads, capacity, splits)

    def load(self, tensors, dtype, device):
        if self.finishes_heads:
            return self._load_finished(tensors, dtype, device)
        q, k, v, o = (tensors[n].to(device) for n in ("q", "k", "v", "o"))
        common = torch.float32 if (dtype == torch.float32 or torch.float32 in (q.dtype, k.dtype, v.dtype)) else q.dtype
        self.qkv = Linear(torch.cat([q.to(common), k.to(common), v.to(common)], dim=0).contiguous())
        self.o = Linear(o.to(torch.float32 if dtype == torch.float32 else o.dtype).contiguous())

    def _load_finished(self, tensors, dtype, device):
        H, G, dk, dv, D = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim, self.head_dim
        names = ("q",) if self.shares_cache else ("q", "k", "v")
        mats = [tensors[n].to(device) for n in names]
        common = torch.float32 if (dtype == torch.float32 or any(m.dtype == torch.float32 for m in mats)) else mats[0].dtype
        self.qkv = Linear(torch.cat([m.to(common) for m in mats], dim=0).contiguous())
        o = tensors["o"].to(device)
        o = o.to(torch.float32 if dtype == torch.float32 else o.dtype)
        wide = torch.zeros((self.hidden_size, H, D), dtype=o.dtype, device=device)   # columns of the zeros behind a value head
        wide[:, :, :dv] = o.view(self.hidden_size, H, dv)
        self.o = Linear(wide.view(self.hidden_size, H * D).contiguous())
        if self.bias:
            self.head_bias = torch.cat([tensors[n + "_bias"].to(device=device, dtype=torch.float32) for n in names]).contiguous()
        # the scale is folded into the queries: the attention kernels divide every score by sqrt(their head size)
        mul = (self.scale if self.scale is not None else dk ** -0.5) * D ** 0.5
        norm = self.qk_norm_eps is not None
        b = (lambda off: off) if self.bias else (lambda off: -1)
        # without rotation the finished keys and values go straight into their cache pages; with it they go to the
        # dense rows that the rotation kernel reads
        direct = not self.position.rotary_dim
        keys, values = (ops.TO_CACHE_KEYS, ops.TO_CACHE_VALUES) if direct else (ops.TO_ROWS, ops.TO_ROWS)
        segs = [ops.head_row_segment(0, H, dk, 0, D, b(0), norm, -1, mul)]
        if not self.shares_cache:
            segs.append(ops.head_row_segment(H * dk, G, dk, H * D, D, b(H * dk), norm, target=keys))
            segs.append(ops.head_row_segment((H + G) * dk, G, dv, (H + G) * D, D, b((H + G) * dk), target=values))
        self.segments = ops.head_row_segments(*segs)
        self.query_segment = ops.head_row_segments(segs[0])
        self.writes_direct = direct

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return not self.finishes_heads and ctx.all_decode and self.qkv.links_with(ctx.n_tokens, ctx.dtype)

    def forward(self, x, ctx: StepContext, cache: KVView, residual, writes_cache=True, then_norm=None):
        table = ctx.page_tables[cache.group]
        out = ctx.empty((x.shape[0], self.q_dim), ctx.dtype)
        attended = False
        if self.finishes_heads:
            if writes_cache and self.shares_cache:
                raise ConfigError("a mixer without key and value projections cannot write a cache entry")
            raw = self.qkv.store(x, ctx.dtype, ctx.empty)
            if self.writes_direct:
                qkv = ctx.empty((x.shape[0], self.q_dim), ctx.dtype)
                ops.head_rows(raw, qkv, self.segments if writes_cache else self.query_segment, self.qk_norm_eps or 0.0,
                              self.head_bias, cache=(ctx.positions, ctx.seq_ids, table, cache.k, cache.v) if writes_cache else None)
            else:
                qkv = ctx.empty((x.shape[0], self.q_dim + 2 * self.kv_dim), ctx.dtype)   # (a reader leaves the key and value columns unused)
                ops.head_rows(raw, qkv, self.segments, self.qk_norm_eps or 0.0, self.head_bias)
                ops.rope_cache_write(qkv, ctx.positions, ctx.seq_ids, table, self.position.inverse_frequencies(x.device),
                                     cache.k, cache.v, self.n_heads, self.n_kv_heads, self.head_dim,
                                     self.position.rotary_dim, self.position.pairing, write_cache=writes_cache)
        elif isinstance(x, torch.Tensor) and not ctx.all_decode:
            # a prompt pass: projection, rotation and cache write as one product where its epilogue can do all three
            qkv = ctx.empty((x.shape[0], self.qkv.out_features), ctx.dtype)
            if not fast.try_projection_with_rope(x, self.qkv.weight, qkv, ctx, table, cache, self, writes_cache):
                self.qkv.into(x, qkv)
                ops.rope_cache_write(qkv, ctx.positions, ctx.seq_ids, table, self.position.inverse_frequencies(x.device),
                                     cache.k, cache.v, self.n_heads, self.n_kv_heads, self.head_dim,
                                     self.position.rotary_dim, self.position.pairing, write_cache=writes_cache)
        else:
            qkv = self.qkv.store(x, ctx.dtype, ctx.empty)  # [T, q_dim + 2 kv_dim]; queries are rotated in place below
            # a decode step: one kernel rotates, writes the cache and attends, where the sizes allow
            attended = fast.try_decode_attention_with_rope(qkv, out, ctx, table, cache, self, writes_cache)
            if not attended:
                ops.rope_cache_write(qkv, ctx.positions, ctx.seq_ids, table, self.position.inverse_frequencies(x.device),
                                     cache.k, cache.v, self.n_heads, self.n_kv_heads, self.head_dim,
                                     self.position.rotary_dim, self.position.pairing, write_cache=writes_cache)
        if not attended and not fast.try_attention(qkv, out, ctx, table, cache, self):
            # (the plain kernel: a step of few tokens cuts their keys into spans so that the GPU has CTAs to run)
            rows = x.shape[0] * self.n_heads
            splits = 1 if rows >= 1024 else max(1, min(16, 1024 // rows, ctx.capacity(cache.group) // 512))
            ops.attention_paged(qkv, qkv.shape[1], out, ctx.positions, ctx.seq_ids, table, cache.k, cache.v,
                                self.n_heads, self.n_kv_heads, self.head_dim, self.window or 0, n_splits=splits)
        return self.o.add_to(out, residual, then_norm)


def kernel_head_dim(d: int) -> int:
    """The head size the attention kernels are given for heads of ``d``: the next size the tensor-core kernels take
    (steps of 32 up to 128), beyond that the next step of the plain kernel."""
    step = 32 if d <= 128 else ops.HEAD_DIM_STEP
    return -(-d // step) * step


register_mixer("attention", GroupedQueryAttention)

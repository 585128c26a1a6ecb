"""Latent attention: keys and values of all heads are products of one small cached row per position.

    c_q = norm(W_dq x) ;  q_h = W_uq,h c_q                      queries through a latent of their own
    c   = norm(W_dkv x)                                        the only thing the cache keeps ([kv_rank] per position)
    k_h = W_uk,h c ;  v_h = W_uv,h c ;  score = scale q_h . k_h ;  softmax ;  o_h = sum p v_h ;  W_o on the heads

Since q_h . (W_uk,h c) = (W_uk,h^T q_h) . c and sum p (W_uv,h c) = W_uv,h (sum p c), the cache is never expanded:
the queries are carried into the latent space (one small product per head, all heads in one launch), attention runs with ONE key/value head
whose keys and values are both c (head size kv_rank, all query heads in its group), and the result is carried back
through W_uv,h.  That is grouped-query attention over a paged cache, so the attention kernels and the cache group
of ``GroupedQueryAttention`` serve it; the latent is stored twice, row-wise as the keys and transposed as the values.
Positions do not enter the scores.  The score scale is folded into c_q (everything after it is linear)."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import KVCacheNeed, KVView
from ..config.base import ConfigError
from ..kernels import fast, ops
from ..weights.loader import ParamSpec
from .attention import kernel_head_dim
from .base import Mixer, StepContext, register_mixer
from .linear import Linear


class LatentAttention(Mixer):
    graph_safe = True
    pad_safe = True
    DECODE_GROUP = 16   # query heads per key/value head that the decode attention kernel takes

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, value_dim: int, kv_rank: int, q_rank: int,
                 norm_eps: float, scale: float | None = None, window: int | None = None):
        self.hidden_size, self.n_heads, self.key_dim, self.value_dim = hidden_size, n_heads, int(head_dim), int(value_dim)
        self.kv_rank, self.q_rank, self.norm_eps = int(kv_rank), int(q_rank), float(norm_eps)
        self.scale = float(scale) if scale is not None else self.key_dim ** -0.5
        if min(self.kv_rank, self.q_rank, self.key_dim, self.value_dim, n_heads) < 1:
            raise ConfigError("latent attention: every size must be positive")
        # the sizes the attention kernels see: one key/value head as wide as the (widened) latent
        self.head_dim = kernel_head_dim(self.kv_rank)
        if self.head_dim > ops.MAX_HEAD_DIM:
            raise ConfigError(f"kv_rank {kv_rank}: the attention kernels take rows of at most {ops.MAX_HEAD_DIM}")
        if window is not None and window < 1:
            raise ConfigError(f"window {window} must be at least 1 (or None for no window)")
        self.n_kv_heads, self.window = 1, window
        self.q_pad = -(-self.q_rank // 8) * 8

    def parameters(self):
        H, dk, dv, h = self.n_heads, self.key_dim, self.value_dim, self.hidden_size
        return {"dq": ParamSpec((self.q_rank, h)), "dq_norm": ParamSpec((self.q_rank,), "norm"),
                "uq": ParamSpec((H * dk, self.q_rank)), "dkv": ParamSpec((self.kv_rank, h)),
                "dkv_norm": ParamSpec((self.kv_rank,), "norm"), "uk": ParamSpec((H * dk, self.kv_rank)),
                "uv": ParamSpec((H * dv, self.kv_rank)), "o": ParamSpec((h, H * dv))}

    def cache_need(self):
        return KVCacheNeed(1, self.head_dim, self.window)

    def plan_decode(self, ctx: StepContext, cache: KVView) -> tuple[int, bool]:
        capacity = ctx.capacity(cache.group)
        if self.window:
            capacity = min(capacity, self.window)
        resident = ops.resident_ctas(ctx.device, self.head_dim, min(self.n_heads, self.DECODE_GROUP))
        splits = ops.attention_decode_splits(ctx.n_seqs, 1, capacity, resident)
        return splits, ops.attention_decode_early_start(ctx.n_seqs, 1, capacity, splits)

    def load(self, tensors, dtype, device):
        H, dk, dv, R, D = self.n_heads, self.key_dim, self.value_dim, self.kv_rank, self.head_dim
        keep = lambda t: t.to(device).to(torch.float32 if dtype == torch.float32 else t.dtype)
        dq, dkv, uq, uk, uv, o = (keep(tensors[n]) for n in ("dq", "dkv", "uq", "uk", "uv", "o"))
        common = torch.float32 if torch.float32 in (dq.dtype, dkv.dtype) else dq.dtype
        self.down = Linear(torch.cat([dq.to(common), dkv.to(common)], dim=0).contiguous())   # rows: c_q, then c
        self.uq = Linear(uq.contiguous())
        # head h: queries into the latent space with W_uk,h^T (rows widened with zeros to D), results back with W_uv,h
        uk_t = torch.zeros((H, D, dk), dtype=uk.dtype, device=device)
        uk_t[:, :R] = uk.view(H, dk, R).transpose(1, 2)
        uv_w = torch.zeros((H, dv, D), dtype=uv.dtype, device=device)
        uv_w[:, :, :R] = uv.view(H, dv, R)
        self.carry_in, self.carry_out = uk_t.contiguous(), uv_w.contiguous()   # [H, D, dk] and [H, dv, D]
        self.o = Linear(o.contiguous())
        self.norm_weights = torch.cat([tensors["dq_norm"].to(device=device, dtype=torch.float32),
                                       tensors["dkv_norm"].to(device=device, dtype=torch.float32)]).contiguous()
        mul = self.scale * D ** 0.5   # the attention kernels divide every score by sqrt(their head size)
        qr = self.q_rank
        self.query_segment = ops.head_row_segments(ops.head_row_segment(0, 1, qr, 0, self.q_pad, -1, True, 0, mul))   # c_q
        self.latent_segments = ops.head_row_segments(   # c, once as a key row and once as a value row of its cache page
            ops.head_row_segment(qr, 1, R, 0, D, -1, True, qr, target=ops.TO_CACHE_KEYS),
            ops.head_row_segment(qr, 1, R, 0, D, -1, True, qr, target=ops.TO_CACHE_VALUES))

    def forward(self, x, ctx: StepContext, cache: KVView, residual, writes_cache=True, then_norm=None):
        H, dk, dv, D, T = self.n_heads, self.key_dim, self.value_dim, self.head_dim, x.shape[0]
        table = ctx.page_tables[cache.group]
        down = self.down.store(x, ctx.dtype, ctx.empty)                       # [T, q_rank + kv_rank]
        c_q = ctx.empty((T, self.q_pad), ctx.dtype)
        ops.head_rows(down, c_q, self.query_segment, self.norm_eps, None, self.norm_weights)
        if writes_cache:
            ops.head_rows(down, None, self.latent_segments, self.norm_eps, None, self.norm_weights,
                          cache=(ctx.positions, ctx.seq_ids, table, cache.k, cache.v))
        q = self.uq.store(c_q[:, :self.q_rank], ctx.dtype, ctx.empty)         # [T, H dk]
        carried = ctx.empty((T, H * D), ctx.dtype)                            # queries in the latent space
        ops.gemm_per_head(q, self.carry_in, carried)
        heads = ctx.empty((T, H * dv), ctx.dtype)
        if ctx.all_decode and H > self.DECODE_GROUP and ops.attention_decode_supported(ctx.dtype, self.DECODE_GROUP, 1, D):
            # the decode kernel takes up to DECODE_GROUP query heads per key/value head: the heads go in groups, each
            # group over the same cached latents
            splits, early = self.plan_decode(ctx, cache)
            for g in range(0, H, self.DECODE_GROUP):
                n = min(self.DECODE_GROUP, H - g)
                part = ctx.empty((T, n * D), ctx.dtype)
                ops.attention_decode(carried[:, g * D:], carried.stride(0), part, ctx.kv_lens, table, cache.k, cache.v, n, 1,
                                     D, self.window or 0, splits, early_start=early)
                ops.gemm_per_head(part, self.carry_out[g:g + n], heads[:, g * dv:(g + n) * dv])
            return self.o.add_to(heads, residual, then_norm)
        out = ctx.empty((T, H * D), ctx.dtype)
        if not fast.try_attention(carried, out, ctx, table, cache, self):
            n_rows = T * H
            splits = 1 if n_rows >= 1024 else max(1, min(16, 1024 // n_rows, ctx.capacity(cache.group) // 512))
            ops.attention_paged(carried, carried.stride(0), out, ctx.positions, ctx.seq_ids, table, cache.k, cache.v,
                                H, 1, D, self.window or 0, n_splits=splits)
        ops.gemm_per_head(out, self.carry_out, heads)
        return self.o.add_to(heads, residual, then_norm)


register_mixer("latent_attention", LatentAttention)

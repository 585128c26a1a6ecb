"""Several residual streams (hyper-connections) and the block that runs its sublayers through them.

Instead of one residual row a token has ``streams`` of them, [T, S, width] in float32, all equal to the embedding
at the start.  A sublayer reads one weighted sum of the streams, and its result y goes back into every stream
while the streams are mixed among themselves:

    u = sum_a read[a] x_a ;   y = sublayer(norm(u)) ;   x_j <- sum_a mix[a, j] x_a + write[j] y   (all j at once)

The model's output is the sum of the streams.  ``StreamConnection`` holds the three small tensors of one sublayer;
``ConnectedBlock`` is the pre-norm arrangement (mixer, optional feed-forward) over such connections, or over the
plain residual sum x <- x + y when it is built without them."""
from __future__ import annotations

import torch

from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import Block, Part, StepContext, all_parts, register_block, register_part


def _norm_form(norm):
    form = norm.row_factor_form()
    if form is None:
        raise ConfigError("a stream connection reads through a norm of the form weight * x / rms(x)")
    weight, eps, dim = form
    if weight.dtype != torch.float32:
        cached = getattr(norm, "_weight_f32", None)
        if cached is None or cached.device != weight.device:
            cached = norm._weight_f32 = weight.to(torch.float32)
        weight = cached
    return weight, eps, dim


class StreamConnection(Part):
    graph_safe = True
    pad_safe = True

    def __init__(self, streams: int):
        if not (1 <= int(streams) <= ops.MAX_STREAMS):
            raise ConfigError(f"streams {streams}: the stream kernels take 1 to {ops.MAX_STREAMS}")
        self.streams = int(streams)
        self.read = self.write = self.mix = None

    def parameters(self):
        s = self.streams
        return {"read": ParamSpec((s,), "normal", 1.0 / s, 0.1), "write": ParamSpec((s,), "normal", 1.0, 0.1),
                "mix": ParamSpec((s, s), "normal", 1.0 / s, 0.2)}

    def load(self, tensors, dtype, device):
        self.read, self.write, self.mix = (tensors[n].to(device=device, dtype=torch.float32).contiguous()
                                           for n in ("read", "write", "mix"))

    def read_norm(self, residual: torch.Tensor, norm, ctx: StepContext) -> torch.Tensor:
        """norm(sum_a read[a] x_a) as rows of the run dtype; residual float32 [T, S, width]."""
        weight, eps, dim = _norm_form(norm)
        out = ctx.empty((residual.shape[0], dim), ctx.dtype)
        ops.streams_read_norm(residual, self.read, weight, out, eps)
        return out

    def write_back(self, residual: torch.Tensor, y: torch.Tensor) -> None:
        ops.streams_combine(residual, residual, self.mix, self.write, y)

    def step(self, residual: torch.Tensor, y: torch.Tensor, then: "StreamRead | None", ctx: StepContext, alloc):
        """This sublayer's write-back (which also clears ``y`` for the next sublayer's product) and, in the same
        kernel, the read and norm of the sublayer that runs next (``then``); returns that sublayer's input rows, or
        None when nothing runs next."""
        if then is None:
            ops.streams_step(residual, self.mix, self.write, y)
            return None
        weight, eps, dim = _norm_form(then.norm)
        out = alloc((residual.shape[0], dim), ctx.dtype)
        ops.streams_step(residual, self.mix, self.write, y, then.connection.read, weight, out, eps)
        return out


class StreamRead:
    """How a connected sublayer takes its input: the read weights of its connection and the norm behind them.  A
    block hands this out as its first norm, so that the block before it can do the read in its own last kernel."""

    def __init__(self, norm, connection: StreamConnection):
        self.norm, self.connection = norm, connection

    def row_factor_form(self):
        return self.norm.row_factor_form()


_ones: dict = {}


def _ones_on(device, n: int) -> torch.Tensor:
    key = (str(device), n)
    t = _ones.get(key)
    if t is None:
        t = _ones[key] = torch.ones(n, dtype=torch.float32, device=device)
    return t


def open_streams(x: torch.Tensor, streams: int, alloc) -> torch.Tensor:
    """[T, width] -> [T, streams, width], every stream a copy of x."""
    T, width = x.shape
    if streams == 1:
        return x.view(T, 1, width)
    out = alloc((T, streams, width), torch.float32)
    ops.streams_combine(x.view(T, 1, width), out, _ones_on(x.device, streams))
    return out


def close_streams_norm(residual: torch.Tensor, norm, out_dtype, rows, alloc) -> torch.Tensor:
    """The model's last norm over the sum of the streams, for the rows whose logits are wanted."""
    T, s, width = residual.shape
    if s == 1:
        return norm.forward(residual.view(T, width), out_dtype, rows=rows, alloc=alloc)
    weight, eps, dim = _norm_form(norm)
    n = T if rows is None else rows.numel()
    out = alloc((n, dim), out_dtype)
    ops.streams_read_norm(residual, _ones_on(residual.device, s), weight, out, eps, rows)
    return out


class ConnectedBlock(Block):
    """x <- connect(x, mixer(norm(read(x)))), then the same with the feed-forward if the layer has one.  With
    connections the residual is [T, S, width]; without, [T, width] and the connection is the plain sum."""

    def __init__(self, mixer, mixer_norm, mixer_connection=None, feed_forward=None, feed_forward_norm=None,
                 feed_forward_connection=None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ConfigError("a feed-forward and its norm come together")
        if feed_forward is None and feed_forward_connection is not None:
            raise ConfigError("a feed-forward connection without a feed-forward")
        if feed_forward is not None and (mixer_connection is None) != (feed_forward_connection is None):
            raise ConfigError("either every sublayer of a block has a stream connection or none")
        given = {"mixer": mixer, "mixer_norm": mixer_norm, "mixer_connection": mixer_connection,
                 "feed_forward": feed_forward, "feed_forward_norm": feed_forward_norm,
                 "feed_forward_connection": feed_forward_connection}
        super().__init__(**{k: v for k, v in given.items() if v is not None})
        for k, v in given.items():
            setattr(self, k, v)
        self.streams = mixer_connection.streams if mixer_connection is not None else None
        if feed_forward_connection is not None and feed_forward_connection.streams != self.streams:
            raise ConfigError("the connections of one block differ in their number of streams")

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in all_parts(self).values())

    @property
    def pad_safe(self):
        return all(p.pad_safe for p in all_parts(self).values())

    def first_norm(self):
        if self.mixer_connection is None:
            return self.mixer_norm
        return StreamRead(self.mixer_norm, self.mixer_connection)

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        """With stream connections the block takes its first input from the block before it (``x_in``) and leaves the
        next block's (``then_norm``, that block's ``StreamRead``): a write-back and the read behind it are one kernel."""
        return self.mixer_connection is not None

    def forward(self, residual, ctx: StepContext, cache, writes_cache=True, x_in=None, then_norm=None):
        if self.mixer_connection is None:     # one residual stream: x <- x + sublayer(norm(x))
            self.mixer.forward(self.mixer_norm.forward(residual, ctx.dtype, alloc=ctx.empty), ctx, cache, residual, writes_cache)
            if self.feed_forward is not None:
                self.feed_forward.forward(self.feed_forward_norm.forward(residual, ctx.dtype, alloc=ctx.empty), ctx, residual)
            return None
        # what a sublayer's last product adds into, as it would into a residual stream: one buffer per pass, cleared
        # by the kernel that consumes it
        y = ctx.extras.get("stream sublayer result")
        if y is None:
            y = ctx.extras["stream sublayer result"] = torch.zeros((residual.shape[0], residual.shape[2]),
                                                                   dtype=torch.float32, device=residual.device)
        x = x_in if x_in is not None else self.mixer_connection.read_norm(residual, self.mixer_norm, ctx)
        self.mixer.forward(x, ctx, cache, y, writes_cache)
        last = self.mixer_connection
        if self.feed_forward is not None:
            x = last.step(residual, y, StreamRead(self.feed_forward_norm, self.feed_forward_connection), ctx, ctx.empty)
            self.feed_forward.forward(x, ctx, y)
            last = self.feed_forward_connection
        if then_norm is not None and not isinstance(then_norm, StreamRead):
            then_norm = None
        # (rows handed to the next block outlive this block's workspace: they come from the allocator)
        return last.step(residual, y, then_norm, ctx,
                         lambda shape, dtype: torch.empty(shape, dtype=dtype, device=residual.device))


register_part("connection", "streams", StreamConnection)
register_block("connected", ConnectedBlock)

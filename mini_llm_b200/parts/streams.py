"""Hyper-connections: the residual is ``n_streams`` copies of the width instead of one.

All streams start as the embedding output.  A sublayer with a connection reads
``u = sum_s in[s] x_s``, computes ``y = sublayer(norm(u))`` and then replaces all streams at once
from the old ones, ``x_t <- sum_s mix[s, t] x_s + out[t] y`` (the mixing matrix is indexed
[from, to]).  After the last layer the model's residual is the sum of the streams.  Streams,
weights and sums are 32-bit.

``stream_connection`` is the connection of one sublayer: its three weight tensors and the passes
over ``ctx.streams`` [T, n_streams, width].  A pass is one kernel: the write of one sublayer's
result, the read-out for the next sublayer and that sublayer's norm (an RMS norm over the whole
width) may be one pass.  A layer's last write may wait (``write(defer=True)``) for the next read-out of
the streams, the next layer's or the model's final sum, and go with it in one pass; the result that
waits must stay untouched until then (``ctx.streams_pending``).
"""

from __future__ import annotations

import torch

from .base import Part, register_part
from .spec import WeightSpec


def take_pending(ctx) -> dict:
    """The arguments of the write that waits for the next pass over the streams (none: an empty dict)."""
    pending = getattr(ctx, "streams_pending", None) or {}
    ctx.streams_pending = None
    return pending


def flush(ctx) -> None:
    """The write that waits, as a pass of its own."""
    pending = take_pending(ctx)
    if pending:
        ctx.kernels.streams_step(ctx.streams, **pending)


def read_sum(ctx, out) -> None:
    """The plain sum of the streams (the model's residual) into ``out`` (fp32 [T, width]), after the write that waits."""
    ctx.kernels.streams_step(ctx.streams, read=True, u_out=out, **take_pending(ctx))


class StreamConnection(Part):
    graph_safe = True

    def __init__(self, prefix, n_streams: int, in_name: str = "in", out_name: str = "out", mix_name: str = "mix"):
        super().__init__(prefix)
        self.n_streams = int(n_streams)
        if not 1 <= self.n_streams <= 16:
            raise ValueError(f"{prefix}: between 1 and 16 streams, got {self.n_streams}")
        self.names = dict(read=in_name, write=out_name, mix=mix_name)

    def weight_specs(self):
        n, s = self.names, self.n_streams
        return [WeightSpec(self.full_name(n["read"]), (s,), role="vector", init="gain"),
                WeightSpec(self.full_name(n["write"]), (s,), role="vector", init="gain"),
                WeightSpec(self.full_name(n["mix"]), (s, s), role="vector", init="identity")]

    def _streams(self, ctx):
        streams = getattr(ctx, "streams", None)
        if streams is None or streams.shape[1] != self.n_streams:
            raise RuntimeError(f"{self.prefix}: the model keeps no {self.n_streams} residual streams (ModelSpec.residual_streams)")
        return streams

    @staticmethod
    def _fusable(norm) -> bool:
        """Whether the pass can apply this norm itself: an RMS norm over the whole width."""
        from .norm import GroupedRmsNorm
        return isinstance(norm, GroupedRmsNorm) and norm.groups == 1

    def _pass(self, ctx, norm, tag, reader, **write):
        """One pass: an optional write (of this connection), then ``reader``'s read-out, normed by ``norm``."""
        streams = self._streams(ctx)
        n, width = streams.shape[0], streams.shape[2]
        read_weights = reader.w(reader.names["read"])
        if self._fusable(norm):
            out = ctx.buffer(tag, (n, width), ctx.act_dtype)
            ctx.kernels.streams_step(streams, read=True, w_in=read_weights, normed=out, gain=norm.w(norm.name), eps=norm.eps, **write)
            return out
        u = ctx.buffer("streams_read", (n, width), torch.float32)
        ctx.kernels.streams_step(streams, read=True, w_in=read_weights, u_out=u, **write)
        return norm.forward(ctx, u, tag=tag)

    def _write_arguments(self, y):
        return dict(y=y, mix=self.w(self.names["mix"]), w_out=self.w(self.names["write"]))

    def read(self, ctx, norm, tag="norm_1"):
        """The normed read-out of the streams: what this connection's sublayer takes in.  A write that
        waits goes first, in the same pass."""
        return self._pass(ctx, norm, tag, self, **take_pending(ctx))

    def write(self, ctx, y, defer=False):
        """The sublayer's result ``y`` (fp32 [T, width]) onto the streams; with ``defer`` together with the
        next read-out of the streams, whoever asks for it."""
        if defer:
            flush(ctx)
            self._streams(ctx)
            ctx.streams_pending = self._write_arguments(y)
            return
        ctx.kernels.streams_step(self._streams(ctx), **self._write_arguments(y))

    def write_then_read(self, ctx, y, reader, norm, tag="norm_2"):
        """``write(y)``, then the next connection's (``reader``) normed read-out, in one pass."""
        return self._pass(ctx, norm, tag, reader, **self._write_arguments(y))


register_part("stream_connection", StreamConnection)

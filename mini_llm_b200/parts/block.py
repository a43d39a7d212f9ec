"""Arrangements: how one layer's parts are wired around the residual stream.

"pre_norm" is the reference's block (engine/src/transformer_block.c:49-71):
``r = x + mixer(norm_1(x))``, then ``out = r + feed_forward(norm_2(r))``.  The
residual stream stays 32-bit; mixers and feed-forwards add into it in place.

"sandwich_norm" norms every sublayer on both sides:
``x <- x + norm_1b(mixer(filter(norm_1(x))))``, then, if the layer has a feed-forward,
``x <- x + norm_2b(feed_forward(norm_2(x)))``, then, if it has one, its "depth_mix" part replaces
x by a weighted sum of all layer results so far.  The input filter (a short convolution, say) and
the feed-forward are optional roles; the mixer and the feed-forward hand over their output itself
(``compute``), and the outer norm adds it onto the stream (``add_normed``).

"output_norm" norms a sublayer's OUTPUT only: ``x <- x + norm_1(mixer(x))``, then, if the layer has a feed-forward,
``x <- x + norm_2(feed_forward(x))``.  The sublayers read the stream itself, rounded to the activations' type; the
rounded rows are written by the pass that adds the normed result before them (the first layer rounds by itself).

"hyper_connections" is the pre-norm block over several residual streams (``ctx.streams``; see
``parts.streams``): each sublayer reads a weighted sum of the streams through its norm and writes
its result back onto all of them through a mixing matrix.  ``hidden`` is not touched; the model
sums the streams after its last layer.
"""

from __future__ import annotations

from .base import Arrangement, register_arrangement


def _defer(norm, consumer) -> dict:
    if getattr(consumer, "accepts_deferred_norm", False) and getattr(norm, "can_defer", False):
        return {"defer": True}
    return {}


class PreNorm(Arrangement):
    roles = ("norm_1", "mixer")
    optional_roles = ("norm_2", "feed_forward")      # a layer may have no feed-forward

    def run(self, ctx, parts, hidden, cache):
        # A part that states ``accepts_deferred_norm`` may get its input norm unevaluated
        # (to fuse it into its first product); any other part gets a tensor.
        x = parts["norm_1"].forward(ctx, hidden, tag="norm_1", **_defer(parts["norm_1"], parts["mixer"]))
        if getattr(cache, "kind", "none") == "composite":
            cache = cache.sub("mixer")               # a mixer that keeps several things gets them by its own names
        parts["mixer"].forward(ctx, x, hidden, cache)
        if "feed_forward" in parts:
            x = parts["norm_2"].forward(ctx, hidden, tag="norm_2", **_defer(parts["norm_2"], parts["feed_forward"]))
            parts["feed_forward"].forward(ctx, x, hidden)


class SandwichNorm(Arrangement):
    roles = ("norm_1", "mixer", "norm_1b")
    optional_roles = ("input_filter", "norm_2", "feed_forward", "norm_2b", "depth_mix")

    def cache_roles(self, parts):
        return tuple(role for role in ("mixer", "input_filter") if role in parts)

    def run(self, ctx, parts, hidden, cache):
        composite = getattr(cache, "kind", "none") == "composite"
        if "input_filter" in parts:
            x = parts["norm_1"].forward(ctx, hidden, tag="norm_1", **_defer(parts["norm_1"], parts["input_filter"]))
            x = parts["input_filter"].forward(ctx, x, cache.of("input_filter") if composite else cache)
        else:
            x = parts["norm_1"].forward(ctx, hidden, tag="norm_1")
        y = parts["mixer"].compute(ctx, x, cache.of("mixer") if composite else cache)
        parts["norm_1b"].add_normed(ctx, hidden, y)
        if "feed_forward" in parts:
            x = parts["norm_2"].forward(ctx, hidden, tag="norm_2")
            parts["norm_2b"].add_normed(ctx, hidden, parts["feed_forward"].compute(ctx, x))
        if "depth_mix" in parts:
            parts["depth_mix"].forward(ctx, hidden)


class OutputNorm(Arrangement):
    roles = ("mixer", "norm_1")
    optional_roles = ("feed_forward", "norm_2")     # a layer may have no feed-forward

    @staticmethod
    def _stream(ctx, hidden):
        """What a sublayer reads: the 32-bit stream itself, or its rows rounded to the activations' type."""
        if ctx.act_dtype == hidden.dtype:
            return hidden
        if getattr(ctx, "rounded_stream", None) is None:
            ctx.rounded_stream = ctx.buffer("stream_rounded", tuple(hidden.shape), ctx.act_dtype)
            ctx.kernels.add_normed_cast(hidden, act=ctx.rounded_stream)
        return ctx.rounded_stream

    @staticmethod
    def _add(ctx, norm, hidden, y):
        if ctx.act_dtype == hidden.dtype:
            norm.add_normed(ctx, hidden, y)
        else:
            ctx.rounded_stream = ctx.buffer("stream_rounded", tuple(hidden.shape), ctx.act_dtype)
            norm.add_normed(ctx, hidden, y, rounded=ctx.rounded_stream)

    def run(self, ctx, parts, hidden, cache):
        if getattr(cache, "kind", "none") == "composite":
            cache = cache.sub("mixer")
        self._add(ctx, parts["norm_1"], hidden, parts["mixer"].compute(ctx, self._stream(ctx, hidden), cache))
        if "feed_forward" in parts:
            self._add(ctx, parts["norm_2"], hidden, parts["feed_forward"].compute(ctx, self._stream(ctx, hidden)))


class HyperConnections(Arrangement):
    roles = ("streams_1", "norm_1", "mixer")
    optional_roles = ("streams_2", "norm_2", "feed_forward")     # a layer may have no feed-forward

    def run(self, ctx, parts, hidden, cache):
        first = parts["streams_1"]
        x = first.read(ctx, parts["norm_1"], tag="norm_1")
        if getattr(cache, "kind", "none") == "composite":
            cache = cache.sub("mixer")
        y = parts["mixer"].compute(ctx, x, cache)
        # the layer's last write waits for the next read-out of the streams (the next layer's, or the model's sum)
        if "feed_forward" not in parts:
            first.write(ctx, y, defer=True)
            return
        # the mixer's result goes onto the streams and the feed-forward's input comes off them in one pass
        second = parts["streams_2"]
        x = first.write_then_read(ctx, y, second, parts["norm_2"], tag="norm_2")
        second.write(ctx, parts["feed_forward"].compute(ctx, x), defer=True)


register_arrangement("pre_norm", PreNorm())
register_arrangement("output_norm", OutputNorm())
register_arrangement("hyper_connections", HyperConnections())
register_arrangement("sandwich_norm", SandwichNorm())

"""Layer norm: mean, biased variance of the centred values, then
``(x - mean) / sqrt(var + eps) * gain + shift`` (engine/src/layernorm.c:12-33).
Statistics are 32-bit; the output has the engine's element type.

Norm by root mean square in groups (``grouped_rms_norm``): the row is cut into ``groups`` equal
consecutive pieces, each divided by ``sqrt(mean(piece^2) + eps)``, and the whole multiplied by one
gain vector; ``groups=1`` is the plain RMS norm.  Besides the interface of every norm it can norm
the residual stream in place and add a normed sublayer result onto it, which is what an
arrangement with norms on both sides of a sublayer needs.  With ``unit_offset`` the stored weight lies
around zero and the gain is ``1 + weight`` (added once, in 32-bit, when the weights arrive)."""

from __future__ import annotations

from ..kernels.dispatch import DeferredNorm
from .base import Norm, register_part
from .spec import WeightSpec


class LayerNorm(Norm):
    graph_safe = True
    can_defer = True

    def __init__(self, prefix, width: int, eps: float):
        super().__init__(prefix)
        self.width = int(width)
        self.eps = float(eps)

    def weight_specs(self):
        return [
            WeightSpec(self.full_name("weight"), (self.width,), role="vector", init="gain"),
            WeightSpec(self.full_name("bias"), (self.width,), role="vector", init="shift"),
        ]

    def forward(self, ctx, x, rows=None, tag="norm", defer=False):
        if defer:
            gamma, beta = self.w("weight"), self.w("bias")
            return DeferredNorm("layer_norm", x, rows, tag,
                                lambda c, out: c.kernels.layernorm(out, x, gamma, beta, self.eps, rows),
                                gamma=gamma, beta=beta, eps=self.eps)
        n_rows = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(tag, (n_rows, self.width), ctx.act_dtype)
        ctx.kernels.layernorm(out, x, self.w("weight"), self.w("bias"), self.eps, rows)
        return out


class GroupedRmsNorm(Norm):
    graph_safe = True
    can_defer = True

    def __init__(self, prefix, width: int, eps: float, groups: int = 1, name: str = "weight", unit_offset: bool = False):
        super().__init__(prefix)
        self.width, self.eps, self.groups, self.name = int(width), float(eps), int(groups), name
        self.unit_offset = bool(unit_offset)
        if self.groups <= 0 or self.width % self.groups != 0:
            raise ValueError(f"{self.full_name(name)}: a width of {self.width} does not split into {self.groups} equal groups")

    def weight_specs(self):
        return [WeightSpec(self.full_name(self.name), (self.width,), role="vector", init="shift" if self.unit_offset else "gain")]

    def bind(self, tensors, runtime):
        if self.unit_offset:
            name = self.full_name(self.name)
            tensors = {**tensors, name: tensors[name] + 1.0}
        super().bind(tensors, runtime)

    def forward(self, ctx, x, rows=None, tag="norm", defer=False):
        if defer:
            gain = self.w(self.name)
            return DeferredNorm("grouped_rms_norm", x, rows, tag,
                                lambda c, out: c.kernels.grouped_rms_norm(out, x, gain, self.groups, self.eps, rows),
                                gain=gain, groups=self.groups, eps=self.eps)
        n_rows = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(tag, (n_rows, self.width), ctx.act_dtype)
        ctx.kernels.grouped_rms_norm(out, x, self.w(self.name), self.groups, self.eps, rows)
        return out

    def normalize_in_place(self, ctx, hidden):
        """The fp32 stream itself is normed (after an embedding, for instance)."""
        ctx.kernels.grouped_rms_norm(hidden, hidden, self.w(self.name), self.groups, self.eps)
        return hidden

    def add_normed(self, ctx, hidden, y, rounded=None):
        """hidden += norm(y): a sublayer's fp32 result is normed on its way onto the stream.  ``rounded``: the
        stream's rows as they then are also go there, in that tensor's element type (the same pass where the
        norm is over the whole row)."""
        if rounded is not None and self.groups == 1:
            ctx.kernels.add_normed_cast(hidden, y, self.w(self.name), self.eps, rounded)
            return hidden
        ctx.kernels.grouped_rms_norm(hidden, y, self.w(self.name), self.groups, self.eps, add=True)
        if rounded is not None:
            ctx.kernels.add_normed_cast(hidden, act=rounded)
        return hidden


register_part("layer_norm", LayerNorm)
register_part("grouped_rms_norm", GroupedRmsNorm)

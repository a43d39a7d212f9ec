"""Dense feed-forward: ``act(x W_up + b_up) W_down + b_down``, added onto the
residual stream (engine/src/transformer_block.c:64-71).  The activation is a
parameter: the tanh form of gelu (engine/include/gelu_math.h:6-11) or the erf
form (engine/src/gelu.c:5-9), or the square of relu.  Biases are optional, and the tensors'
names are parameters (``weight_suffix=""`` for files that name a matrix by its layer alone).
``compute`` returns the output itself, in 32-bit, for arrangements that norm it before the sum.

``gated_mlp``: ``W_down (act(W_gate x + b_gate) * (W_up x + b_up)) + b_down``; gate and up are one
product over the stacked matrices, the activation and the product of the halves one pass."""

from __future__ import annotations

import torch

from .base import FeedForward, register_part
from .spec import WeightSpec

ACTIVATION_EPILOGUES = ("gelu_tanh", "gelu_erf", "relu_squared", "silu")


class DenseMlp(FeedForward):
    graph_safe = True
    def __init__(self, prefix, width: int, inner: int, activation: str,
                 up_name: str = "c_fc", down_name: str = "c_proj", stored_in_out: bool = True, bias: bool = True,
                 weight_suffix: str = ".weight"):
        super().__init__(prefix)
        self.width, self.inner = int(width), int(inner)
        if activation not in ACTIVATION_EPILOGUES:
            raise ValueError(f"{prefix}: unknown activation '{activation}' (known: {', '.join(ACTIVATION_EPILOGUES)})")
        self.activation = activation
        self.up_name, self.down_name = up_name, down_name
        self.stored_in_out = bool(stored_in_out)
        self.bias, self.weight_suffix = bool(bias), weight_suffix

    def _matrix_shape(self, n_in, n_out):
        return (n_in, n_out) if self.stored_in_out else (n_out, n_in)

    def weight_specs(self):
        t, suffix = self.stored_in_out, self.weight_suffix
        specs = [
            WeightSpec(self.full_name(f"{self.up_name}{suffix}"), self._matrix_shape(self.width, self.inner), transpose=t),
            WeightSpec(self.full_name(f"{self.down_name}{suffix}"), self._matrix_shape(self.inner, self.width), transpose=t,
                       init="residual_matrix"),
        ]
        if self.bias:
            specs.insert(1, WeightSpec(self.full_name(f"{self.up_name}.bias"), (self.inner,), role="vector", init="bias"))
            specs.append(WeightSpec(self.full_name(f"{self.down_name}.bias"), (self.width,), role="vector", init="bias"))
        return specs

    accepts_deferred_norm = True

    def _bias(self, name):
        return self.w(f"{name}.bias") if self.bias else None

    def _up(self, ctx, x):
        up = ctx.buffer("mlp_up", (x.shape[0], self.inner), ctx.act_dtype)
        ctx.kernels.linear(ctx, up, x, self.w(f"{self.up_name}{self.weight_suffix}"), self._bias(self.up_name),
                           epilogue=self.activation)
        return up

    def forward(self, ctx, x, hidden):
        ctx.kernels.linear(ctx, hidden, self._up(ctx, x), self.w(f"{self.down_name}{self.weight_suffix}"),
                           self._bias(self.down_name), epilogue="add")

    def compute(self, ctx, x):
        out = ctx.buffer("mlp_out", (x.shape[0], self.width), torch.float32)
        ctx.kernels.linear(ctx, out, self._up(ctx, x), self.w(f"{self.down_name}{self.weight_suffix}"),
                           self._bias(self.down_name))
        return out


class GatedMlp(FeedForward):
    graph_safe = True
    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, prefix, width: int, inner: int, activation: str = "silu", bias: bool = True, gate_name: str = "gate",
                 up_name: str = "up", down_name: str = "down", bias_suffix: str = ".b"):
        super().__init__(prefix)
        self.width, self.inner = int(width), int(inner)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"{prefix}: unknown gate activation '{activation}' (known: {', '.join(self.ACTIVATIONS)})")
        if min(self.width, self.inner) <= 0:
            raise ValueError(f"{prefix}: width and inner size must be positive")
        self.activation, self.bias, self.bias_suffix = activation, bool(bias), bias_suffix
        self.names = dict(gate=gate_name, up=up_name, down=down_name)

    def weight_specs(self):
        n = self.names
        specs = [WeightSpec(self.full_name(n["gate"]), (self.inner, self.width)),
                 WeightSpec(self.full_name(n["up"]), (self.inner, self.width)),
                 WeightSpec(self.full_name(n["down"]), (self.width, self.inner), init="residual_matrix")]
        if self.bias:
            specs += [WeightSpec(self.full_name(n[key] + self.bias_suffix), (size,), role="vector", init="bias")
                      for key, size in (("gate", self.inner), ("up", self.inner), ("down", self.width))]
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        self.stacked = torch.cat([self.w(n["gate"]), self.w(n["up"])]).contiguous()
        self.stacked_bias = (torch.cat([self.w(n["gate"] + self.bias_suffix), self.w(n["up"] + self.bias_suffix)]).contiguous()
                             if self.bias else None)
        self.down_bias = self.w(n["down"] + self.bias_suffix) if self.bias else None

    def _activated(self, ctx, x):
        both = ctx.buffer("mlp_gate_up", (x.shape[0], 2 * self.inner), ctx.act_dtype)
        ctx.kernels.linear(ctx, both, x, self.stacked, self.stacked_bias)
        act = ctx.buffer("mlp_up", (x.shape[0], self.inner), ctx.act_dtype)
        ctx.kernels.gated_act(act, both, self.activation)
        return act

    def forward(self, ctx, x, hidden):
        ctx.kernels.linear(ctx, hidden, self._activated(ctx, x), self.w(self.names["down"]), self.down_bias, epilogue="add")

    def compute(self, ctx, x):
        out = ctx.buffer("mlp_out", (x.shape[0], self.width), torch.float32)
        ctx.kernels.linear(ctx, out, self._activated(ctx, x), self.w(self.names["down"]), self.down_bias)
        return out


register_part("dense_mlp", DenseMlp)
register_part("gated_mlp", GatedMlp)

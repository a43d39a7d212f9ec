"""Mixers whose memory is a matrix per head that every token decays and writes with strengths of
its own: ``S <- a_t S + k_t u_t^T``, read after the write as ``S^T q_t``.  With
``step_t = softplus(w . x_t + step_bias[h])`` and ``a_t = exp(-exp(log_rate[h]) * step_t)``:

``gated_delta_memory`` (the gated delta rule): ``u_t = beta_t (v_t - (a_t S)^T k_t)`` with
    ``beta_t = sigmoid(w_b . x_t)``: the write replaces what the key read.  q, k and v pass a short
    causal convolution and silu; q and k are then unit vectors per head (``x / sqrt(sum(x^2) + 1e-6)``),
    q times ``dim^(-1/2)``; value head h reads query/key head ``h // (heads / qk_heads)``.  Each head's
    output is divided by its root mean square, multiplied by a gain shared by the heads and by
    ``silu(W_g x)``, then ``W_o``.
``state_space_duality`` (Mamba-2): one input product laid out as [z | x | B | C | dt]; x, B and C
    pass a causal convolution with bias and silu; ``u_t = step_t x_t``, key ``B_t`` and query ``C_t``
    per group (head h reads group ``h // (heads / groups)``), plus ``D[h] x_t`` on the output; the
    output times ``silu(z)`` is then normed in ``norm_groups`` equal parts, times a gain, then ``W_o``.

``channel_delta_memory``: the gated delta rule with one decay per head and key channel,
    ``a_t[h, i] = exp(-exp(log_rate[h]) * softplus((W_a2 (W_a1 x_t))[h, i] + step_bias[h, i]))``, which multiplies
    row i of S before the old state is read; the step's projection is a product of two thin
    matrices, and so is the output gate, which is ``sigmoid(W_g2 (W_g1 x))``.

``gated_linear_recurrence`` (the real-gated linear recurrent unit of Griffin): the state is a vector, one number per
    channel: ``S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t`` with ``a_t = exp(-decay_scale * r_t * softplus(lam))``; see the class.

State per request (32-bit, in its slot): S [heads, dim, vdim] and the convolution's last
``taps - 1`` inputs.  Steps, decays, write gates, unit norms and the recurrence are 32-bit; the
projections that feed gates and steps leave their product in 32-bit.
"""

from __future__ import annotations

import torch

from .base import Mixer, register_part
from .spec import FixedState, WeightSpec


def _padded_rows(matrix, least: int = 16):
    """The matrix with rows of zeros up to ``least`` output features (the least a tensor-core tile takes)."""
    if matrix.shape[0] >= least:
        return matrix.contiguous()
    out = torch.zeros((least, matrix.shape[1]), dtype=matrix.dtype, device=matrix.device)
    out[:matrix.shape[0]] = matrix
    return out


class GatedDeltaMemory(Mixer):
    graph_safe = True

    def __init__(self, prefix, width: int, n_heads: int, n_qk_heads: int, key_size: int, value_size: int, taps: int,
                 eps: float, names: dict | None = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.n_qk_heads = int(width), int(n_heads), int(n_qk_heads)
        self.dim, self.vdim, self.taps, self.eps = int(key_size), int(value_size), int(taps), float(eps)
        if min(self.n_heads, self.n_qk_heads, self.dim, self.vdim) <= 0 or self.n_heads % self.n_qk_heads != 0:
            raise ValueError(f"{prefix}: {self.n_heads} heads are not a positive multiple of {self.n_qk_heads} query/key heads")
        if self.taps < 1:
            raise ValueError(f"{prefix}: a convolution has at least one tap")
        self.names = dict(q="q", k="k", v="v", g="g", o="o", norm="norm", write="b", step="a", log_rate="A_log",
                          step_bias="dt_bias", taps=".conv")
        self.names.update(names or {})
        self.qk, self.vw = self.n_qk_heads * self.dim, self.n_heads * self.vdim
        self.filtered = 2 * self.qk + self.vw

    def weight_specs(self):
        n, h = self.names, self.n_heads
        specs = []
        for name, rows in ((n["q"], self.qk), (n["k"], self.qk), (n["v"], self.vw)):
            specs += [WeightSpec(self.full_name(name), (rows, self.width)),
                      WeightSpec(self.full_name(name + n["taps"]), (rows, self.taps), role="vector", init="matrix")]
        return specs + [
            WeightSpec(self.full_name(n["write"]), (h, self.width)),
            WeightSpec(self.full_name(n["step"]), (h, self.width)),
            WeightSpec(self.full_name(n["log_rate"]), (h,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["step_bias"]), (h,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["norm"]), (self.vdim,), role="vector", init="gain"),
            WeightSpec(self.full_name(n["g"]), (self.vw, self.width)),
            WeightSpec(self.full_name(n["o"]), (self.width, self.vw), init="residual_matrix"),
        ]

    def cache_need(self):
        need = {"state": FixedState((self.n_heads * self.dim * self.vdim,), "float32")}
        if self.taps > 1:
            need["taps"] = FixedState((self.taps - 1, self.filtered), "float32")
        return need

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        self.stacked = torch.cat([self.w(n["q"]), self.w(n["k"]), self.w(n["v"]), self.w(n["g"])]).contiguous()
        self.stacked_taps = torch.cat([self.w(name + n["taps"]) for name in (n["q"], n["k"], n["v"])]).contiguous()
        self.gate_matrix = _padded_rows(torch.cat([self.w(n["step"]), self.w(n["write"])]))
        self.gain = self.w(n["norm"]).repeat(self.n_heads).contiguous()
        self._no_state = torch.zeros((1, 0, self.filtered), dtype=torch.float32, device=self.stacked.device)

    def compute(self, ctx, x, cache):
        k, n, h = ctx.kernels, x.shape[0], self.n_heads
        projected = ctx.buffer("memory_qkvg", (n, self.filtered + self.vw), ctx.act_dtype)
        k.linear(ctx, projected, x, self.stacked)
        held = cache.of("taps") if self.taps > 1 else None
        filtered = ctx.buffer("memory_filtered", (n, self.filtered), ctx.act_dtype)
        k.causal_taps(ctx, filtered, projected[:, :self.filtered], self.stacked_taps,
                      held.state if held is not None else self._no_state, held.writes if held is not None else False,
                      identity=False, silu=True)
        gates = ctx.buffer("memory_gates", (n, self.gate_matrix.shape[0]), torch.float32)
        k.linear(ctx, gates, x, self.gate_matrix)
        read = ctx.buffer("memory_read", (n, self.vw), torch.float32)
        state = cache.of("state")
        k.linear_recurrence(ctx, read, filtered[:, :self.qk], filtered[:, self.qk:2 * self.qk], filtered[:, 2 * self.qk:],
                            gates[:, :h], gates[:, h:2 * h], self.w(self.names["log_rate"]), self.w(self.names["step_bias"]),
                            state.state, h, self.n_qk_heads, self.dim, self.vdim, delta=True, unit_norm=True,
                            q_scale=self.dim ** -0.5, writes=state.writes)
        mixed = ctx.buffer("attn_out", (n, self.vw), ctx.act_dtype)
        k.grouped_rms_norm(mixed, read, self.gain, h, self.eps, gate=projected[:, self.filtered:], gate_mode="silu")
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(self.names["o"]))
        return out

    def forward(self, ctx, x, hidden, cache):
        ctx.kernels.scaled_add(hidden, self.compute(ctx, x, cache), 1.0)


class ChannelDeltaMemory(GatedDeltaMemory):
    """``gated_delta_memory`` with a decay per key channel and thin pairs of matrices for the decay's
    step (``step_rank``) and for the output gate (``gate_rank``, a sigmoid gate).  An inner size of
    None is read off the stored matrices."""

    def __init__(self, prefix, width: int, n_heads: int, n_qk_heads: int, key_size: int, value_size: int, taps: int,
                 eps: float, step_rank: int | None = None, gate_rank: int | None = None, names: dict | None = None):
        more = dict(step_down="a1", step_up="a2", gate_down="g1", gate_up="g2")
        more.update(names or {})
        super().__init__(prefix, width, n_heads, n_qk_heads, key_size, value_size, taps, eps, more)
        self.step_rank = int(step_rank) if step_rank is not None else None
        self.gate_rank = int(gate_rank) if gate_rank is not None else None
        if min(self.step_rank or 1, self.gate_rank or 1) <= 0:
            raise ValueError(f"{prefix}: the thin matrices' inner sizes must be positive")

    def weight_specs(self):
        n, h = self.names, self.n_heads
        specs = []
        for name, rows in ((n["q"], self.qk), (n["k"], self.qk), (n["v"], self.vw)):
            specs += [WeightSpec(self.full_name(name), (rows, self.width)),
                      WeightSpec(self.full_name(name + n["taps"]), (rows, self.taps), role="vector", init="matrix")]
        return specs + [
            WeightSpec(self.full_name(n["write"]), (h, self.width)),
            WeightSpec(self.full_name(n["log_rate"]), (h,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["norm"]), (self.vdim,), role="vector", init="gain"),
            WeightSpec(self.full_name(n["step_down"]), (self.step_rank, self.width)),
            WeightSpec(self.full_name(n["step_up"]), (h * self.dim, self.step_rank)),
            WeightSpec(self.full_name(n["step_bias"]), (h * self.dim,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["gate_down"]), (self.gate_rank, self.width)),
            WeightSpec(self.full_name(n["gate_up"]), (self.vw, self.gate_rank)),
            WeightSpec(self.full_name(n["o"]), (self.width, self.vw), init="residual_matrix"),
        ]

    def bind(self, tensors, runtime):
        Mixer.bind(self, tensors, runtime)
        n = self.names
        for down, up in (("step_down", "step_up"), ("gate_down", "gate_up")):
            if self.w(n[down]).shape[0] != self.w(n[up]).shape[1]:
                raise ValueError(f"{self.full_name(n[down])} has {self.w(n[down]).shape[0]} rows but {self.full_name(n[up])} "
                                 f"has {self.w(n[up]).shape[1]} columns")
        self.step_rank, self.gate_rank = self.w(n["step_down"]).shape[0], self.w(n["gate_down"]).shape[0]
        self.stacked = torch.cat([self.w(n["q"]), self.w(n["k"]), self.w(n["v"])]).contiguous()
        self.stacked_taps = torch.cat([self.w(name + n["taps"]) for name in (n["q"], n["k"], n["v"])]).contiguous()
        self.write_matrix = _padded_rows(self.w(n["write"]))
        self.gain = self.w(n["norm"]).repeat(self.n_heads).contiguous()
        self._no_state = torch.zeros((1, 0, self.filtered), dtype=torch.float32, device=self.stacked.device)

    def compute(self, ctx, x, cache):
        k, n, h, names = ctx.kernels, x.shape[0], self.n_heads, self.names
        projected = ctx.buffer("memory_qkvg", (n, self.filtered), ctx.act_dtype)
        k.linear(ctx, projected, x, self.stacked)
        held = cache.of("taps") if self.taps > 1 else None
        filtered = ctx.buffer("memory_filtered", (n, self.filtered), ctx.act_dtype)
        k.causal_taps(ctx, filtered, projected, self.stacked_taps,
                      held.state if held is not None else self._no_state, held.writes if held is not None else False,
                      identity=False, silu=True)
        # the thin pairs: the steps stay 32-bit (they enter the recurrence), the output gate is an activation
        thin = ctx.buffer("memory_step_thin", (n, self.step_rank), ctx.act_dtype)
        k.linear(ctx, thin, x, self.w(names["step_down"]))
        steps = ctx.buffer("memory_steps", (n, h * self.dim), torch.float32)
        k.linear(ctx, steps, thin, self.w(names["step_up"]))
        thin = ctx.buffer("memory_gate_thin", (n, self.gate_rank), ctx.act_dtype)
        k.linear(ctx, thin, x, self.w(names["gate_down"]))
        gate = ctx.buffer("memory_gate", (n, self.vw), ctx.act_dtype)
        k.linear(ctx, gate, thin, self.w(names["gate_up"]))
        writes = ctx.buffer("memory_gates", (n, self.write_matrix.shape[0]), torch.float32)
        k.linear(ctx, writes, x, self.write_matrix)
        read = ctx.buffer("memory_read", (n, self.vw), torch.float32)
        state = cache.of("state")
        k.linear_recurrence(ctx, read, filtered[:, :self.qk], filtered[:, self.qk:2 * self.qk], filtered[:, 2 * self.qk:],
                            steps, writes[:, :h], self.w(names["log_rate"]), self.w(names["step_bias"]), state.state, h,
                            self.n_qk_heads, self.dim, self.vdim, delta=True, unit_norm=True, q_scale=self.dim ** -0.5,
                            writes=state.writes, channel_decay=True)
        mixed = ctx.buffer("attn_out", (n, self.vw), ctx.act_dtype)
        k.grouped_rms_norm(mixed, read, self.gain, h, self.eps, gate=gate, gate_mode="sigmoid")
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(names["o"]))
        return out


class StateSpaceDuality(Mixer):
    graph_safe = True

    def __init__(self, prefix, width: int, n_heads: int, value_size: int, state_size: int, n_groups: int,
                 norm_groups: int, taps: int, eps: float, names: dict | None = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.vdim, self.state_size = int(width), int(n_heads), int(value_size), int(state_size)
        self.n_groups, self.norm_groups, self.taps, self.eps = int(n_groups), int(norm_groups), int(taps), float(eps)
        if min(self.n_heads, self.vdim, self.state_size, self.n_groups) <= 0 or self.n_heads % self.n_groups != 0:
            raise ValueError(f"{prefix}: {self.n_heads} heads are not a positive multiple of {self.n_groups} groups")
        self.inner, self.bc = self.n_heads * self.vdim, self.n_groups * self.state_size
        if self.norm_groups <= 0 or self.inner % self.norm_groups != 0:
            raise ValueError(f"{prefix}: {self.inner} inner channels do not split into {self.norm_groups} equal parts")
        if self.taps < 1:
            raise ValueError(f"{prefix}: a convolution has at least one tap")
        self.names = dict(input="in", taps="conv", taps_bias="conv.b", step_bias="dt_bias", log_rate="A_log", skip="D",
                          norm="norm", o="o")
        self.names.update(names or {})
        self.filtered = self.inner + 2 * self.bc

    def weight_specs(self):
        n, h = self.names, self.n_heads
        return [
            WeightSpec(self.full_name(n["input"]), (2 * self.inner + 2 * self.bc + h, self.width)),
            WeightSpec(self.full_name(n["taps"]), (self.filtered, self.taps), role="vector", init="matrix"),
            WeightSpec(self.full_name(n["taps_bias"]), (self.filtered,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["step_bias"]), (h,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["log_rate"]), (h,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["skip"]), (h,), role="vector", init="gain"),
            WeightSpec(self.full_name(n["norm"]), (self.inner,), role="vector", init="gain"),
            WeightSpec(self.full_name(n["o"]), (self.width, self.inner), init="residual_matrix"),
        ]

    def cache_need(self):
        need = {"state": FixedState((self.n_heads * self.state_size * self.vdim,), "float32")}
        if self.taps > 1:
            need["taps"] = FixedState((self.taps - 1, self.filtered), "float32")
        return need

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        full = self.w(self.names["input"])
        cut = self.inner + self.filtered
        self.main = full[:cut].contiguous()                       # z, x, B, C
        self.step_matrix = _padded_rows(full[cut:])               # dt, whose product stays 32-bit
        self._no_state = torch.zeros((1, 0, self.filtered), dtype=torch.float32, device=full.device)

    def compute(self, ctx, x, cache):
        k, n, names = ctx.kernels, x.shape[0], self.names
        projected = ctx.buffer("memory_qkvg", (n, self.inner + self.filtered), ctx.act_dtype)
        k.linear(ctx, projected, x, self.main)
        held = cache.of("taps") if self.taps > 1 else None
        filtered = ctx.buffer("memory_filtered", (n, self.filtered), ctx.act_dtype)
        k.causal_taps(ctx, filtered, projected[:, self.inner:], self.w(names["taps"]),
                      held.state if held is not None else self._no_state, held.writes if held is not None else False,
                      identity=False, bias=self.w(names["taps_bias"]), silu=True)
        steps = ctx.buffer("memory_gates", (n, self.step_matrix.shape[0]), torch.float32)
        k.linear(ctx, steps, x, self.step_matrix)
        read = ctx.buffer("memory_read", (n, self.inner), torch.float32)
        state = cache.of("state")
        k.linear_recurrence(ctx, read, filtered[:, self.inner + self.bc:], filtered[:, self.inner:self.inner + self.bc],
                            filtered[:, :self.inner], steps[:, :self.n_heads], None, self.w(names["log_rate"]),
                            self.w(names["step_bias"]), state.state, self.n_heads, self.n_groups, self.state_size, self.vdim,
                            delta=False, skip=self.w(names["skip"]), writes=state.writes)
        mixed = ctx.buffer("attn_out", (n, self.inner), ctx.act_dtype)
        k.grouped_rms_norm(mixed, read, self.w(names["norm"]), self.norm_groups, self.eps, gate=projected[:, :self.inner],
                           gate_mode="silu_before")
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(names["o"]))
        return out

    def forward(self, ctx, x, hidden, cache):
        ctx.kernels.scaled_add(hidden, self.compute(ctx, x, cache), 1.0)


class GatedLinearRecurrence(Mixer):
    """A recurrent block with two branches of ``inner`` channels: ``y = gelu_tanh(W_y x + b_y)`` and
    ``u = conv(W_x x + b_x)``, a causal convolution per channel with a bias and no activation (the last ``taps - 1``
    inputs of a request are state).  The channels are cut into ``blocks`` equal parts; in part b,
    ``r = sigmoid(A_r[b] u_b + b_r[b])`` and ``i = sigmoid(A_i[b] u_b + b_i[b])`` with square matrices.  Then per channel
    ``a = exp(-decay_scale * r * softplus(lam))`` and ``S_t = a S_(t-1) + sqrt(1 - a^2) * i * u`` from S = 0 (no special
    case for a first token); the output is ``W_o (S * y)``.  Both input products are one product over the stacked
    matrices and both gates one product per part; gates, decays and the state are 32-bit."""

    graph_safe = True

    def __init__(self, prefix, width: int, inner: int, blocks: int, taps: int, decay_scale: float = 8.0, names: dict | None = None):
        super().__init__(prefix)
        self.width, self.inner, self.blocks, self.taps = int(width), int(inner), int(blocks), int(taps)
        self.decay_scale = float(decay_scale)
        if self.blocks <= 0 or self.inner <= 0 or self.inner % self.blocks != 0:
            raise ValueError(f"{prefix}: {self.inner} channels do not split into {self.blocks} equal parts")
        if self.taps < 1:
            raise ValueError(f"{prefix}: a convolution has at least one tap")
        self.part = self.inner // self.blocks
        self.names = dict(y="y", x="x", bias=".b", taps="conv", taps_bias="conv.b", gate_r="ra", gate_i="ri", rate="lam", o="o")
        self.names.update(names or {})

    def weight_specs(self):
        n, part = self.names, self.part
        return [
            WeightSpec(self.full_name(n["y"]), (self.inner, self.width)),
            WeightSpec(self.full_name(n["y"] + n["bias"]), (self.inner,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["x"]), (self.inner, self.width)),
            WeightSpec(self.full_name(n["x"] + n["bias"]), (self.inner,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["taps"]), (self.inner, self.taps), role="vector", init="matrix"),
            WeightSpec(self.full_name(n["taps_bias"]), (self.inner,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["gate_r"]), (self.blocks, part, part)),
            WeightSpec(self.full_name(n["gate_r"] + n["bias"]), (self.blocks, part), role="vector", init="bias"),
            WeightSpec(self.full_name(n["gate_i"]), (self.blocks, part, part)),
            WeightSpec(self.full_name(n["gate_i"] + n["bias"]), (self.blocks, part), role="vector", init="bias"),
            WeightSpec(self.full_name(n["rate"]), (self.inner,), role="vector", init="shift"),
            WeightSpec(self.full_name(n["o"]), (self.width, self.inner), init="residual_matrix"),
        ]

    def cache_need(self):
        need = {"state": FixedState((self.inner,), "float32")}
        if self.taps > 1:
            need["taps"] = FixedState((self.taps - 1, self.inner), "float32")
        return need

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        self.stacked = torch.cat([self.w(n["y"]), self.w(n["x"])]).contiguous()
        self.stacked_bias = torch.cat([self.w(n["y"] + n["bias"]), self.w(n["x"] + n["bias"])]).contiguous()
        # per part: the rows of its r gate, then those of its i gate
        self.gate_matrices = torch.cat([self.w(n["gate_r"]), self.w(n["gate_i"])], dim=1).contiguous()
        self.bias_r = self.w(n["gate_r"] + n["bias"]).reshape(-1).contiguous()
        self.bias_i = self.w(n["gate_i"] + n["bias"]).reshape(-1).contiguous()
        self._no_state = torch.zeros((1, 0, self.inner), dtype=torch.float32, device=self.stacked.device)

    def compute(self, ctx, x, cache):
        k, n, names, inner = ctx.kernels, x.shape[0], self.names, self.inner
        both = ctx.buffer("unit_branches", (n, 2 * inner), ctx.act_dtype)
        k.linear(ctx, both, x, self.stacked, self.stacked_bias)
        held = cache.of("taps") if self.taps > 1 else None
        u = ctx.buffer("unit_filtered", (n, inner), ctx.act_dtype)
        k.causal_taps(ctx, u, both[:, inner:], self.w(names["taps"]), held.state if held is not None else self._no_state,
                      held.writes if held is not None else False, identity=False, bias=self.w(names["taps_bias"]))
        gates = ctx.buffer("unit_gates", (n, 2 * inner), torch.float32)
        k.head_linear(ctx, gates, u, self.gate_matrices, self.blocks, self.part, 2 * self.part)
        state = cache.of("state")
        mixed = ctx.buffer("attn_out", (n, inner), ctx.act_dtype)
        k.gated_recurrence(ctx, mixed, u, both[:, :inner], gates, self.bias_r, self.bias_i, self.w(names["rate"]),
                           self.decay_scale, state.state, self.part, state.writes)
        out = ctx.buffer("unit_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(names["o"]))
        return out

    def forward(self, ctx, x, hidden, cache):
        ctx.kernels.scaled_add(hidden, self.compute(ctx, x, cache), 1.0)


class ParallelMixers(Mixer):
    """Several mixers side by side on one input: the stream gets ``sum_i scale_i * mixer_i(x)``.
    ``branches``: a tuple of (name, description of the mixer, scale); each mixer has ``compute`` and
    keeps its own cache under its name."""

    def __init__(self, prefix, branches):
        super().__init__(prefix)
        from .base import build_part
        self.branches = [(str(name), build_part(spec), float(scale)) for name, spec, scale in branches]
        if not self.branches:
            raise ValueError(f"{prefix}: no mixers")
        for name, part, _ in self.branches:
            if not hasattr(part, "compute"):
                raise ValueError(f"{prefix}: the mixer '{name}' cannot hand over its output (no compute)")
        self.graph_safe = all(getattr(part, "graph_safe", False) for _, part, _ in self.branches)
        self.wants_attention_tiles = any(getattr(part, "wants_attention_tiles", False) for _, part, _ in self.branches)

    def weight_specs(self):
        return [spec for _, part, _ in self.branches for spec in part.weight_specs()]

    def cache_need(self):
        need = {}
        for name, part, _ in self.branches:
            mine = part.cache_need()
            if isinstance(mine, dict):
                need.update({f"{name}.{key}": one for key, one in mine.items()})
            else:
                need[name] = mine
        return need

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        for _, part, _ in self.branches:
            part.bind({w.name: tensors[w.name] for w in part.weight_specs() if w.name in tensors}, runtime)

    def forward(self, ctx, x, hidden, cache):
        for name, part, scale in self.branches:
            mine = cache.sub(name) if isinstance(part.cache_need(), dict) else cache.of(name)
            ctx.kernels.scaled_add(hidden, part.compute(ctx, x, mine), scale)

    def compute(self, ctx, x, cache):
        """The weighted sum itself, in 32-bit, for arrangements that norm a mixer's output before the residual sum."""
        out = ctx.buffer("parallel_out", tuple(x.shape), torch.float32)      # (every mixer maps the width onto itself)
        if len(self.branches) == 2:
            # two sides: both results go into the sum in one pass
            (name_a, part_a, scale_a), (name_b, part_b, scale_b) = self.branches
            mine = lambda name, part: cache.sub(name) if isinstance(part.cache_need(), dict) else cache.of(name)
            first, second = part_a.compute(ctx, x, mine(name_a, part_a)), part_b.compute(ctx, x, mine(name_b, part_b))
            if first.data_ptr() != second.data_ptr():
                ctx.kernels.scaled_add(out, first, scale_a, second, scale_b, assign=True)
                return out
            raise RuntimeError(f"{self.prefix}: the two mixers hand over their results in one buffer")
        out.zero_()
        self.forward(ctx, x, out, cache)
        return out


register_part("gated_delta_memory", GatedDeltaMemory)
register_part("channel_delta_memory", ChannelDeltaMemory)
register_part("state_space_duality", StateSpaceDuality)
register_part("gated_linear_recurrence", GatedLinearRecurrence)
register_part("parallel_mixers", ParallelMixers)

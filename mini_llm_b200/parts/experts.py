"""Routed feed-forward (mixture of experts) with sigmoid scores.

Router logits ``z = W_router x`` and scores ``s = sigmoid(z)`` in 32-bit; each token takes the
``top`` experts with the largest scores.  The weight of a chosen expert is its score (not
renormalized) and multiplies the expert's INPUT: the layer adds ``sum_e expert_e(s_e * x)`` onto
the stream, with ``expert(u) = W_down (silu(W_gate u) * (W_up u))`` and no biases.  A shared expert of
the same form (with an inner size of its own) may run for every token; its output is multiplied
by ``sigmoid(w_sg . x)``, one number per token.

``weights="softmax_of_chosen"`` is the other common rule: the logits themselves (plus ``router_bias``, one number per
expert, if the model has one) rank the experts, the chosen experts' OUTPUTS are weighed by the softmax over the
chosen logits only, and their inputs are the token itself.  ``shared_gate=False``: the shared expert has no
gate and is simply added.

Experts are named by tables of pointers and inner sizes, so the shared expert goes through the
kernels as one more chosen expert with input weight 1 and its gate as the output weight.  A step
of few tokens runs pair by pair (token, chosen expert) and reads only the chosen experts'
matrices.  A step of many tokens runs two products over all experts at once: an expert a token
did not choose weighs 0 there, ``expert(0) = 0`` exactly, and the score multiplies the result
of the first product instead of its input (``W (s x) = s (W x)``).
"""

from __future__ import annotations

import torch

from .base import FeedForward, register_part
from .spec import WeightSpec


class RoutedExperts(FeedForward):
    graph_safe = True

    WEIGHTS = ("sigmoid_on_input", "softmax_of_chosen")

    def __init__(self, prefix, width: int, n_experts: int, top: int, expert_inner: int, shared_inner: int | None = None,
                 names: dict | None = None, weights: str = "sigmoid_on_input", router_bias: bool = False,
                 shared_gate: bool = True):
        super().__init__(prefix)
        if weights not in self.WEIGHTS:
            raise ValueError(f"{prefix}: unknown rule for the experts' weights '{weights}' (known: {', '.join(self.WEIGHTS)})")
        self.weights_rule, self.router_bias, self.shared_gate = weights, bool(router_bias), bool(shared_gate)
        self.width, self.n_experts, self.top, self.inner = int(width), int(n_experts), int(top), int(expert_inner)
        self.shared_inner = int(shared_inner) if shared_inner else None
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"{prefix}: every token takes between 1 and {self.n_experts} experts, got {self.top}")
        if self.inner <= 0:
            raise ValueError(f"{prefix}: the experts' inner size must be positive")
        self.names = dict(router="router", router_bias="router.b", expert="e{index}", shared="shared", shared_gate="shared.sg",
                          gate="gate", up="up", down="down")
        self.names.update(names or {})
        self.pairs = self.top + (1 if self.shared_inner else 0)

    def _expert_names(self):
        found = [(self.names["expert"].format(index=e), self.inner) for e in range(self.n_experts)]
        if self.shared_inner:
            found.append((self.names["shared"], self.shared_inner))
        return found

    def weight_specs(self):
        n = self.names
        specs = [WeightSpec(self.full_name(n["router"]), (self.n_experts, self.width))]
        for name, inner in self._expert_names():
            specs += [WeightSpec(self.full_name(f"{name}.{n['gate']}"), (inner, self.width)),
                      WeightSpec(self.full_name(f"{name}.{n['up']}"), (inner, self.width)),
                      WeightSpec(self.full_name(f"{name}.{n['down']}"), (self.width, inner), init="residual_matrix")]
        if self.shared_inner and self.shared_gate:
            specs.append(WeightSpec(self.full_name(n["shared_gate"]), (1, self.width)))
        if self.router_bias:
            specs.append(WeightSpec(self.full_name(n["router_bias"]), (self.n_experts,), role="vector", init="bias"))
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        experts = self._expert_names()
        router = self.w(n["router"])
        device = router.device
        # All gates, then all ups, as the rows of one matrix; all down matrices side by side as the
        # columns of another.  An expert's own matrices are row and column ranges of these (the pair
        # kernels get them by pointer), so a step of many tokens can run two products over all
        # experts and a step of few tokens reads only the experts it chose, from the same memory.
        self.total = sum(inner for _, inner in experts)
        self.up_matrix = torch.cat([self.w(f"{name}.{n[which]}") for which in ("gate", "up") for name, _ in experts]).contiguous()
        self.down_matrix = torch.cat([self.w(f"{name}.{n['down']}") for name, _ in experts], dim=1).contiguous()
        starts = [sum(inner for _, inner in experts[:e]) for e in range(len(experts))]
        size = self.up_matrix.element_size()

        def table(base, offsets):
            return torch.tensor([base + offset * size for offset in offsets], dtype=torch.int64, device=device)

        self.gate_of = table(self.up_matrix.data_ptr(), [start * self.width for start in starts])
        self.up_of = table(self.up_matrix.data_ptr(), [(self.total + start) * self.width for start in starts])
        self.down_of = table(self.down_matrix.data_ptr(), starts)
        self.inner_of = torch.tensor([inner for _, inner in experts], dtype=torch.int32, device=device)
        self.max_inner = max(inner for _, inner in experts)
        # the loaded matrices are held in the stacked ones now
        self.weights = {name: tensor for name, tensor in self.weights.items()
                        if name in (self.full_name(n["router"]), self.full_name(n["shared_gate"]), self.full_name(n["router_bias"]))}

    def forward(self, ctx, x, hidden, assign=False):
        """``assign``: ``hidden`` becomes the experts' sum instead of growing by it."""
        k, n = ctx.kernels, x.shape[0]
        choice = ctx.buffer("expert_choice", (n * self.pairs,), torch.int32)
        in_weight = ctx.buffer("expert_in_weight", (n * self.pairs,), torch.float32)
        out_weight = ctx.buffer("expert_out_weight", (n * self.pairs,), torch.float32)
        gated = self.shared_inner and self.shared_gate
        k.route(x, self.w(self.names["router"]), self.w(self.names["shared_gate"]) if gated else None, self.top,
                choice, in_weight, out_weight, bias=self.w(self.names["router_bias"]) if self.router_bias else None,
                softmax_of_chosen=self.weights_rule == "softmax_of_chosen", shared_plain=bool(self.shared_inner) and not gated)
        if k.experts_at_once(n, x, self.up_matrix, self.down_matrix):
            gu = ctx.buffer("expert_gate_up", (n, 2 * self.total), ctx.act_dtype)
            k.linear(ctx, gu, x, self.up_matrix)
            act = ctx.buffer("expert_act_all", (n, self.total), ctx.act_dtype)
            k.expert_combine(act, gu, choice, in_weight, out_weight, self.n_experts, self.inner, self.top, self.pairs)
            k.linear(ctx, hidden, act, self.down_matrix, None, epilogue="store" if assign else "add")
            return
        act = ctx.buffer("expert_act", (n * self.pairs, self.max_inner), ctx.act_dtype)
        k.experts(hidden, act, x, choice, in_weight, out_weight, self.gate_of, self.up_of, self.down_of, self.inner_of,
                  self.max_inner, self.pairs, ld_down=self.total, assign=assign)

    def compute(self, ctx, x):
        out = ctx.buffer("mlp_out", (x.shape[0], self.width), torch.float32)
        self.forward(ctx, x, out, assign=True)
        return out


register_part("routed_experts", RoutedExperts)

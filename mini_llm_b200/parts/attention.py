"""Causal self-attention over the paged cache.

One fused projection gives queries, keys and values (the reference splits the
fused ``c_attn`` matrix into three at load, engine/src/gpt2.c:79-90; here it
stays one product).  Head ``h`` is the column range ``h*D .. h*D+D-1`` of q, k,
v and of the output (engine/src/attention.c:78-87).  Scores are
``(q . k) * score_scale`` over the keys at positions ``<=`` the query's
(engine/src/attention.c:24-35, engine/src/softmax.c:29-55); the softmax and
the weighted sum of values run in 32-bit.  The output projection adds its
result and bias onto the block's input (engine/src/transformer_block.c:60-62).

The keys and values of this step's tokens are first stored into the request's
pages; attention then reads the cache only, so a prompt portion and a single
decoded token take the same path.

A position encoding that acts on queries and keys (a rotation, for instance)
is a parameter of the mixer: ``position``, the description of a
``PositionEncoding`` part with ``rotate(ctx, q, k, n_heads, n_kv_heads,
head_size)``, which changes the step's queries [T, heads * head_size] and
keys [T, kv_heads * head_size] in place, each row by its ``ctx.positions``.
The projection then writes q, k and v side by side, the encoding rotates, and
the keys and values are stored into the pages by a pass of their own (the
fused projection, which scatters straight into the pages, knows no rotation).
"""

from __future__ import annotations

import torch

from .base import Mixer, build_part, register_part
from .spec import FixedState, PagedKV, WeightSpec


class CausalSelfAttention(Mixer):
    graph_safe = True
    wants_attention_tiles = True      # its prompt kernel reads the step's work list of (128 queries, entry) tiles
    # (set per instance: its head count if it can also read a work list of units of 256 queries, else 0)
    attention_unit_heads = 0
    def __init__(self, prefix, width: int, n_heads: int, head_size: int, score_scale: float,
                 n_kv_heads: int | None = None, window: int | None = None,
                 qkv_name: str = "c_attn", out_name: str = "c_proj", stored_in_out: bool = True,
                 position=None):
        super().__init__(prefix)
        self.width = int(width)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads if n_kv_heads is not None else n_heads)
        self.head_size = int(head_size)
        self.attention_unit_heads = self.n_heads if self.head_size == 64 else 0
        self.score_scale = float(score_scale)
        self.window = int(window) if window else None
        self.qkv_name, self.out_name = qkv_name, out_name
        self.stored_in_out = bool(stored_in_out)
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"{prefix}: {self.n_heads} heads are not a multiple of {self.n_kv_heads} key/value heads")
        if self.head_size % 16 != 0 or not 16 <= self.head_size <= 256:
            raise ValueError(f"{prefix}: head size {self.head_size} is not a multiple of 16 in 16..256")
        self.position = build_part(position) if position is not None else None
        if self.position is not None:
            if not hasattr(self.position, "rotate"):
                raise ValueError(f"{prefix}: the position encoding '{position.kind}' has no rotate(ctx, q, k, ...)")
            self.graph_safe = bool(getattr(self.position, "graph_safe", False))
        self.q_width = self.n_heads * self.head_size
        self.kv_width = self.n_kv_heads * self.head_size
        self.qkv_width = self.q_width + 2 * self.kv_width

    def _matrix_shape(self, n_in, n_out):
        return (n_in, n_out) if self.stored_in_out else (n_out, n_in)

    def weight_specs(self):
        t = self.stored_in_out
        return (self.position.weight_specs() if self.position is not None else []) + [
            WeightSpec(self.full_name(f"{self.qkv_name}.weight"), self._matrix_shape(self.width, self.qkv_width), transpose=t),
            WeightSpec(self.full_name(f"{self.qkv_name}.bias"), (self.qkv_width,), role="vector", init="bias"),
            WeightSpec(self.full_name(f"{self.out_name}.weight"), self._matrix_shape(self.q_width, self.width), transpose=t,
                       init="residual_matrix"),
            WeightSpec(self.full_name(f"{self.out_name}.bias"), (self.width,), role="vector", init="bias"),
        ]

    def cache_need(self):
        return PagedKV(self.n_kv_heads, self.head_size, self.window)

    accepts_deferred_norm = True

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        if self.position is not None:
            self.position.bind({w.name: tensors[w.name] for w in self.position.weight_specs() if w.name in tensors},
                               runtime)

    def forward(self, ctx, x, hidden, cache):
        k = ctx.kernels
        if self.position is None:
            q = k.qkv_projection(ctx, x, self.w(f"{self.qkv_name}.weight"), self.w(f"{self.qkv_name}.bias"), cache,
                                 self.q_width, self.kv_width)
        else:
            qkv = ctx.buffer("qkv", (x.shape[0], self.qkv_width), ctx.act_dtype)
            k.linear(ctx, qkv, x, self.w(f"{self.qkv_name}.weight"), self.w(f"{self.qkv_name}.bias"))
            q, keys = qkv[:, :self.q_width], qkv[:, self.q_width:self.q_width + self.kv_width]
            self.position.rotate(ctx, q, keys, self.n_heads, self.n_kv_heads, self.head_size)
            if cache.writes:
                k.kv_store(cache.k_pages, cache.v_pages, keys, qkv[:, self.q_width + self.kv_width:], ctx.positions,
                           ctx.token_item, cache.block_table, cache.page_size)
        mixed = ctx.buffer("attn_out", (q.shape[0], self.q_width), ctx.act_dtype)
        k.attention(ctx, mixed, q, cache, self.n_heads, self.n_kv_heads, self.head_size, self.score_scale,
                    self.window or 0)
        k.linear(ctx, hidden, mixed, self.w(f"{self.out_name}.weight"), self.w(f"{self.out_name}.bias"),
                 epilogue="add")


class FilteredAttention(Mixer):
    """Causal attention whose queries, keys and values pass a short causal convolution over time
    before rotary positions, with a tanh cap on the scores and values of a size of their own.

    ``q = W_q x + b_q`` and likewise k, v (one product over the stacked matrices); every channel of
    q, k and v is then filtered, ``y_t = sum_j w[:, j] u_(t - taps + 1 + j)`` (no bias, zeros before
    the sequence's start; the last ``taps - 1`` projected rows of a request are its state); the
    position encoding (``position``: a part with ``rotate_store``) turns q and k and the keys and
    values go to the pages; ``score = cap * tanh(q . k * scale / cap)`` over the keys at positions
    <= the query's (or the last ``window``), softmax and the weighted sum in 32-bit; query head h
    reads key/value head ``h // (heads / kv_heads)``; then ``W_o`` with its bias.  ``compute`` returns
    the output itself in 32-bit; ``forward`` adds it onto the stream."""

    graph_safe = True

    def __init__(self, prefix, width: int, n_heads: int, n_kv_heads: int, key_size: int, value_size: int,
                 score_scale: float, taps: int, position, softcap: float | None = None, window: int | None = None,
                 names: dict | None = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.dim, self.vdim, self.taps = int(key_size), int(value_size), int(taps)
        self.score_scale = float(score_scale)
        self.softcap = float(softcap) if softcap else 0.0
        self.window = int(window) if window else None
        if min(self.n_heads, self.n_kv_heads, self.dim, self.vdim) <= 0 or self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"{prefix}: {self.n_heads} heads are not a positive multiple of {self.n_kv_heads} key/value heads")
        if self.taps < 1:
            raise ValueError(f"{prefix}: a convolution has at least one tap")
        self.position = build_part(position)
        if not hasattr(self.position, "rotate_store"):
            raise ValueError(f"{prefix}: the position encoding '{position.kind}' has no rotate_store(ctx, cache, qkv, ...)")
        self.names = dict(q="q", k="k", v="v", o="o", bias=".b", taps=".conv")
        self.names.update(names or {})
        self.q_width, self.k_width, self.v_width = self.n_heads * self.dim, self.n_kv_heads * self.dim, self.n_kv_heads * self.vdim
        self.qkv_width = self.q_width + self.k_width + self.v_width

    def weight_specs(self):
        n = self.names
        specs = list(self.position.weight_specs())
        for name, rows in ((n["q"], self.q_width), (n["k"], self.k_width), (n["v"], self.v_width)):
            specs += [WeightSpec(self.full_name(name), (rows, self.width)),
                      WeightSpec(self.full_name(name + n["bias"]), (rows,), role="vector", init="bias"),
                      WeightSpec(self.full_name(name + n["taps"]), (rows, self.taps), role="vector", init="matrix")]
        specs += [WeightSpec(self.full_name(n["o"]), (self.width, self.n_heads * self.vdim), init="residual_matrix"),
                  WeightSpec(self.full_name(n["o"] + n["bias"]), (self.width,), role="vector", init="bias")]
        return specs

    def cache_need(self):
        need = {"kv": PagedKV(self.n_kv_heads, self.dim, self.window, value_size=self.vdim)}
        if self.taps > 1:
            need["taps"] = FixedState((self.taps - 1, self.qkv_width), "float32")
        return need

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        self.position.bind({w.name: tensors[w.name] for w in self.position.weight_specs() if w.name in tensors}, runtime)
        three = (n["q"], n["k"], n["v"])
        self.stacked = torch.cat([self.w(name) for name in three]).contiguous()
        self.stacked_bias = torch.cat([self.w(name + n["bias"]) for name in three]).contiguous()
        self.stacked_taps = torch.cat([self.w(name + n["taps"]) for name in three]).contiguous()
        self._no_state = torch.zeros((1, 0, self.qkv_width), dtype=torch.float32, device=self.stacked.device)

    def compute(self, ctx, x, cache):
        k, n = ctx.kernels, x.shape[0]
        pages = cache.of("kv")
        projected = ctx.buffer("qkv", (n, self.qkv_width), ctx.act_dtype)
        k.linear(ctx, projected, x, self.stacked, self.stacked_bias)
        if self.taps > 1:
            held = cache.of("taps")
            qkv = ctx.buffer("qkv_filtered", (n, self.qkv_width), ctx.act_dtype)
            k.causal_taps(ctx, qkv, projected, self.stacked_taps, held.state, held.writes, identity=False)
        else:
            qkv = ctx.buffer("qkv_filtered", (n, self.qkv_width), ctx.act_dtype)
            k.causal_taps(ctx, qkv, projected, self.stacked_taps, self._no_state, False, identity=False)
        self.position.rotate_store(ctx, pages, qkv, self.q_width, self.q_width + self.k_width, self.n_heads, self.n_kv_heads,
                                   self.dim, self.vdim)
        mixed = ctx.buffer("attn_out", (n, self.n_heads * self.vdim), ctx.act_dtype)
        k.capped_attention(ctx, mixed, qkv[:, :self.q_width], pages, self.n_heads, self.n_kv_heads, self.dim, self.vdim,
                           self.score_scale, self.softcap, self.window or 0)
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(self.names["o"]), self.w(self.names["o"] + self.names["bias"]))
        return out

    def forward(self, ctx, x, hidden, cache):
        ctx.kernels.scaled_add(hidden, self.compute(ctx, x, cache), 1.0)


class GatedAttention(Mixer):
    """Causal attention without positions in its scores: ``q = W_q x + b_q`` and likewise k, v (one product
    over the stacked matrices; ``bias=False``: no biases); with ``head_norm_eps`` every query and key head is
    divided by its root mean square, ``x / sqrt(mean(x^2) + eps)``, without a gain; ``score = q . k * scale``
    over the keys the mask shows: positions <= the query's, of those the last ``window`` if given, and of
    those the ones in the query's own block of ``chunk`` positions if given (blocks are counted from
    position 0 of the sequence); softmax and the weighted sum in 32-bit; query head h reads key/value
    head ``h // (heads / kv_heads)``.  With ``gate`` head h's result is multiplied by
    ``sigmoid(w_g[h] . x)`` (one number per token and head, read off the same input); then ``W_o``
    (``out_bias``: with its bias).  The normed keys and the values are what the pages hold."""

    graph_safe = True

    def __init__(self, prefix, width: int, n_heads: int, n_kv_heads: int, key_size: int, value_size: int,
                 score_scale: float, head_norm_eps: float | None = None, window: int | None = None, chunk: int | None = None,
                 gate: bool = False, bias: bool = True, out_bias: bool = False, names: dict | None = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.dim, self.vdim, self.score_scale = int(key_size), int(value_size), float(score_scale)
        if min(self.n_heads, self.n_kv_heads, self.dim, self.vdim) <= 0 or self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"{prefix}: {self.n_heads} heads are not a positive multiple of {self.n_kv_heads} key/value heads")
        self.head_norm_eps = float(head_norm_eps) if head_norm_eps is not None else None
        self.window, self.chunk = (int(window) if window else None), (int(chunk) if chunk else None)
        self.gate, self.bias, self.out_bias = bool(gate), bool(bias), bool(out_bias)
        self.names = dict(q="q", k="k", v="v", o="o", g="g", bias=".b")
        self.names.update(names or {})
        self.q_width, self.k_width, self.v_width = self.n_heads * self.dim, self.n_kv_heads * self.dim, self.n_kv_heads * self.vdim
        self.qkv_width = self.q_width + self.k_width + self.v_width

    def weight_specs(self):
        n = self.names
        specs = []
        for name, rows in ((n["q"], self.q_width), (n["k"], self.k_width), (n["v"], self.v_width)):
            specs.append(WeightSpec(self.full_name(name), (rows, self.width)))
            if self.bias:
                specs.append(WeightSpec(self.full_name(name + n["bias"]), (rows,), role="vector", init="bias"))
        if self.gate:
            specs.append(WeightSpec(self.full_name(n["g"]), (self.n_heads, self.width)))
        specs.append(WeightSpec(self.full_name(n["o"]), (self.width, self.n_heads * self.vdim), init="residual_matrix"))
        if self.out_bias:
            specs.append(WeightSpec(self.full_name(n["o"] + n["bias"]), (self.width,), role="vector", init="bias"))
        return specs

    def cache_need(self):
        return PagedKV(self.n_kv_heads, self.dim, self.window, value_size=self.vdim, block=self.chunk)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        three = (n["q"], n["k"], n["v"])
        self.stacked = torch.cat([self.w(name) for name in three]).contiguous()
        self.stacked_bias = torch.cat([self.w(name + n["bias"]) for name in three]).contiguous() if self.bias else None
        if self.gate:
            # rows of zeros up to the least a tensor-core tile takes; the gate leaves its product in 32-bit
            gate = self.w(n["g"])
            self.gate_matrix = gate.contiguous()
            if gate.shape[0] < 16:
                self.gate_matrix = torch.zeros((16, gate.shape[1]), dtype=gate.dtype, device=gate.device)
                self.gate_matrix[:gate.shape[0]] = gate

    def compute(self, ctx, x, cache):
        k, n = ctx.kernels, x.shape[0]
        qkv = ctx.buffer("qkv", (n, self.qkv_width), ctx.act_dtype)
        k.linear(ctx, qkv, x, self.stacked, self.stacked_bias)
        gate = None
        if self.gate:
            gate = ctx.buffer("attention_gate", (n, self.gate_matrix.shape[0]), torch.float32)
            k.linear(ctx, gate, x, self.gate_matrix)
        k.head_norm_store(ctx, cache, qkv, self.q_width, self.q_width + self.k_width, self.n_heads, self.n_kv_heads, self.dim,
                          self.vdim, self.head_norm_eps)
        mixed = ctx.buffer("attn_out", (n, self.n_heads * self.vdim), ctx.act_dtype)
        k.capped_attention(ctx, mixed, qkv[:, :self.q_width], cache, self.n_heads, self.n_kv_heads, self.dim, self.vdim,
                           self.score_scale, 0.0, self.window or 0, chunk=self.chunk or 0, gate=gate)
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(self.names["o"]),
                 self.w(self.names["o"] + self.names["bias"]) if self.out_bias else None)
        return out

    def forward(self, ctx, x, hidden, cache):
        ctx.kernels.scaled_add(hidden, self.compute(ctx, x, cache), 1.0)


class NormedAttention(Mixer):
    """Causal attention whose queries and keys are normed before their rotary positions, with an optional sink.

    ``q = W_q x``, ``k = W_k x`` and, with ``values="projected"``, ``v = W_v x`` (one product over the stacked
    matrices, left in 32-bit; no biases); with ``values="keys"`` there is no W_v and the values are the keys as
    projected, before norm and rotation.  With ``taps`` > 1 every channel of q, k and v then passes a short causal
    convolution, ``y_t = sum_j w[:, j] u_(t - taps + 1 + j)`` (no bias; the last ``taps - 1`` projected rows of a
    request are its state).  ``norm="whole"``: q (and k) are divided by the root mean square of the whole
    projection, all heads at once, and multiplied by a gain of that size; ``norm="head"``: every head by its
    own, times one gain of the head's size that all heads share; eps inside the root.  Then the position
    encoding (``position``: a part with ``norm_rotate_store``) turns q and k, and the keys and values go to the
    pages.  ``score = q . k * scale``, with ``softcap`` ``cap * tanh(score / cap)``, over the keys at positions <= the
    query's (of those the last ``window`` if given); with ``sink`` the softmax's denominator also holds
    ``exp(sink[h])``, a learned number per head that has no key and no value; softmax and the weighted sum in
    32-bit; query head h reads key/value head ``h // (heads / kv_heads)``; then ``W_o``.  ``own_kv=False``: the part
    has no keys and values (no projections, taps or norm of them): it attends, with its own queries, over the
    pages of the run entry named by ``RunEntry.cache_of``."""

    graph_safe = True

    def __init__(self, prefix, width: int, n_heads: int, n_kv_heads: int, key_size: int, value_size: int, score_scale: float,
                 eps: float, position, norm: str | None = "whole", values: str = "projected", taps: int | None = None,
                 softcap: float | None = None, window: int | None = None, sink: bool = False, own_kv: bool = True,
                 names: dict | None = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.dim, self.vdim, self.taps = int(key_size), int(value_size), int(taps) if taps is not None else 0
        self.score_scale, self.eps = float(score_scale), float(eps)
        self.softcap = float(softcap) if softcap else 0.0
        self.window = int(window) if window else None
        self.sink, self.own_kv = bool(sink), bool(own_kv)
        if min(self.n_heads, self.n_kv_heads, self.dim, self.vdim) <= 0 or self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"{prefix}: {self.n_heads} heads are not a positive multiple of {self.n_kv_heads} key/value heads")
        if norm not in (None, "whole", "head"):
            raise ValueError(f"{prefix}: unknown query and key norm '{norm}' (known: head, whole)")
        if values not in ("projected", "keys"):
            raise ValueError(f"{prefix}: the values are 'projected' or the 'keys', got '{values}'")
        if values == "keys" and self.vdim != self.dim:
            raise ValueError(f"{prefix}: values that are the keys have the keys' size {self.dim}, not {self.vdim}")
        if self.taps < 0:
            raise ValueError(f"{prefix}: a convolution has at least one tap")
        self.norm, self.values = norm, values
        self.position = build_part(position)
        if not hasattr(self.position, "norm_rotate_store"):
            raise ValueError(f"{prefix}: the position encoding '{position.kind}' has no norm_rotate_store(ctx, cache, qkv, ...)")
        self.names = dict(q="q", k="k", v="v", o="o", norm=".norm", taps=".conv", sink="sink")
        self.names.update(names or {})
        self.q_width, self.k_width, self.v_width = self.n_heads * self.dim, self.n_kv_heads * self.dim, self.n_kv_heads * self.vdim
        self.projections = [("q", self.q_width)]
        if self.own_kv:
            self.projections.append(("k", self.k_width))
            if values == "projected":
                self.projections.append(("v", self.v_width))
        self.proj_width = sum(rows for _, rows in self.projections)

    def weight_specs(self):
        n = self.names
        specs = list(self.position.weight_specs())
        for key, rows in self.projections:
            specs.append(WeightSpec(self.full_name(n[key]), (rows, self.width)))
            if self.taps >= 1:
                specs.append(WeightSpec(self.full_name(n[key] + n["taps"]), (rows, self.taps), role="vector", init="matrix"))
            if self.norm is not None and key != "v":
                specs.append(WeightSpec(self.full_name(n[key] + n["norm"]), (rows if self.norm == "whole" else self.dim,),
                                        role="vector", init="gain"))
        if self.sink:
            specs.append(WeightSpec(self.full_name(n["sink"]), (self.n_heads,), role="vector", init="shift"))
        specs.append(WeightSpec(self.full_name(n["o"]), (self.width, self.n_heads * self.vdim), init="residual_matrix"))
        return specs

    def cache_need(self):
        # (an entry that reads another's pages gets them under the same name, "kv")
        need = {"kv": PagedKV(self.n_kv_heads, self.dim, self.window, value_size=self.vdim)}
        if self.taps > 1:
            need["taps"] = FixedState((self.taps - 1, self.proj_width), "float32")
        return need

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        self.position.bind({w.name: tensors[w.name] for w in self.position.weight_specs() if w.name in tensors}, runtime)
        keys = [key for key, _ in self.projections]
        self.stacked = torch.cat([self.w(n[key]) for key in keys]).contiguous()
        self.stacked_taps = torch.cat([self.w(n[key] + n["taps"]) for key in keys]).contiguous() if self.taps >= 1 else None
        self._no_state = torch.zeros((1, 0, self.proj_width), dtype=torch.float32, device=self.stacked.device)
        self.q_gain = self.w(n["q"] + n["norm"]) if self.norm is not None else None
        self.k_gain = self.w(n["k"] + n["norm"]) if self.norm is not None and self.own_kv else None

    def compute(self, ctx, x, cache):
        k, n = ctx.kernels, x.shape[0]
        pages = cache.of("kv")
        if self.own_kv != bool(pages.writes):
            raise RuntimeError(f"{self.prefix}: a part {'with' if self.own_kv else 'without'} keys and values of its own got pages "
                               f"it may {'not ' if self.own_kv else ''}store into (RunEntry.cache_of)")
        # projections, taps, norm and rotation in 32-bit: the queries and the cache are rounded once
        projected = ctx.buffer("qkv_32", (n, self.proj_width), torch.float32)
        k.linear(ctx, projected, x, self.stacked)
        if self.taps >= 1:
            held = cache.of("taps") if self.taps > 1 else None
            filtered = ctx.buffer("qkv_32_filtered", (n, self.proj_width), torch.float32)
            k.causal_taps(ctx, filtered, projected, self.stacked_taps, held.state if held is not None else self._no_state,
                          held.writes if held is not None else False, identity=False)
            projected = filtered
        q = ctx.buffer("q", (n, self.q_width), ctx.act_dtype)
        k_off = self.q_width
        v_off = k_off + self.k_width if self.values == "projected" else k_off
        self.position.norm_rotate_store(ctx, pages, projected, q, k_off, v_off, self.n_heads, self.n_kv_heads, self.dim, self.vdim,
                                        self.q_gain, self.k_gain, self.norm, self.eps)
        mixed = ctx.buffer("attn_out", (n, self.n_heads * self.vdim), ctx.act_dtype)
        k.capped_attention(ctx, mixed, q, pages, self.n_heads, self.n_kv_heads, self.dim, self.vdim, self.score_scale,
                           self.softcap, self.window or 0, sink=self.w(self.names["sink"]) if self.sink else None)
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(self.names["o"]))
        return out

    def forward(self, ctx, x, hidden, cache):
        ctx.kernels.scaled_add(hidden, self.compute(ctx, x, cache), 1.0)


register_part("causal_self_attention", CausalSelfAttention)
register_part("normed_attention", NormedAttention)
register_part("filtered_attention", FilteredAttention)
register_part("gated_attention", GatedAttention)

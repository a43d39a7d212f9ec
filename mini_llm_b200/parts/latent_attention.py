"""Causal attention over a shared low-rank latent.

Per token one projection gives ``rank + rot`` numbers: the first ``rank``, normed by their root
mean square and multiplied by a gain, are the latent ``c``; the last ``rot``, with rotary
positions, are a key part ``r`` that all heads share.  Head ``h`` has the key
``[U_k[h] c | r]`` and the value ``U_v[h] c``; its query is ``[q_h | rotated q'_h]`` with
``dim`` and ``rot`` entries.  Only ``[c | r]`` is cached, one row per token for all heads.

The products with U_k and U_v are moved to the query's side (both are linear in ``c``):
``q_h . (U_k[h] c) = (U_k[h]^T q_h) . c``, and ``sum_j p_j U_v[h] c_j = U_v[h] (sum_j p_j c_j)``.
So the step computes, per token and head, the effective query ``[U_k[h]^T q_h | rotated q'_h]``
in 32-bit, attends over the cached rows (score = effective query . row * scale, value = the row's
first ``rank`` entries; softmax in 32-bit), and expands the result with U_v[h].  A prompt portion
and a single decoded token take the same path, and no key or value per head is ever stored.

Rotary positions: among the first ``rotary_dims`` entries of the rotated part, pair i turns by
``position * base^(-2i/rotary_dims)``; ``rotary_layout`` says which entries form pair i: 2i and 2i+1
("interleaved") or i and i + rotary_dims/2 ("half").

Options: ``window``: a query sees only the last ``window`` positions (itself included); the cache then
keeps ``keep`` >= ``window`` positions (``keep``: the widest window of all entries that read these
rows).  ``query_rank``: the queries go through a latent of their own, ``q = W_uq rms(W_dq x) * g_q``.
``own_rows=False``: the part has no down projection and stores nothing; it attends over the rows that
another run entry stores (``RunEntry.cache_of``), with its own expansions, queries and mask.
"""

from __future__ import annotations

import torch

from .base import Mixer, register_part
from .spec import PagedKV, WeightSpec


class LatentAttention(Mixer):
    graph_safe = True
    wants_attention_tiles = True      # its prompt kernel reads the step's work list of (up to 128 tokens, entry) tiles

    def __init__(self, prefix, width: int, n_heads: int, head_size: int, rotated_size: int, value_size: int,
                 latent_size: int, score_scale: float, rotary_base: float, rotary_dims: int, eps: float,
                 q_name: str = "q", down_name: str = "dkv", latent_norm_name: str = "dkv.norm",
                 key_up_name: str = "uk", value_up_name: str = "uv", out_name: str = "o", window: int | None = None,
                 keep: int | None = None, rotary_layout: str = "interleaved", query_rank: int | None = None,
                 query_down_name: str = "dq", query_norm_name: str = "dq.norm", query_up_name: str = "uq",
                 own_rows: bool = True):
        super().__init__(prefix)
        self.width, self.n_heads = int(width), int(n_heads)
        self.dim, self.rot, self.vdim, self.rank = int(head_size), int(rotated_size), int(value_size), int(latent_size)
        self.score_scale, self.rotary_base, self.rotary_dims = float(score_scale), float(rotary_base), int(rotary_dims)
        self.eps = float(eps)
        if self.rotary_dims % 2 != 0 or not 0 <= self.rotary_dims <= self.rot:
            raise ValueError(f"{prefix}: {self.rotary_dims} rotated dimensions do not fit a rotated part of {self.rot} "
                             f"(an even number, at most the part)")
        if min(self.n_heads, self.dim, self.vdim, self.rank) <= 0:
            raise ValueError(f"{prefix}: heads, head size, value size and latent size must be positive")
        self.names = dict(q=q_name, down=down_name, norm=latent_norm_name, uk=key_up_name, uv=value_up_name, o=out_name,
                          dq=query_down_name, dq_norm=query_norm_name, uq=query_up_name)
        self.row = self.rank + self.rot
        self.window = int(window) if window else None
        self.keep = max(int(keep), self.window) if keep and self.window else self.window
        if rotary_layout not in ("interleaved", "half"):
            raise ValueError(f"{prefix}: unknown layout of the rotated pairs '{rotary_layout}' (known: half, interleaved)")
        self.rotary_layout = rotary_layout
        self.query_rank = int(query_rank) if query_rank else None
        self.own_rows = bool(own_rows)

    def weight_specs(self):
        n, h = self.names, self.n_heads
        if self.query_rank:
            specs = [WeightSpec(self.full_name(n["dq"]), (self.query_rank, self.width)),
                     WeightSpec(self.full_name(n["dq_norm"]), (self.query_rank,), role="vector", init="gain"),
                     WeightSpec(self.full_name(n["uq"]), (h * (self.dim + self.rot), self.query_rank))]
        else:
            specs = [WeightSpec(self.full_name(n["q"]), (h * (self.dim + self.rot), self.width))]
        if self.own_rows:
            specs += [WeightSpec(self.full_name(n["down"]), (self.row, self.width)),
                      WeightSpec(self.full_name(n["norm"]), (self.rank,), role="vector", init="gain")]
        return specs + [
            WeightSpec(self.full_name(n["uk"]), (h * self.dim, self.rank)),
            WeightSpec(self.full_name(n["uv"]), (h * self.vdim, self.rank)),
            WeightSpec(self.full_name(n["o"]), (self.width, h * self.vdim), init="residual_matrix"),
        ]

    def cache_need(self):
        return PagedKV(1, self.row, self.keep, has_values=False)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        h = self.n_heads
        uk = self.w(self.names["uk"])
        # per head, [rank, dim]: the key expansion as the product's weight on the query's side
        self.key_up_t = uk.view(h, self.dim, self.rank).transpose(1, 2).contiguous()
        self.value_up = self.w(self.names["uv"]).view(h, self.vdim, self.rank)
        half = self.rotary_dims // 2
        exponent = -2.0 * torch.arange(half, dtype=torch.float64) / max(self.rotary_dims, 1)
        self.inv_freq = (torch.tensor(self.rotary_base, dtype=torch.float64) ** exponent).to(uk.device)
        if half == 0:
            self.inv_freq = torch.zeros(1, dtype=torch.float64, device=uk.device)
        self._no_gain = torch.ones(self.rank, dtype=torch.float32, device=uk.device)

    def compute(self, ctx, x, cache):
        k, n, h, names = ctx.kernels, x.shape[0], self.n_heads, self.names
        if self.own_rows != bool(cache.writes):
            raise RuntimeError(f"{self.prefix}: a part {'with' if self.own_rows else 'without'} a down projection got a cache "
                               f"it may {'not ' if self.own_rows else ''}store into (RunEntry.cache_of)")
        q = ctx.buffer("latent_q", (n, h * (self.dim + self.rot)), ctx.act_dtype)
        if self.query_rank:
            # the query's own latent: its norm reads the product in 32-bit
            thin = ctx.buffer("latent_q_down", (n, self.query_rank), torch.float32)
            k.linear(ctx, thin, x, self.w(names["dq"]))
            normed = ctx.buffer("latent_q_normed", (n, self.query_rank), ctx.act_dtype)
            k.grouped_rms_norm(normed, thin, self.w(names["dq_norm"]), 1, self.eps)
            k.linear(ctx, q, normed, self.w(names["uq"]))
        else:
            k.linear(ctx, q, x, self.w(names["q"]))
        down = None
        if self.own_rows:
            down = ctx.buffer("latent_down", (n, self.row), torch.float32)
            k.linear(ctx, down, x, self.w(names["down"]))
        q_eff = ctx.buffer("latent_q_eff", (n, h * self.row), torch.float32)
        k.latent_prepare(ctx, cache, q_eff, down, q, self.w(names["norm"]) if self.own_rows else self._no_gain, self.inv_freq,
                         self.rank, self.rot, self.rotary_dims, h, self.dim, self.eps, layout=self.rotary_layout)
        k.head_linear(ctx, q_eff, q, self.key_up_t, h, self.dim + self.rot, self.row)
        mixed_latent = ctx.buffer("latent_mixed", (n, h * self.rank), k.latent_mixed_dtype(cache, self.rank, self.rot))
        k.latent_attention(ctx, mixed_latent, q_eff, cache, h, self.rank, self.rot, self.score_scale, window=self.window or 0)
        mixed = ctx.buffer("attn_out", (n, h * self.vdim), ctx.act_dtype)
        k.head_linear(ctx, mixed, mixed_latent, self.value_up, h, self.rank, self.vdim)
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(self.names["o"]))
        return out

    def forward(self, ctx, x, hidden, cache):
        hidden += self.compute(ctx, x, cache)


register_part("latent_attention", LatentAttention)

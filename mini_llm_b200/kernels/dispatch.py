"""Which kernel runs an operation.

``Kernels`` is what parts call.  With ``plain_only`` (always the case for the
32-bit path) every operation runs its plain kernel.  Otherwise a fast kernel is
asked first whether it takes the sizes at hand; if it does not, the plain
kernel runs: never a wrong result, never a CPU path.

A norm whose only consumer is a matrix product may be handed over unevaluated
(``DeferredNorm``): the product kernel for few rows normalises on the way in;
every other kernel has it evaluated first.
"""

from __future__ import annotations

import torch

from . import ops

SKINNY_MAX_ROWS = 8           # up to here a product streams the weights once through the SIMT kernel (measured:
                              # from 9 rows on the tensor-core kernel with swapped operands is faster)
SPLIT_ATTENTION_MAX_ROWS = 64 # up to here attention runs one CTA per (token, head, chunk of keys)


class DeferredNorm:
    """A norm that has not run yet: ``rows`` (or all rows) of the fp32 ``x``.

    ``kind`` names the arithmetic ("layer_norm": gain ``gamma``, shift ``beta``, ``eps``).  A
    product kernel that can norm its input on the way in takes a deferred norm only of a
    kind it knows (``Kernels.FUSED_NORM_KINDS``); any other kind is evaluated first by
    ``evaluate(ctx, out)``, the norm's own kernel.  A new norm therefore works everywhere
    from its first day and gets fused once a product kernel learns its kind."""

    def __init__(self, kind, x, rows, tag, evaluate, **params):
        self.kind, self.x, self.rows, self.tag, self.evaluate = kind, x, rows, tag, evaluate
        self.params = params
        self._value = None

    def __getattr__(self, name):
        try:
            return self.__dict__["params"][name]
        except KeyError:
            raise AttributeError(name) from None

    @property
    def shape(self):
        return (self.x.shape[0] if self.rows is None else self.rows.shape[0], self.x.shape[1])

    def materialize(self, ctx):
        if self._value is None:
            out = ctx.buffer(self.tag, self.shape, ctx.act_dtype)
            self.evaluate(ctx, out)
            self._value = out
        return self._value


class Kernels:
    FUSED_NORM_KINDS = ("layer_norm",)    # what the few-row product kernel can apply on the way in

    def __init__(self, act_dtype: torch.dtype, plain_only: bool = False):
        self.act_dtype = act_dtype
        self.plain_only = bool(plain_only) or act_dtype == torch.float32
        self.launches = 0            # kernels launched (or recorded into a graph) since the start
        self.choices = {}            # (operation, sizes...) -> name of the kernel that ran it last
        self._split_scratch = None
        self._sample_scratch = None
        self.scratch_generation = 0  # grows when scratch moves (captured graphs are then stale)
        self._status = None          # device word the tensor-core kernels report a timed-out wait in
        self._att_scratch = None
        self._att_work = None

    # ---- operations without a fast variant --------------------------------------------------
    def keep_tokens(self, kept, slots, tokens):
        self.launches += 1
        return ops.keep_tokens(kept, slots, tokens)

    def resolve_tokens(self, token_ids, kept):
        self.launches += 1
        return ops.resolve_tokens(token_ids, kept)

    def embed(self, out, token_ids, positions, table, position_table=None):
        self.launches += 1
        return ops.embed(out, token_ids, positions, table, position_table)

    def add_position_rows(self, hidden, positions, table):
        self.launches += 1
        return ops.add_position_rows(hidden, positions, table)

    def layernorm(self, out, x, gamma, beta, eps, rows=None):
        self.launches += 1
        if not self.plain_only and out.dtype == torch.bfloat16 and x.shape[1] % 4 == 0:
            return ops.layernorm_warp(out, x, gamma, beta, eps, rows)
        return ops.layernorm(out, x, gamma, beta, eps, rows)

    # ---- norms in groups, short convolutions, latent attention, matrix memories, layer results ----
    def grouped_rms_norm(self, out, x, gain, groups, eps, rows=None, gate=None, add=False, gate_mode="sigmoid"):
        self.launches += 1
        return ops.grouped_rms_norm(out, x, gain, groups, eps, rows, gate, add, gate_mode)

    def causal_taps(self, ctx, out, h, w, state, writes=True, identity=True, bias=None, silu=False):
        plain_filter = identity and bias is None and not silu
        if isinstance(h, DeferredNorm):
            if (plain_filter and h.kind == "grouped_rms_norm" and h.rows is None and ctx.decode_only
                    and w.shape[1] > 1):
                # single tokens: norm, filter and the state's move in one kernel
                self.launches += 1
                self.chose("causal_taps", "norm_taps_step", out.shape[0], out.shape[1], w.shape[1])
                return ops.norm_taps_step(out, h.x, h.gain, h.groups, h.eps, w, state, ctx.token_item, ctx.item_slot, writes)
            h = h.materialize(ctx)
        self.chose("causal_taps", "causal_taps", out.shape[0], out.shape[1], w.shape[1])
        single = bool(ctx.decode_only)            # every entry brings one token: the filter's kernel moves the state too
        self.launches += 2 if writes and w.shape[1] > 1 and not single else 1
        return ops.causal_taps(out, h, w, state, ctx.positions, ctx.token_item, ctx.item_slot, ctx.item_start,
                               ctx.item_offset, ctx.item_count, writes, identity, bias, silu, single)

    # ---- rotary positions with the cache store, capped attention, linear recurrences, routed experts ----
    def rotary_store(self, ctx, cache, qkv, k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, inv_freq, amplitude):
        self.launches += 1
        return ops.rotary_store(qkv, k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, inv_freq, amplitude, ctx.positions,
                                ctx.token_item, cache.block_table, cache.page_size, cache.k_pages, cache.v_pages, cache.writes)

    def head_norm_store(self, ctx, cache, qkv, k_off, v_off, heads, kv_heads, dim, vdim, eps):
        self.launches += 1
        return ops.head_norm_store(qkv, k_off, v_off, heads, kv_heads, dim, vdim, -1.0 if eps is None else eps, ctx.positions, ctx.token_item,
                                   cache.block_table, cache.page_size, cache.k_pages, cache.v_pages, cache.writes)

    def capped_attention(self, ctx, out, q, cache, n_heads, n_kv_heads, dim, vdim, scale, cap=0.0, window=0, chunk=0,
                         gate=None, sink=None):
        """Attention whose weights stay 32-bit, with a cap on the scores and values of a size of
        their own; the mask is causal, over the last ``window`` positions or within blocks of
        ``chunk`` positions; ``gate`` [T, heads] opens each head's result by its sigmoid; ``sink`` [heads] adds
        exp(sink[h]) to head h's denominator.  Steps with
        prompt portions take the tiles (tokens of a request side by side share the cached rows they
        read); steps of single tokens, and sizes the tiles do not take, one block per (token, head)."""
        self.launches += 1
        n = q.shape[0]
        if (not self.plain_only and ctx.decode_only and n <= SPLIT_ATTENTION_MAX_ROWS and dim == vdim
                and dim in ops.SPLIT_ATTENTION_HEAD_SIZES and q.dtype == torch.bfloat16 and q.stride(0) % 8 == 0):
            # single tokens: each token's keys in chunks over many CTAs, merged by the last to arrive
            # (its exponentials, weights and sums are 32-bit, which this attention asks for)
            pairs = n * n_heads
            span = 64 if pairs < 64 else (128 if pairs < 128 else (256 if pairs < 256 else 512))
            reach = cache.block_table.shape[1] * cache.page_size
            acc, ml, counters = self._scratch(ctx, SPLIT_ATTENTION_MAX_ROWS * n_heads, -(-reach // 64), dim)
            self.chose("capped_attention", "split_attention", n, n_heads, dim, vdim)
            return ops.split_attention(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions, ctx.token_item,
                                       n_heads, n_kv_heads, dim, cache.page_size, scale, window, span, -(-reach // span), acc,
                                       ml, counters, cap=cap, block=chunk, gate=gate, sink=sink)
        tiled = not ctx.decode_only and ops.capped_attention_tiled_takes(dim, vdim, q.dtype)
        self.chose("capped_attention", "capped_attention_tiled" if tiled else "capped_attention_plain", q.shape[0], n_heads, dim, vdim)
        return ops.capped_attention(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions, ctx.token_item,
                                    n_heads, n_kv_heads, dim, vdim, cache.page_size, scale, cap, window, tiled, chunk, gate, sink)

    def linear_recurrence(self, ctx, out, q, k, v, gate_a, gate_b, log_rate, step_bias, state, heads, qk_heads, dim, vdim,
                          delta, unit_norm=False, q_scale=1.0, skip=None, writes=True, channel_decay=False):
        self.launches += 1
        return ops.linear_recurrence(out, q, k, v, gate_a, gate_b, log_rate, step_bias, state, ctx.item_slot, ctx.item_offset,
                                     ctx.item_count, heads, qk_heads, dim, vdim, delta, unit_norm, q_scale, skip, writes,
                                     channel_decay)

    def route(self, x, router, shared_gate, top, choice, in_weight, out_weight, bias=None, softmax_of_chosen=False,
              shared_plain=False):
        self.launches += 1
        return ops.route(x, router, shared_gate, top, choice, in_weight, out_weight, bias, softmax_of_chosen, shared_plain)

    def experts(self, hidden, act, x, choice, in_weight, out_weight, gate_of, up_of, down_of, inner_of, max_inner, pairs,
                ld_down=None, assign=False):
        self.launches += 2
        return ops.experts(hidden, act, x, choice, in_weight, out_weight, gate_of, up_of, down_of, inner_of, max_inner, pairs,
                           ld_down, assign)

    EXPERTS_AT_ONCE_TOKENS = 32    # from here on a step's tokens go through all experts as two products

    def experts_at_once(self, n_tokens, x, up_matrix, down_matrix) -> bool:
        """Whether the routed feed-forward of this step runs as two tensor-core products over all
        experts (unchosen experts weigh 0) instead of pair by pair: many tokens, bfloat16, shapes
        the product kernel takes."""
        return (not self.plain_only and n_tokens >= self.EXPERTS_AT_ONCE_TOKENS and isinstance(x, torch.Tensor)
                and ops.gemm_takes(x, up_matrix) and down_matrix.shape[1] % 8 == 0 and down_matrix.shape[0] >= 16)

    def expert_combine(self, act, gu, choice, in_weight, out_weight, n_experts, inner, top, pairs):
        self.launches += 1
        return ops.expert_combine(act, gu, choice, in_weight, out_weight, n_experts, inner, top, pairs)

    # ---- norms on a sublayer's output, query and key norms with rotary positions, the gated linear recurrence ----
    def norm_rotary_store(self, ctx, cache, qkv, q_out, k_off, v_off, heads, kv_heads, dim, vdim, q_gain, k_gain, norm, eps,
                          rot_dims, layout, inv_freq):
        self.launches += 1
        writes = bool(cache.writes)
        return ops.norm_rotary_store(qkv, k_off, v_off, heads, kv_heads, dim, vdim, q_out, q_gain, k_gain, norm, eps, rot_dims,
                                     layout, inv_freq, ctx.positions, ctx.token_item, cache.block_table if writes else None,
                                     cache.page_size, cache.k_pages if writes else None, cache.v_pages if writes else None, writes)

    def gated_recurrence(self, ctx, out, u, y, gates, bias_r, bias_i, lam, decay_scale, state, block_width, writes=True):
        self.launches += 1
        return ops.gated_recurrence(out, u, y, gates, bias_r, bias_i, lam, decay_scale, state, ctx.item_slot, ctx.item_offset,
                                    ctx.item_count, block_width, writes)

    def add_normed_cast(self, hidden, y=None, gain=None, eps=0.0, act=None):
        self.launches += 1
        return ops.add_normed_cast(hidden, y, gain, eps, act)

    def softcap(self, x, cap):
        self.launches += 1
        return ops.softcap(x, cap)

    def scaled_add(self, x, u, a, v=None, b=0.0, assign=False):
        self.launches += 1
        return ops.scaled_add(x, u, a, v, b, assign)

    def latent_prepare(self, ctx, cache, q_eff, down, q, gain, inv_freq, rank, rot, rot_dims, heads, dim, eps,
                       layout="interleaved"):
        self.launches += 1
        return ops.latent_prepare(cache.k_pages, q_eff, down, q, gain, inv_freq, ctx.positions, ctx.token_item,
                                  cache.block_table, cache.page_size, rank, rot, rot_dims, heads, dim, eps, cache.writes, layout)

    HEAD_LINEAR_GEMM_ROWS = 128   # from here on each head's product goes to the tensor-core kernel by itself

    def head_linear(self, ctx, out, a, w, heads, a_head, o_head):
        m, n, k = a.shape[0], w.shape[1], w.shape[2]
        if (not self.plain_only and m >= self.HEAD_LINEAR_GEMM_ROWS and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and n >= 16 and all(ops.gemm_takes(a[:, h * a_head:h * a_head + k], w[h]) for h in (0, heads - 1))
                and (a_head * 2) % 16 == 0):
            # prompt portions: one launch per head (strided views of a and out; no copy)
            self.launches += heads
            self.chose("head_linear", "gemm_tcgen05", m, n, k, heads)
            status = self.status(ctx.device)
            for h in range(heads):
                ops.gemm_bf16(out[:, h * o_head:h * o_head + n], a[:, h * a_head:h * a_head + k], w[h], None, "store", status)
            return out
        self.launches += 1
        self.chose("head_linear", "head_linear_plain", m, n, k, heads)
        return ops.head_linear(out, a, w, heads, a_head, o_head)

    def latent_mixed_dtype(self, cache, rank, rot):
        """The element type attention over a latent hands its result on in: bfloat16 where the tiled
        kernel runs (the expansion per head then takes the tensor cores), else 32-bit."""
        tiled = not self.plain_only and ops.latent_attention_tiled_takes(cache.k_pages, rank, rot)
        return torch.bfloat16 if tiled and self.act_dtype == torch.bfloat16 else torch.float32

    def latent_attention(self, ctx, out, q_eff, cache, heads, rank, rot, scale, window=0):
        self.launches += 1
        n = q_eff.shape[0]
        if not self.plain_only and ops.latent_attention_tiled_takes(cache.k_pages, rank, rot):
            common = (out, q_eff, cache.k_pages, cache.block_table, ctx.positions, ctx.token_item, heads, rank, rot,
                      cache.page_size, scale)
            if ctx.att_tiles is not None:
                # prompt portions: 32 rows (tokens x heads) a block share every cached row they read
                self.chose("latent_attention", "latent_attention_tiled", n, heads, rank + rot)
                return ops.latent_attention_tiled(*common, tiles=ctx.att_tiles, n_tiles=ctx.n_att_tiles, window=window)
            if ctx.decode_only:
                # single tokens: all heads of a token share the cached rows; while the (token, head
                # block) pairs are fewer than twice the SMs, each token's keys come in parts
                blocks = n * (1 if heads <= 16 else -(-heads // ops.LATENT_TILE_ROWS))
                parts = max(1, min(32, 296 // blocks))
                scratch = self._latent_scratch(ctx.device, n * heads * parts * rank, n * heads * parts * 2) if parts > 1 else None
                self.launches += 1 if parts > 1 else 0
                self.chose("latent_attention", "latent_attention_tiled_parts", n, heads, rank + rot)
                return ops.latent_attention_tiled(*common, parts=parts, scratch=scratch, window=window)
        self.chose("latent_attention", "latent_attention_plain", n, heads, rank + rot)
        plain_out = out if out.dtype == torch.float32 else ctx.buffer("latent_mixed_32", out.shape, torch.float32)
        ops.latent_attention_plain(plain_out, q_eff, cache.k_pages, cache.block_table, ctx.positions, ctx.token_item,
                                   heads, rank, rot, cache.page_size, scale, window)
        if plain_out is not out:
            out.copy_(plain_out)
        return out

    def memory_scan(self, ctx, out, q, k, v, state, heads, dim, vdim, writes=True, **how):
        self.launches += 1
        # prompt portions go through the kernel that takes 32 tokens at a time; a step of single
        # tokens walks each token's one update (the state is read and written once either way)
        chunked = not ctx.decode_only and ops.memory_chunk_takes(dim)
        passes = None
        if chunked and q.shape[0] >= self.MEMORY_PASSES_TOKENS:
            # long portions: the chunks side by side (their sums, a scan over their states, their outputs)
            passes = self._memory_scratch(ctx.device, ops.memory_passes_scratch(q.shape[0], ctx.n_items, heads, dim, vdim))
            self.launches += 3 if "gates" in how else 2
        self.chose("memory_scan", "memory_passes" if passes else ("memory_chunk" if chunked else "memory_scan"),
                   q.shape[0], heads, dim, vdim)
        return ops.memory_scan(out, q, k, v, state, ctx.item_slot, ctx.item_offset, ctx.item_count, heads, dim, vdim,
                               writes=writes, chunked=chunked, passes=passes, **how)

    MEMORY_PASSES_TOKENS = 128     # from here on a step's chunks are worth four launches

    def _memory_scratch(self, device, floats):
        held = getattr(self, "_memory_passes", None)
        if held is None or any(t.numel() < n for t, n in zip(held, floats)):
            self._memory_passes = held = tuple(torch.empty(max(n, 1), dtype=torch.float32, device=device) for n in floats)
            self.scratch_generation += 1
        return held

    # ---- residual streams, gated feed-forwards ----------------------------------------------------
    def streams_fill(self, streams, hidden):
        self.launches += 1
        return ops.streams_fill(streams, hidden)

    def streams_step(self, streams, **what):
        self.launches += 1
        return ops.streams_step(streams, **what)

    def gated_act(self, out, gu, activation="silu"):
        self.launches += 1
        return ops.gated_act(out, gu, activation)

    def depth_mix(self, hidden, kept, weights, index):
        self.launches += 1
        return ops.depth_mix(hidden, kept, weights, index)

    def kv_store(self, k_pages, v_pages, k_src, v_src, positions, token_item, block_table, page_size):
        self.launches += 1
        return ops.kv_store(k_pages, v_pages, k_src, v_src, positions, token_item, block_table, page_size)

    def sample_rows(self, out, logits, temperature=None, top_p=None, seeds=None, counters=None, any_nucleus=True):
        """One token per row.  ``any_nucleus``: whether some row may have a nucleus cut (top_p < 1
        with temperature > 0); rows without are drawn by many blocks each."""
        self.launches += 1
        rows = logits.shape[0]
        held = self._sample_scratch
        if held is None or held[2].numel() < rows:
            capacity = max(rows, 256)
            device = logits.device
            held = self._sample_scratch = (torch.empty(capacity * ops.SAMPLE_SLICES, dtype=torch.float32, device=device),
                                           torch.empty(capacity * ops.SAMPLE_SLICES, dtype=torch.int32, device=device),
                                           torch.zeros(capacity, dtype=torch.int32, device=device))
            self.scratch_generation += 1
        if any_nucleus:
            self.launches += 1
        return ops.sample_rows_sliced(out, logits, temperature, top_p, seeds, counters, held, any_nucleus)

    # ---- matrix products --------------------------------------------------------------------
    def _skinny(self, m, k, n=0) -> bool:
        # a product as wide as a vocabulary streams faster through the tensor-core kernel from
        # three rows on (measured at 50,257 x 768: 23 against 51 us at eight rows)
        rows = 2 if n >= 8192 and k % 8 == 0 else SKINNY_MAX_ROWS
        return not self.plain_only and m <= rows and ops.skinny_linear_takes(m, k)

    def linear(self, ctx, out, a, w, bias=None, epilogue="store"):
        """out = epilogue(a @ w.T + bias).  ``a``: an activation tensor or a ``DeferredNorm``."""
        m, k = a.shape
        self.launches += 1
        # activations the fast kernels do not apply, and products too narrow for a tile, go to the plain kernel
        fast = w.shape[0] >= 16                  # (a product narrower than a tile's smallest box goes to the plain kernel)
        skinny = self._skinny(m, k, w.shape[0])
        deferred = isinstance(a, DeferredNorm)
        if deferred and not (skinny and a.kind in self.FUSED_NORM_KINDS):
            a, deferred = a.materialize(ctx), False      # no kernel here norms this kind on the way in: the norm runs first
        if skinny:
            self.chose("linear", "skinny_linear", m, w.shape[0], k)
            if deferred:
                return ops.skinny_linear(out, a.x, w, bias, epilogue, norm=(a.gamma, a.beta, a.eps, a.rows))
            return ops.skinny_linear(out, a, w, bias, epilogue)
        if fast and not self.plain_only and ops.gemm_takes(a, w):
            self.chose("linear", "gemm_tcgen05", m, w.shape[0], k)
            return ops.gemm_bf16(out, a, w, bias, epilogue, self.status(ctx.device))
        self.chose("linear", "linear_plain", m, w.shape[0], k)
        return ops.linear_plain(out, a, w, bias, epilogue)

    def chose(self, operation: str, kernel: str, *sizes) -> None:
        """Note which kernel ran an operation at which sizes (tests pin the choices)."""
        self.choices[(operation, *sizes)] = kernel

    def status(self, device):
        if self._status is None:
            self._status = torch.zeros(1, dtype=torch.int32, device=device)
        return self._status

    def read_status(self) -> int:
        """The code a kernel left when one of its bounded waits ran out, or 0 (synchronises)."""
        return int(self._status.item()) if self._status is not None else 0

    def reset_after_failure(self) -> None:
        """After a kernel gave up: the status word and every counter that kernels leave at
        zero between launches start over (a tile that was given up left its counter)."""
        if self._status is not None:
            self._status.zero_()
        if self._att_scratch is not None:
            self._att_scratch[1].zero_()
        if self._att_work is not None:
            self._att_work.zero_()
        if self._split_scratch is not None:
            self._split_scratch[2].zero_()
        if self._sample_scratch is not None:
            self._sample_scratch[2].zero_()

    def check_status(self) -> None:
        """Raise if a kernel reported that one of its bounded waits ran out (synchronises)."""
        code = self.read_status()
        if code != 0:
            self.reset_after_failure()
            raise ops.KernelError(f"a tensor-core kernel gave up waiting (code {code}): its result is invalid")

    def qkv_projection(self, ctx, a, w, bias, cache, q_width, kv_width):
        """The fused query/key/value projection.  Keys and values of the step's tokens go into
        the cache pages (if this entry writes its cache); returns the queries [T, q_width]."""
        m, k = a.shape
        skinny = cache.writes and self._skinny(m, k)
        deferred = isinstance(a, DeferredNorm)
        if deferred and not (skinny and a.kind in self.FUSED_NORM_KINDS):
            a, deferred = a.materialize(ctx), False
        if skinny:
            q = ctx.buffer("q", (m, q_width), ctx.act_dtype)
            scatter = (cache.k_pages, cache.v_pages, ctx.positions, ctx.token_item, cache.block_table,
                       cache.page_size, q_width, kv_width)
            self.launches += 1
            self.chose("qkv", "skinny_linear", m, w.shape[0], k)
            if deferred:
                ops.skinny_linear(q, a.x, w, bias, "store", norm=(a.gamma, a.beta, a.eps, a.rows), scatter=scatter)
            else:
                ops.skinny_linear(q, a, w, bias, "store", scatter=scatter)
            return q
        if cache.writes and not self.plain_only and ops.gemm_qkv_takes(a, w, q_width, kv_width):
            q = ctx.buffer("q", (m, q_width), ctx.act_dtype)
            self.launches += 1
            self.chose("qkv", "gemm_tcgen05", m, w.shape[0], k)
            return ops.gemm_bf16_qkv(q, a, w, bias, self.status(ctx.device), cache.k_pages, cache.v_pages,
                                     ctx.positions, ctx.token_item, cache.block_table, cache.page_size, q_width,
                                     kv_width)
        qkv = ctx.buffer("qkv", (m, q_width + 2 * kv_width), ctx.act_dtype)
        self.linear(ctx, qkv, a, w, bias)
        if cache.writes:
            self.kv_store(cache.k_pages, cache.v_pages, qkv[:, q_width:q_width + kv_width],
                          qkv[:, q_width + kv_width:], ctx.positions, ctx.token_item, cache.block_table,
                          cache.page_size)
        return qkv[:, :q_width]

    # ---- attention --------------------------------------------------------------------------
    def attention(self, ctx, out, q, cache, n_heads, n_kv_heads, head_size, scale, window=0):
        self.launches += 1
        n = q.shape[0]
        if (not self.plain_only and n <= SPLIT_ATTENTION_MAX_ROWS and head_size in ops.SPLIT_ATTENTION_HEAD_SIZES):
            # chunk of keys per CTA: small when there are few (token, head) pairs, so that the
            # chunks still fill the GPU
            pairs = n * n_heads
            chunk = 64 if pairs < 64 else (128 if pairs < 128 else (256 if pairs < 256 else 512))
            reach = cache.block_table.shape[1] * cache.page_size
            max_chunks = -(-reach // chunk)
            acc, ml, counters = self._scratch(ctx, SPLIT_ATTENTION_MAX_ROWS * n_heads, -(-reach // 64), head_size)
            # query heads that share a key/value head go through the tensor-core tiles together,
            # reading the keys once; with one query head per key/value head the SIMT kernel is
            # as fast or faster (measured at 9 to 64 requests of 12 heads)
            grouped = n_heads // n_kv_heads >= 2 and ops.group_attention_takes(q, n_heads, n_kv_heads, head_size)
            run = ops.group_attention if grouped else ops.split_attention
            self.chose("attention", "group_attention" if grouped else "split_attention", n, n_heads, head_size)
            return run(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions, ctx.token_item,
                       n_heads, n_kv_heads, head_size, cache.page_size, scale, window, chunk, max_chunks, acc, ml,
                       counters)
        if (not self.plain_only and ctx.att_tiles is not None
                and ops.attention_prefill_takes(q, head_size, cache.page_size)):
            scratch = None
            if ctx.att_parts > 1:
                # Room for the most cells a step can have, whatever this one has: a step replayed
                # from a graph brings its number of split tiles as data and passes by here no more.
                # (Tiles are split in steps of at most eight of them; units while records x heads
                # stay within the SMs, of which no GPU has 256.)
                most = max(ctx.n_split_tiles * n_heads, 8 * n_heads, 256)
                # (cells of a unit's 256 rows, also for the kernel with tiles of 128: one size, no regrowth)
                scratch = self._attention_scratch(ctx.device, most, ops.ATTENTION_MAX_PARTS * ops.ATTENTION_UNIT * (head_size + 4))
            if ctx.att_units:
                self.chose("attention", "attention_two_tiles", n, n_heads, head_size)
                return ops.attention_prefill_two_tiles(out, q, cache.k_pages, cache.v_pages, cache.block_table,
                                                       ctx.att_tiles, ctx.n_att_tiles, n_heads, n_kv_heads, head_size,
                                                       cache.page_size, scale, window, self.status(ctx.device),
                                                       self.attention_work(ctx.device), scratch, ctx.n_split_tiles,
                                                       ops.ATTENTION_MAX_PARTS if ctx.att_parts > 1 else 1)
            self.chose("attention", "attention_tcgen05", n, n_heads, head_size)
            return ops.attention_prefill(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.att_tiles,
                                         ctx.n_att_tiles, n_heads, n_kv_heads, head_size, cache.page_size, scale,
                                         window, self.status(ctx.device), self.attention_work(ctx.device), scratch,
                                         ctx.n_split_tiles,
                                         ops.ATTENTION_MAX_PARTS if ctx.att_parts > 1 else 1)
        self.chose("attention", "attention_plain", n, n_heads, head_size)
        return ops.attention_plain(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions,
                                   ctx.token_item, n_heads, n_kv_heads, head_size, cache.page_size, scale, window)

    def _latent_scratch(self, device, floats, pairs):
        """Partial results of single tokens' latent attention in parts; grows when a step needs more."""
        held = getattr(self, "_latent_parts", None)
        if held is None or held[0].numel() < floats or held[1].numel() < pairs:
            self._latent_parts = held = (torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device),
                                         torch.empty(max(pairs, 1 << 14), dtype=torch.float32, device=device))
            self.scratch_generation += 1
        return held

    def attention_work(self, device):
        """The work counter of the persistent prompt-attention kernel (zero between launches)."""
        if self._att_work is None:
            self._att_work = torch.zeros(2, dtype=torch.int32, device=device)
            self.scratch_generation += 1
        return self._att_work

    def _attention_scratch(self, device, cells, floats_per_cell):
        """Partial states and counters of prompt attention tiles that come in parts; grows
        (doubling) when a step has more split tiles than any before."""
        held = self._att_scratch
        if held is None or held[1].shape[0] < 2 * cells or held[0].shape[0] < cells * floats_per_cell:
            cells = max(cells, held[1].shape[0] if held is not None else 256)
            # (two counters a cell: the kernel with two tiles per CTA counts each tile's parts apart)
            self._att_scratch = held = (torch.empty(cells * floats_per_cell, dtype=torch.float32, device=device),
                                        torch.zeros(2 * cells, dtype=torch.int32, device=device))
            self.scratch_generation += 1
        return held

    def _scratch(self, ctx, pairs, chunks, head_size):
        """Scratch of split_attention, sized for the largest step it takes; allocated once
        (the counters must start at zero and the kernel leaves them so)."""
        need = (pairs * chunks * head_size, pairs * chunks * 2, pairs)
        held = self._split_scratch
        if held is None or any(h.numel() < n for h, n in zip(held, need)):
            device = ctx.device
            self._split_scratch = (torch.empty(need[0], dtype=torch.float32, device=device),
                                   torch.empty(need[1], dtype=torch.float32, device=device),
                                   torch.zeros(need[2], dtype=torch.int32, device=device))
            self.scratch_generation += 1
        return self._split_scratch

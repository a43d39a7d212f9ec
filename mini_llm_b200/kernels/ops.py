"""The operations of a step, as functions over CUDA tensors.

Every function checks what its kernel assumes (device, element types, inner
stride, sizes), then launches on torch's current stream.  There is no CPU
path: a tensor that is not on a CUDA device is an error.  The plain kernels
take every size; a fast kernel either takes a size or is not chosen for it.
"""

from __future__ import annotations

import ctypes

import torch

from .lib import F, I, L, P, Function, KernelError, set_dependent_launch  # noqa: F401  (re-exported)

DT_F32, DT_BF16 = 0, 1
EPILOGUES = {"store": 0, "gelu_tanh": 1, "gelu_erf": 2, "add": 3, "relu_squared": 4, "silu": 5}
GEMM_EPILOGUES = tuple(EPILOGUES)      # what the tensor-core and few-row kernels apply

_DTYPE_CODE = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {dtype}") from None


_pinned_stream = None


def _stream() -> int:
    """The stream launches go to: the current stream, looked up per launch, or the one a
    caller pinned for a run of launches (the lookup costs more than a launch's own checks)."""
    return _pinned_stream if _pinned_stream is not None else torch.cuda.current_stream().cuda_stream


class launches_on_current_stream:
    """Within the block every launch of this module goes to the stream that is current at
    entry (do not switch streams inside)."""

    def __enter__(self):
        global _pinned_stream
        self.before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self.before
        return False


def _check(t: torch.Tensor, name: str, dtype=None, dims=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name}: expected {dims} dimensions, got shape {tuple(t.shape)}")
    if t.dim() > 0 and t.numel() > 0 and t.stride(-1) != 1:
        raise KernelError(f"{name}: the last dimension must be contiguous")


def _ptr(t):
    return None if t is None else t.data_ptr()


_embed = Function("plain", "mllm_plain_embed", [P, P, P, P, P, I, I, I, P])
_add_rows = Function("plain", "mllm_plain_add_rows", [P, P, P, I, I, I, P])
_layernorm = Function("plain", "mllm_plain_layernorm", [P, P, P, P, P, I, I, F, I, P])
_linear = Function("plain", "mllm_plain_linear", [P, P, P, P, I, I, I, L, L, I, I, I, P])
_kv_store = Function("plain", "mllm_plain_kv_store", [P, P, P, P, L, P, P, P, I, I, I, I, I, P])
_attention = Function("plain", "mllm_plain_attention",
                      [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, F, I, I, P])
_sample_rows = Function("sampling", "mllm_sampling_sample_rows", [P, P, L, I, I, P, P, P, P, P])


def embed(out, token_ids, positions, table, position_table=None):
    """out[t] = table[token_ids[t]] (+ position_table[positions[t]]); out is fp32 [T, width]."""
    _check(out, "embed.out", torch.float32, 2)
    _check(token_ids, "embed.token_ids", torch.int32, 1)
    _check(table, "embed.table", None, 2)
    n, width = out.shape
    if not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed: out and table must be contiguous")
    if table.shape[1] != width or token_ids.shape[0] < n:
        raise KernelError("embed: sizes do not agree")
    if position_table is not None:
        _check(position_table, "embed.position_table", table.dtype, 2)
        _check(positions, "embed.positions", torch.int32, 1)
        if position_table.shape[1] != width or not position_table.is_contiguous():
            raise KernelError("embed: position table has another width")
    _embed(out.data_ptr(), token_ids.data_ptr(), _ptr(positions), table.data_ptr(), _ptr(position_table),
           n, width, dtype_code(table.dtype), _stream())
    return out


def add_position_rows(hidden, positions, table):
    """hidden[t] += table[positions[t]]."""
    _check(hidden, "add_position_rows.hidden", torch.float32, 2)
    _check(positions, "add_position_rows.positions", torch.int32, 1)
    _check(table, "add_position_rows.table", None, 2)
    if not hidden.is_contiguous() or not table.is_contiguous() or table.shape[1] != hidden.shape[1]:
        raise KernelError("add_position_rows: sizes do not agree")
    _add_rows(hidden.data_ptr(), positions.data_ptr(), table.data_ptr(), hidden.shape[0], hidden.shape[1],
              dtype_code(table.dtype), _stream())
    return hidden


def layernorm(out, x, gamma, beta, eps, rows=None):
    """out[r] = LN(x[rows[r]] or x[r]); x fp32 [*, width]; out fp32 or bf16 [R, width]."""
    _check(out, "layernorm.out", None, 2)
    _check(x, "layernorm.x", torch.float32, 2)
    _check(gamma, "layernorm.gamma", torch.float32, 1)
    _check(beta, "layernorm.beta", torch.float32, 1)
    width = x.shape[1]
    if not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("layernorm: x and out must be contiguous")
    if out.shape[1] != width or gamma.shape[0] != width or beta.shape[0] != width:
        raise KernelError("layernorm: widths do not agree")
    if rows is not None:
        _check(rows, "layernorm.rows", torch.int32, 1)
        if rows.shape[0] < out.shape[0]:
            raise KernelError("layernorm: fewer row indices than output rows")
    elif x.shape[0] < out.shape[0]:
        raise KernelError("layernorm: fewer input rows than output rows")
    _layernorm(out.data_ptr(), x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), _ptr(rows),
               out.shape[0], width, float(eps), dtype_code(out.dtype), _stream())
    return out


def linear_plain(out, a, w, bias=None, epilogue="store"):
    """out = epilogue(a @ w.T + bias); a [M, K], w [N, K] (K contiguous), out [M, N].

    epilogue "add": out (fp32) += a @ w.T + bias.
    """
    _check(out, "linear.out", None, 2)
    _check(a, "linear.a", None, 2)
    _check(w, "linear.w", a.dtype, 2)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n or not w.is_contiguous():
        raise KernelError(f"linear: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _check(bias, "linear.bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("linear: bias has another length")
    _linear(out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), m, n, k, a.stride(0), out.stride(0),
            dtype_code(a.dtype), dtype_code(out.dtype), EPILOGUES[epilogue], _stream())
    return out


def kv_store(k_pages, v_pages, k_src, v_src, positions, token_item, block_table, page_size):
    """Write this step's keys and values (rows of k_src, v_src: [T, width]) into their pages."""
    _check(k_pages, "kv_store.k_pages")
    _check(v_pages, "kv_store.v_pages", k_pages.dtype)
    _check(k_src, "kv_store.k_src", k_pages.dtype, 2)
    _check(v_src, "kv_store.v_src", k_pages.dtype, 2)
    _check(block_table, "kv_store.block_table", torch.int32, 2)
    _check(positions, "kv_store.positions", torch.int32, 1)
    _check(token_item, "kv_store.token_item", torch.int32, 1)
    n, width = k_src.shape
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("kv_store: pages and block table must be contiguous")
    if k_src.stride(0) != v_src.stride(0) or v_src.shape != k_src.shape:
        raise KernelError("kv_store: keys and values must share shape and row stride")
    if k_pages.numel() % (page_size * width) != 0:
        raise KernelError("kv_store: page pool does not hold whole pages of this width")
    _kv_store(k_pages.data_ptr(), v_pages.data_ptr(), k_src.data_ptr(), v_src.data_ptr(), k_src.stride(0),
              positions.data_ptr(), token_item.data_ptr(), block_table.data_ptr(), block_table.shape[1],
              page_size, width, n, dtype_code(k_pages.dtype), _stream())


def attention_plain(out, q, k_pages, v_pages, block_table, positions, token_item, n_heads, n_kv_heads,
                    head_size, page_size, scale, window=0):
    """Causal attention of every token of the step over its request's pages."""
    _check(out, "attention.out", q.dtype, 2)
    _check(q, "attention.q", None, 2)
    _check(k_pages, "attention.k_pages", q.dtype)
    _check(v_pages, "attention.v_pages", q.dtype)
    _check(block_table, "attention.block_table", torch.int32, 2)
    _check(positions, "attention.positions", torch.int32, 1)
    _check(token_item, "attention.token_item", torch.int32, 1)
    n = q.shape[0]
    if q.shape[1] != n_heads * head_size or out.shape[1] != n_heads * head_size or out.shape[0] != n:
        raise KernelError("attention: q / out do not have heads * head_size columns")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("attention: pages and block table must be contiguous")
    _attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
               block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), token_item.data_ptr(), n,
               n_heads, n_kv_heads, head_size, page_size, float(scale), int(window or 0),
               dtype_code(q.dtype), _stream())
    return out


def sample_rows(out, logits, temperature=None, top_p=None, seeds=None, counters=None):
    """One token per row of fp32 logits [R, V] into out (int32 [R]).

    temperature / top_p: fp32 [R] or None (greedy / no cut); seeds: int64 [R]
    (bit pattern of a u64); counters: int32 [R].
    """
    _check(out, "sample_rows.out", torch.int32, 1)
    _check(logits, "sample_rows.logits", torch.float32, 2)
    r, vocab = logits.shape
    if out.shape[0] < r:
        raise KernelError("sample_rows: output too short")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                        ("seeds", seeds, torch.int64), ("counters", counters, torch.int32)):
        if t is not None:
            _check(t, f"sample_rows.{name}", dt, 1)
            if t.shape[0] < r:
                raise KernelError(f"sample_rows: {name} too short")
    _sample_rows(out.data_ptr(), logits.data_ptr(), logits.stride(0), r, vocab, _ptr(temperature), _ptr(top_p),
                 _ptr(seeds), _ptr(counters), _stream())
    return out


# ---- kernels for steps of few tokens (bfloat16) --------------------------------------------------

class _SkinnyParams(ctypes.Structure):
    _fields_ = [("out", P), ("x", P), ("w", P), ("bias", P), ("gamma", P), ("beta", P), ("rows", P),
                ("eps", F), ("M", I), ("N", I), ("K", I), ("ldx", L), ("ldo", L), ("epilogue", I), ("out_f32", I),
                ("k_pages", P), ("v_pages", P), ("positions", P), ("token_item", P), ("block_table", P),
                ("max_blocks", I), ("page_size", I), ("q_width", I), ("kv_width", I)]


_skinny = Function("decode", "mllm_decode_skinny_linear", [ctypes.POINTER(_SkinnyParams), P])
_split_attention = Function("decode", "mllm_decode_split_attention_sink",
                            [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, F, F, I, I, P, L, P, I, I, P, P, P, P])

SKINNY_MAX_SMEM = 200 * 1024
SPLIT_ATTENTION_HEAD_SIZES = (16, 32, 64, 128, 256)


def skinny_linear_takes(m, k) -> bool:
    """Whether skinny_linear takes a product with ``m`` rows and inner size ``k``."""
    rows = 1 if m <= 1 else 2 if m <= 2 else 4 if m <= 4 else 8 if m <= 8 else 16
    return k % 8 == 0 and rows * k * 2 <= SKINNY_MAX_SMEM


def skinny_linear(out, x, w, bias=None, epilogue="store", norm=None, scatter=None):
    """out = epilogue(norm?(x) @ w.T + bias) for few rows (bf16 weights, fp32 sums).

    norm: (gamma, beta, eps, rows or None): x is then the fp32 residual stream and is
    layer-normed on the way in.  scatter: (k_pages, v_pages, positions, token_item,
    block_table, page_size, q_width, kv_width): columns past q_width are written into the
    cache pages instead of ``out`` (which then has q_width columns).
    """
    _check(w, "skinny_linear.w", torch.bfloat16, 2)
    n, k = w.shape
    params = _SkinnyParams()
    if norm is not None:
        gamma, beta, eps, rows = norm
        _check(x, "skinny_linear.x", torch.float32, 2)
        _check(gamma, "skinny_linear.gamma", torch.float32, 1)
        _check(beta, "skinny_linear.beta", torch.float32, 1)
        if not x.is_contiguous() or x.shape[1] != k or gamma.shape[0] != k or beta.shape[0] != k:
            raise KernelError("skinny_linear: the normed input does not have K contiguous columns")
        if rows is not None:
            _check(rows, "skinny_linear.rows", torch.int32, 1)
        m = rows.shape[0] if rows is not None else x.shape[0]
        params.gamma, params.beta, params.rows, params.eps = gamma.data_ptr(), beta.data_ptr(), _ptr(rows), float(eps)
    else:
        _check(x, "skinny_linear.x", torch.bfloat16, 2)
        if x.shape[1] != k:
            raise KernelError("skinny_linear: x and w disagree on K")
        m = x.shape[0]
    _check(out, "skinny_linear.out", None, 2)
    if not w.is_contiguous() or not skinny_linear_takes(m, k):
        raise KernelError(f"skinny_linear does not take M={m}, K={k}")
    out_cols = n if scatter is None else scatter[6]
    if out.shape[0] != m or out.shape[1] != out_cols:
        raise KernelError(f"skinny_linear: out is {tuple(out.shape)}, expected {(m, out_cols)}")
    if epilogue == "add" and out.dtype != torch.float32:
        raise KernelError("skinny_linear: the residual sum is kept in 32-bit")
    if epilogue != "add" and out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("skinny_linear: out must be bfloat16 or float32")
    if bias is not None:
        _check(bias, "skinny_linear.bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("skinny_linear: bias has another length")
    params.out, params.x, params.w, params.bias = out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias)
    params.M, params.N, params.K = m, n, k
    params.ldx, params.ldo = x.stride(0), out.stride(0)
    params.epilogue = EPILOGUES[epilogue]
    params.out_f32 = int(out.dtype == torch.float32 and epilogue != "add")
    if scatter is not None:
        k_pages, v_pages, positions, token_item, block_table, page_size, q_width, kv_width = scatter
        _check(k_pages, "skinny_linear.k_pages", torch.bfloat16)
        _check(v_pages, "skinny_linear.v_pages", torch.bfloat16)
        _check(block_table, "skinny_linear.block_table", torch.int32, 2)
        if q_width + 2 * kv_width != n or not k_pages.is_contiguous() or not v_pages.is_contiguous():
            raise KernelError("skinny_linear: scatter widths do not add up to N")
        params.k_pages, params.v_pages = k_pages.data_ptr(), v_pages.data_ptr()
        params.positions, params.token_item = positions.data_ptr(), token_item.data_ptr()
        params.block_table, params.max_blocks = block_table.data_ptr(), block_table.shape[1]
        params.page_size, params.q_width, params.kv_width = page_size, q_width, kv_width
    _skinny(ctypes.byref(params), _stream())
    return out


def split_attention(out, q, k_pages, v_pages, block_table, positions, token_item, n_heads, n_kv_heads, head_size,
                    page_size, scale, window, chunk, max_chunks, part_acc, part_ml, counters, cap=0.0, block=0, gate=None, sink=None):
    """Causal attention over the paged cache for few tokens: one CTA per (token, head, chunk
    of ``chunk`` keys); needs fp32 scratch ``part_acc`` [T*H*max_chunks*D], ``part_ml``
    [T*H*max_chunks*2] and zeroed int32 ``counters`` [T*H] (left zero).  ``cap`` > 0: the scores
    are capped, cap * tanh(score / cap).  ``block`` > 0: a query sees only the keys of its own block of
    ``block`` positions (blocks counted from position 0).  ``gate`` fp32 [T, >= heads]: head h's result
    is multiplied by sigmoid(gate[t, h]).  ``sink`` fp32 [heads]: exp(sink[h]) joins head h's denominator.
    Scores, weights and sums are 32-bit."""
    _check(out, "split_attention.out", torch.bfloat16, 2)
    _check(q, "split_attention.q", torch.bfloat16, 2)
    _check(k_pages, "split_attention.k_pages", torch.bfloat16)
    _check(v_pages, "split_attention.v_pages", torch.bfloat16)
    _check(block_table, "split_attention.block_table", torch.int32, 2)
    _check(part_acc, "split_attention.part_acc", torch.float32)
    _check(part_ml, "split_attention.part_ml", torch.float32)
    _check(counters, "split_attention.counters", torch.int32)
    n = q.shape[0]
    cells = n * n_heads * max_chunks
    if head_size not in SPLIT_ATTENTION_HEAD_SIZES:
        raise KernelError(f"split_attention does not take head size {head_size}")
    if q.shape[1] != n_heads * head_size or out.shape != q.shape:
        raise KernelError("split_attention: q / out do not have heads * head_size columns")
    if part_acc.numel() < cells * head_size or part_ml.numel() < cells * 2 or counters.numel() < n * n_heads:
        raise KernelError("split_attention: scratch too small")
    if max_chunks * chunk < page_size * block_table.shape[1]:
        raise KernelError("split_attention: the chunks do not cover the longest block table")
    if gate is not None:
        _check(gate, "split_attention.gate", torch.float32, 2)
        if gate.shape[0] < n or gate.shape[1] < n_heads or gate.stride(1) != 1:
            raise KernelError("split_attention: one gate per token and head")
    _check_sink(sink, n_heads, "split_attention")
    _split_attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                     block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), token_item.data_ptr(), n,
                     n_heads, n_kv_heads, head_size, page_size, float(scale), float(cap or 0.0), int(window or 0), int(block or 0),
                     _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(sink), int(chunk), int(max_chunks), part_acc.data_ptr(),
                     part_ml.data_ptr(), counters.data_ptr(), _stream())
    return out


def _check_sink(sink, n_heads, who):
    if sink is not None:
        _check(sink, f"{who}.sink", torch.float32, 1)
        if sink.shape[0] != n_heads:
            raise KernelError(f"{who}: one sink per head")


_group_attention = Function("decode", "mllm_decode_group_attention",
                            [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, F, I, I, I, P, P, P, P])
GROUP_ATTENTION_HEAD_SIZES = (64, 128)


def group_attention_takes(q, n_heads, n_kv_heads, head_size) -> bool:
    """Whether ``group_attention`` takes the layout: bfloat16, head size 64 or 128, at most
    eight query heads per key/value head, rows of q on 16-byte boundaries."""
    return (q.dtype == torch.bfloat16 and head_size in GROUP_ATTENTION_HEAD_SIZES and n_kv_heads > 0
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 8 and q.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0)


def group_attention(out, q, k_pages, v_pages, block_table, positions, token_item, n_heads, n_kv_heads, head_size,
                    page_size, scale, window, chunk, max_chunks, part_acc, part_ml, counters):
    """``split_attention`` with the products on mma.sync tiles: one CTA per (token, key/value
    head, chunk of keys), the query heads of the group as the rows of the tiles.  Same
    arguments and scratch; ``chunk`` must be a multiple of 16."""
    _check(out, "group_attention.out", torch.bfloat16, 2)
    _check(q, "group_attention.q", torch.bfloat16, 2)
    _check(k_pages, "group_attention.k_pages", torch.bfloat16)
    _check(v_pages, "group_attention.v_pages", torch.bfloat16)
    _check(block_table, "group_attention.block_table", torch.int32, 2)
    _check(part_acc, "group_attention.part_acc", torch.float32)
    _check(part_ml, "group_attention.part_ml", torch.float32)
    _check(counters, "group_attention.counters", torch.int32)
    n = q.shape[0]
    cells = n * n_heads * max_chunks
    if not group_attention_takes(q, n_heads, n_kv_heads, head_size) or chunk % 16 != 0:
        raise KernelError(f"group_attention does not take head size {head_size} with {n_heads}/{n_kv_heads} heads")
    if q.shape[1] != n_heads * head_size or out.shape != q.shape:
        raise KernelError("group_attention: q / out do not have heads * head_size columns")
    if part_acc.numel() < cells * head_size or part_ml.numel() < cells * 2 or counters.numel() < n * n_heads:
        raise KernelError("group_attention: scratch too small")
    if max_chunks * chunk < page_size * block_table.shape[1]:
        raise KernelError("group_attention: the chunks do not cover the longest block table")
    _group_attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                     block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), token_item.data_ptr(), n,
                     n_heads, n_kv_heads, head_size, page_size, float(scale), int(window or 0), int(chunk),
                     int(max_chunks), part_acc.data_ptr(), part_ml.data_ptr(), counters.data_ptr(), _stream())
    return out


# ---- tensor-core matrix product (bfloat16) -------------------------------------------------------

_gemm_bf16 = Function("gemm", "mllm_gemm_bf16", [P, P, P, P, I, I, I, L, L, I, I, P, P])


def gemm_takes(a, w) -> bool:
    """Whether the tensor-core kernel takes ``a @ w.T``: bf16, K a multiple of 8, 16-byte
    aligned bases and row strides (what its TMA copies need)."""
    if not isinstance(a, torch.Tensor) or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    k = a.shape[1]
    return (k % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1 and a.data_ptr() % 16 == 0
            and w.is_contiguous() and w.data_ptr() % 16 == 0)


def gemm_bf16(out, a, w, bias, epilogue, status):
    """out = epilogue(a @ w.T + bias) on the tensor cores (tcgen05, TMEM accumulators, TMA).

    a [M, K] and w [N, K] bf16; out bf16, or fp32 for logits and for the residual epilogue
    "add".  ``status``: a zeroed int32 device word the kernel writes a code to if one of its
    bounded waits runs out."""
    _check(a, "gemm.a", torch.bfloat16, 2)
    _check(w, "gemm.w", torch.bfloat16, 2)
    _check(out, "gemm.out", None, 2)
    _check(status, "gemm.status", torch.int32)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not gemm_takes(a, w):
        raise KernelError("gemm: operands are not laid out for the tensor-core kernel")
    if out.dtype not in (torch.bfloat16, torch.float32) or (epilogue == "add" and out.dtype != torch.float32):
        raise KernelError("gemm: out must be bfloat16, or float32 for logits and the residual sum")
    if out.dtype == torch.float32 and epilogue not in ("add", "store"):
        raise KernelError("gemm: an activation is stored in bfloat16")
    if bias is not None:
        _check(bias, "gemm.bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("gemm: bias has another length")
    _gemm_bf16(out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), m, n, k, a.stride(0), out.stride(0),
               EPILOGUES[epilogue], int(out.dtype == torch.float32), status.data_ptr(), _stream())
    return out


_gemm_bf16_tile = Function("gemm", "mllm_gemm_bf16_tile", [P, P, P, P, I, I, I, L, L, I, I, P, I, P, P])
GEMM_TILE_WIDTHS = (64, 96, 128, 192, 256)        # 1000 + width: tiles of 256 tokens on pairs of CTAs; 2000 + width (to 128): two issuing threads; 7000 / 7100 + CTAs: shared along K


def gemm_bf16_tile(out, a, w, bias, epilogue, status, tile_width, timeline=None):
    """``gemm_bf16`` through the persistent kernel with tiles of 128 x ``tile_width``, whatever
    the number of rows (tests run every width; the engine lets the library choose).  A code
    5000 + t runs the kernel with swapped operands and tiles of t tokens (16 to 256) instead; a
    code 7000 + c (7100 + c) tiles of 256 (128) features shared along K by clusters of c = 2 to 4 CTAs.
    ``timeline``: an int64 device tensor of nine entries that receives time stamps of CTA 0
    (start, set-up done, first operands landed, last product of the first tile issued, first
    accumulator ready, first epilogue done, end), in nanoseconds, then the number of blocks of K
    that CTA's first issuing thread took and how many of them had not arrived at its first look."""
    if timeline is not None:
        _check(timeline, "gemm.timeline", torch.int64, 1)
        if timeline.shape[0] < 9:
            raise KernelError("gemm: the timeline has nine entries")
    _check(a, "gemm.a", torch.bfloat16, 2)
    _check(w, "gemm.w", torch.bfloat16, 2)
    _check(out, "gemm.out", None, 2)
    _check(status, "gemm.status", torch.int32)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n or not gemm_takes(a, w):
        raise KernelError("gemm: operands are not laid out for the tensor-core kernel")
    if out.dtype not in (torch.bfloat16, torch.float32) or (epilogue == "add" and out.dtype != torch.float32):
        raise KernelError("gemm: out must be bfloat16, or float32 for logits and the residual sum")
    if bias is not None:
        _check(bias, "gemm.bias", torch.float32, 1)
    _gemm_bf16_tile(out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), m, n, k, a.stride(0), out.stride(0),
                    EPILOGUES[epilogue], int(out.dtype == torch.float32), status.data_ptr(), int(tile_width),
                    _ptr(timeline), _stream())
    return out


_gemm_bf16_qkv = Function("gemm", "mllm_gemm_bf16_qkv", [P, P, P, P, I, I, I, L, L, P, P, P, P, P, P, I, I, I, I, P])


def gemm_qkv_takes(a, w, q_width, kv_width) -> bool:
    """Whether ``gemm_bf16_qkv`` takes the product (what ``gemm_takes`` asks, and query and
    key/value widths that are multiples of 32)."""
    return gemm_takes(a, w) and q_width % 32 == 0 and kv_width % 32 == 0 and w.shape[0] == q_width + 2 * kv_width


def gemm_bf16_qkv(q_out, a, w, bias, status, k_pages, v_pages, positions, token_item, block_table, page_size,
                  q_width, kv_width):
    """The fused query/key/value product on the tensor cores: queries into ``q_out``
    [M, q_width]; keys and values into the cache pages, each token at the slot its position
    and its request's block table row name (the epilogue of ``gemm_bf16`` with a scatter)."""
    _check(a, "gemm_qkv.a", torch.bfloat16, 2)
    _check(w, "gemm_qkv.w", torch.bfloat16, 2)
    _check(q_out, "gemm_qkv.q_out", torch.bfloat16, 2)
    _check(k_pages, "gemm_qkv.k_pages", torch.bfloat16)
    _check(v_pages, "gemm_qkv.v_pages", torch.bfloat16)
    _check(positions, "gemm_qkv.positions", torch.int32, 1)
    _check(token_item, "gemm_qkv.token_item", torch.int32, 1)
    _check(block_table, "gemm_qkv.block_table", torch.int32, 2)
    _check(status, "gemm_qkv.status", torch.int32)
    m, k = a.shape
    n = w.shape[0]
    if not gemm_qkv_takes(a, w, q_width, kv_width) or w.shape[1] != k:
        raise KernelError("gemm_qkv: operands are not laid out for the tensor-core kernel with a scatter")
    if q_out.shape[0] != m or q_out.shape[1] != q_width or q_out.stride(1) != 1:
        raise KernelError("gemm_qkv: q_out must be [M, q_width]")
    if not (k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.is_contiguous()):
        raise KernelError("gemm_qkv: pages and block table must be contiguous")
    if positions.shape[0] < m or token_item.shape[0] < m:
        raise KernelError("gemm_qkv: fewer positions than rows")
    if bias is not None:
        _check(bias, "gemm_qkv.bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("gemm_qkv: bias has another length")
    _gemm_bf16_qkv(q_out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), m, n, k, a.stride(0), q_out.stride(0),
                   status.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), positions.data_ptr(), token_item.data_ptr(),
                   block_table.data_ptr(), block_table.shape[1], page_size, q_width, kv_width, _stream())
    return q_out


# ---- tensor-core attention for prompt portions (bfloat16) ----------------------------------------

_attention_prefill = Function("attention", "mllm_attention_prefill",
                              [P, L, P, L, L, L, P, P, I, I, P, I, P, I, I, I, I, F, I, P, P, P, I, P, P])

PREFILL_ATTENTION_HEAD_SIZES = (64, 128)
PREFILL_ATTENTION_PAGE_SIZES = (8, 16, 32, 64, 128)
ATTENTION_TILE = 128


def attention_prefill_takes(q, head_size, page_size) -> bool:
    return (q.dtype == torch.bfloat16 and head_size in PREFILL_ATTENTION_HEAD_SIZES
            and page_size in PREFILL_ATTENTION_PAGE_SIZES and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


ATTENTION_TILE_RECORD = 8           # int32 per CTA of attention_prefill
ATTENTION_BLOCKS_PER_PART = 4       # a tile with more key blocks than this is shared among several CTAs
ATTENTION_MAX_PARTS = 8


def attention_tiles(item_offsets, item_counts, item_starts, split=None):
    """The work list of attention_prefill: tiles of up to 128 consecutive tokens of one
    entry, one record per unit of work: (entry, first row, rows, position of the first row,
    part, parts, number of the tile among the split ones, key blocks of the part), sorted by
    falling number of key blocks.  A tile that reaches over more than
    four blocks of 128 keys can be given to several CTAs (parts), so that the longest CTA of a
    step stays short.  That pays only while the step has few tiles (measured: two CTAs on one
    SM run no faster than one after the other), so by default tiles are split when there are
    at most eight of them; ``split=True`` / ``False`` forces it (whole tiles need no scratch).
    Returns (records, number of split tiles, most parts of a tile)."""
    records, n_split, most = [], 0, 1
    if split is None:
        split = sum(-(-count // ATTENTION_TILE) for count in item_counts) <= 8
    for item, (offset, count, start) in enumerate(zip(item_offsets, item_counts, item_starts)):
        for first in range(0, count, ATTENTION_TILE):
            rows = min(ATTENTION_TILE, count - first)
            blocks = (start + first + rows - 1) // ATTENTION_TILE + 1
            parts = min(ATTENTION_MAX_PARTS, -(-blocks // ATTENTION_BLOCKS_PER_PART)) if split else 1
            share = -(-blocks // parts)
            for part in range(parts):
                records.append((item, offset + first, rows, start + first, part, parts, n_split if parts > 1 else 0,
                                min(share, blocks - part * share)))
            if parts > 1:
                n_split += 1
                most = max(most, parts)
    # the kernel's CTAs take records in this order: the longest first
    records.sort(key=lambda record: -record[7])
    return records, n_split, most


def attention_prefill(out, q, k_pages, v_pages, block_table, tiles, n_tiles, n_heads, n_kv_heads, head_size,
                      page_size, scale, window, status, work, scratch=None, n_split=0, max_parts=1):
    """Causal attention over the paged cache on the tensor cores (tcgen05): one CTA per
    (record of the work list, head).  ``tiles``: device int32 [>= n_tiles, 8] from
    ``attention_tiles``.  ``work``: two zeroed int32 (the kernel's work counter; left zero).
    ``scratch``: (fp32 partial states, zeroed int32 counters) when tiles
    come in parts: n_split * heads * max_parts * 128 * (head_size + 4) floats and
    n_split * heads counters."""
    _check(out, "attention_prefill.out", torch.bfloat16, 2)
    _check(q, "attention_prefill.q", torch.bfloat16, 2)
    _check(k_pages, "attention_prefill.k_pages", torch.bfloat16, 4)
    _check(v_pages, "attention_prefill.v_pages", torch.bfloat16, 4)
    _check(block_table, "attention_prefill.block_table", torch.int32, 2)
    _check(tiles, "attention_prefill.tiles", torch.int32)
    _check(status, "attention_prefill.status", torch.int32)
    _check(work, "attention_prefill.work", torch.int32, 1)
    if work.shape[0] < 2:
        raise KernelError("attention_prefill: the work counter has two entries")
    if not attention_prefill_takes(q, head_size, page_size):
        raise KernelError(f"attention_prefill does not take head size {head_size} with pages of {page_size}")
    n_pages = k_pages.shape[0]
    if tuple(k_pages.shape) != (n_pages, page_size, n_kv_heads, head_size) or v_pages.shape != k_pages.shape:
        raise KernelError("attention_prefill: pages must be [n_pages, page_size, kv_heads, head_size]")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("attention_prefill: pages and block table must be contiguous")
    if q.shape[1] != n_heads * head_size or out.shape != q.shape or tiles.numel() < ATTENTION_TILE_RECORD * n_tiles:
        raise KernelError("attention_prefill: q / out / tiles do not fit")
    partial = counters = None
    if max_parts > 1:
        if scratch is None:
            raise KernelError("attention_prefill: tiles in parts need scratch")
        partial, counters = scratch
        _check(partial, "attention_prefill.scratch", torch.float32, 1)
        _check(counters, "attention_prefill.scratch", torch.int32, 1)
        if (partial.shape[0] < n_split * n_heads * max_parts * ATTENTION_TILE * (head_size + 4)
                or counters.shape[0] < n_split * n_heads):
            raise KernelError("attention_prefill: scratch too small")
    _attention_prefill(out.data_ptr(), out.stride(0), q.data_ptr(), q.shape[0], q.shape[1], q.stride(0),
                       k_pages.data_ptr(), v_pages.data_ptr(), n_pages, page_size, block_table.data_ptr(),
                       block_table.shape[1], tiles.data_ptr(), n_tiles, n_heads, n_kv_heads, head_size, float(scale),
                       int(window or 0), status.data_ptr(), _ptr(partial), _ptr(counters), int(max_parts),
                       work.data_ptr(), _stream())
    return out


_attention_prefill_two_tiles = Function("attention", "mllm_attention_prefill_two_tiles",
                                        [P, L, P, L, L, L, P, P, I, I, P, I, P, I, I, I, I, F, I, P, P, P, I, P, P])
ATTENTION_UNIT = 2 * ATTENTION_TILE     # queries per CTA of attention_prefill_two_tiles


def attention_units(item_offsets, item_counts, item_starts, n_heads=1, n_sms=148):
    """The work list of attention_prefill_two_tiles: units of up to 256 consecutive tokens of
    one entry, one record per CTA: (entry, first row, rows, position of the first row, part,
    parts, number of the unit among the split ones, key blocks of the part), sorted by falling
    number of key blocks.  While the step's records times ``n_heads`` leave SMs idle, the unit
    with the most key blocks per part is given one more part (up to eight, and not below two
    blocks a part), so that the step's longest CTA gets shorter.
    Returns (records, number of split units, most parts of a unit)."""
    units = []
    for item, (offset, count, start) in enumerate(zip(item_offsets, item_counts, item_starts)):
        for first in range(0, count, ATTENTION_UNIT):
            rows = min(ATTENTION_UNIT, count - first)
            units.append([item, offset + first, rows, start + first, (start + first + rows - 1) // ATTENTION_TILE + 1, 1])
    n_records = len(units)
    while units and (n_records + 1) * n_heads <= n_sms:
        longest = max(units, key=lambda u: -(-u[4] // u[5]))
        if -(-longest[4] // longest[5]) < 3 or longest[5] >= ATTENTION_MAX_PARTS:
            break
        longest[5] += 1
        n_records += 1
    records, n_split, most = [], 0, 1
    for item, first_row, rows, position, blocks, parts in units:
        share = -(-blocks // parts)
        for part in range(parts):
            records.append((item, first_row, rows, position, part, parts, n_split if parts > 1 else 0,
                            max(0, min(share, blocks - part * share))))
        if parts > 1:
            n_split += 1
            most = max(most, parts)
    records.sort(key=lambda record: -record[7])
    return records, n_split, most


def attention_prefill_two_tiles(out, q, k_pages, v_pages, block_table, units, n_units, n_heads, n_kv_heads, head_size,
                                page_size, scale, window, status, work, scratch=None, n_split=0, max_parts=1):
    """``attention_prefill`` for steps with long portions: one CTA per (record of the work
    list, head), each half of the unit with softmax warps of its own, one thread per query
    row; head size 64.  ``units``: device int32 [>= n_units, 8] from ``attention_units``.
    ``scratch``: (fp32 partial states, zeroed int32 counters) when units come in parts:
    n_split * heads * max_parts * 256 * (head_size + 4) floats and 2 * n_split * heads counters."""
    _check(out, "attention_prefill.out", torch.bfloat16, 2)
    _check(q, "attention_prefill.q", torch.bfloat16, 2)
    _check(k_pages, "attention_prefill.k_pages", torch.bfloat16, 4)
    _check(v_pages, "attention_prefill.v_pages", torch.bfloat16, 4)
    _check(block_table, "attention_prefill.block_table", torch.int32, 2)
    _check(units, "attention_prefill.units", torch.int32)
    _check(status, "attention_prefill.status", torch.int32)
    _check(work, "attention_prefill.work", torch.int32, 1)
    if work.shape[0] < 2:
        raise KernelError("attention_prefill: the work counter has two entries")
    if head_size != 64 or not attention_prefill_takes(q, head_size, page_size):
        raise KernelError(f"attention_prefill_two_tiles does not take head size {head_size} with pages of {page_size}")
    n_pages = k_pages.shape[0]
    if tuple(k_pages.shape) != (n_pages, page_size, n_kv_heads, head_size) or v_pages.shape != k_pages.shape:
        raise KernelError("attention_prefill: pages must be [n_pages, page_size, kv_heads, head_size]")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("attention_prefill: pages and block table must be contiguous")
    if q.shape[1] != n_heads * head_size or out.shape != q.shape or units.numel() < ATTENTION_TILE_RECORD * n_units:
        raise KernelError("attention_prefill: q / out / units do not fit")
    partial = counters = None
    if max_parts > 1:
        if scratch is None:
            raise KernelError("attention_prefill: units in parts need scratch")
        partial, counters = scratch
        _check(partial, "attention_prefill.scratch", torch.float32, 1)
        _check(counters, "attention_prefill.scratch", torch.int32, 1)
        if (partial.shape[0] < n_split * n_heads * max_parts * ATTENTION_UNIT * (head_size + 4)
                or counters.shape[0] < 2 * n_split * n_heads):
            raise KernelError("attention_prefill: scratch too small")
    _attention_prefill_two_tiles(out.data_ptr(), out.stride(0), q.data_ptr(), q.shape[0], q.shape[1], q.stride(0),
                                 k_pages.data_ptr(), v_pages.data_ptr(), n_pages, page_size, block_table.data_ptr(),
                                 block_table.shape[1], units.data_ptr(), n_units, n_heads, n_kv_heads, head_size,
                                 float(scale), int(window or 0), status.data_ptr(), _ptr(partial), _ptr(counters),
                                 int(max_parts), work.data_ptr(), _stream())
    return out


_sample_rows_sliced = Function("sampling", "mllm_sampling_sample_rows_sliced",
                               [P, P, L, I, I, P, P, P, P, P, P, P, I, P])
SAMPLE_SLICES = 32


def sample_rows_sliced(out, logits, temperature, top_p, seeds, counters, scratch, any_nucleus):
    """``sample_rows`` spread over 32 blocks per row.  scratch: (fp32 [R*32], int32 [R*32],
    zeroed int32 [R]); any_nucleus: whether some row has temperature > 0 and top_p < 1."""
    _check(out, "sample_rows.out", torch.int32, 1)
    _check(logits, "sample_rows.logits", torch.float32, 2)
    r, vocab = logits.shape
    values, indices, done = scratch
    _check(values, "sample_rows.scratch", torch.float32)
    _check(indices, "sample_rows.scratch", torch.int32)
    _check(done, "sample_rows.scratch", torch.int32)
    if values.numel() < r * SAMPLE_SLICES or indices.numel() < r * SAMPLE_SLICES or done.numel() < r or out.shape[0] < r:
        raise KernelError("sample_rows_sliced: scratch or output too small")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                        ("seeds", seeds, torch.int64), ("counters", counters, torch.int32)):
        if t is not None:
            _check(t, f"sample_rows.{name}", dt, 1)
            if t.shape[0] < r:
                raise KernelError(f"sample_rows: {name} too short")
    _sample_rows_sliced(out.data_ptr(), logits.data_ptr(), logits.stride(0), r, vocab, _ptr(temperature), _ptr(top_p),
                        _ptr(seeds), _ptr(counters), values.data_ptr(), indices.data_ptr(), done.data_ptr(),
                        int(bool(any_nucleus)), _stream())
    return out


_sample_rows_nucleus = Function("sampling", "mllm_sampling_sample_rows_nucleus", [P, P, L, I, I, P, P, P, P, P])


def sample_rows_nucleus(out, logits, temperature, top_p, seeds, counters):
    """Draw only the rows with a nucleus cut (temperature > 0, top_p < 1); the rest of ``out`` stays."""
    _check(out, "sample_rows.out", torch.int32, 1)
    _check(logits, "sample_rows.logits", torch.float32, 2)
    _check(temperature, "sample_rows.temperature", torch.float32, 1)
    _check(top_p, "sample_rows.top_p", torch.float32, 1)
    r, vocab = logits.shape
    _sample_rows_nucleus(out.data_ptr(), logits.data_ptr(), logits.stride(0), r, vocab, temperature.data_ptr(),
                         top_p.data_ptr(), _ptr(seeds), _ptr(counters), _stream())
    return out


_layernorm_warp = Function("decode", "mllm_decode_layernorm", [P, P, P, P, P, I, I, F, P])


def layernorm_warp(out, x, gamma, beta, eps, rows=None):
    """``layernorm`` into bfloat16 with one warp per row, the row read once (width % 4 == 0)."""
    _check(out, "layernorm.out", torch.bfloat16, 2)
    _check(x, "layernorm.x", torch.float32, 2)
    _check(gamma, "layernorm.gamma", torch.float32, 1)
    _check(beta, "layernorm.beta", torch.float32, 1)
    width = x.shape[1]
    if not x.is_contiguous() or not out.is_contiguous() or width % 4 != 0:
        raise KernelError("layernorm_warp: x and out must be contiguous, the width a multiple of 4")
    if out.shape[1] != width or gamma.shape[0] != width or beta.shape[0] != width:
        raise KernelError("layernorm_warp: widths do not agree")
    if rows is not None:
        _check(rows, "layernorm.rows", torch.int32, 1)
        if rows.shape[0] < out.shape[0]:
            raise KernelError("layernorm_warp: fewer row indices than output rows")
    elif x.shape[0] < out.shape[0]:
        raise KernelError("layernorm_warp: fewer input rows than output rows")
    _layernorm_warp(out.data_ptr(), x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), _ptr(rows), out.shape[0], width,
                    float(eps), _stream())
    return out


_keep_tokens = Function("sampling", "mllm_sampling_keep_tokens", [P, P, P, I, I, P])
_resolve_tokens = Function("sampling", "mllm_sampling_resolve_tokens", [P, P, I, I, P])


def keep_tokens(kept, slots, tokens):
    """kept[slots[r]] = tokens[r] for every row r with slots[r] >= 0 (all int32, on the device)."""
    _check(kept, "keep_tokens.kept", torch.int32, 1)
    _check(slots, "keep_tokens.slots", torch.int32, 1)
    _check(tokens, "keep_tokens.tokens", torch.int32, 1)
    n = tokens.shape[0]
    if slots.shape[0] < n:
        raise KernelError("keep_tokens: fewer slots than tokens")
    _keep_tokens(kept.data_ptr(), slots.data_ptr(), tokens.data_ptr(), n, kept.shape[0], _stream())
    return kept


def resolve_tokens(token_ids, kept):
    """token_ids[t] = kept[-1 - token_ids[t]] wherever token_ids[t] < 0 (in place)."""
    _check(token_ids, "resolve_tokens.token_ids", torch.int32, 1)
    _check(kept, "resolve_tokens.kept", torch.int32, 1)
    _resolve_tokens(token_ids.data_ptr(), kept.data_ptr(), token_ids.shape[0], kept.shape[0], _stream())
    return token_ids


_device_info = Function("plain", "mllm_plain_device_info", [ctypes.c_char_p, I, ctypes.POINTER(ctypes.c_int),
                                                            ctypes.POINTER(ctypes.c_long)])


def device_info() -> dict:
    """The current device as the kernel library sees it: name, compute capability, SM count,
    memory, CUDA runtime and driver versions."""
    name = ctypes.create_string_buffer(256)
    values = (ctypes.c_int * 5)()
    memory = ctypes.c_long()
    _device_info(name, 256, values, ctypes.byref(memory))
    return {"name": name.value.decode(), "compute": f"{values[0]}.{values[1]}", "sms": values[2],
            "memory_bytes": memory.value, "runtime": values[3], "driver": values[4]}


# ---- norms in groups, short convolutions, latent attention, matrix memories ----------------------

_grouped_rms_norm = Function("sequence", "mllm_sequence_grouped_rms_norm",
                             [P, L, P, L, P, P, P, L, I, I, I, F, I, I, I, I, P])

GATE_MODES = {"sigmoid": 1, "silu": 2, "silu_before": 3}


def grouped_rms_norm(out, x, gain, groups, eps, rows=None, gate=None, add=False, gate_mode="sigmoid"):
    """Rows of the fp32 ``x`` [*, width], cut into ``groups`` equal consecutive pieces, each divided by
    sqrt(mean(piece^2) + eps), the whole times ``gain``.  ``rows`` gathers input rows.  ``gate``
    [R, width]: the result is also multiplied by sigmoid(gate) (``gate_mode`` "sigmoid") or by
    silu(gate) ("silu"); with "silu_before" the input is multiplied by silu(gate) before the norm.
    ``add``: the fp32 ``out`` is added to.  ``out`` may be ``x``."""
    _check(out, "grouped_rms_norm.out", None, 2)
    _check(x, "grouped_rms_norm.x", torch.float32, 2)
    _check(gain, "grouped_rms_norm.gain", torch.float32, 1)
    n_rows, width = out.shape
    if x.shape[1] != width or gain.shape[0] != width or width % groups != 0:
        raise KernelError(f"grouped_rms_norm: widths do not agree, or {width} is not a multiple of {groups} groups")
    if rows is not None:
        _check(rows, "grouped_rms_norm.rows", torch.int32, 1)
        if rows.shape[0] < n_rows:
            raise KernelError("grouped_rms_norm: fewer row indices than output rows")
    elif x.shape[0] < n_rows:
        raise KernelError("grouped_rms_norm: fewer input rows than output rows")
    if gate is not None:
        _check(gate, "grouped_rms_norm.gate", None, 2)
        if gate.shape[0] < n_rows or gate.shape[1] != width:
            raise KernelError("grouped_rms_norm: the gate has another shape")
    if add and (out.dtype != torch.float32 or gate is not None):
        raise KernelError("grouped_rms_norm: the residual sum is kept in 32-bit and takes no gate")
    _grouped_rms_norm(out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), gain.data_ptr(), _ptr(rows), _ptr(gate),
                      gate.stride(0) if gate is not None else 0, n_rows, width, int(groups), float(eps), int(bool(add)),
                      dtype_code(out.dtype), dtype_code(gate.dtype) if gate is not None else 0, GATE_MODES[gate_mode],
                      _stream())
    return out


_causal_taps = Function("sequence", "mllm_sequence_causal_taps",
                        [P, L, P, L, P, P, P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P])


def causal_taps(out, h, w, state, positions, token_item, item_slot, item_start, item_offset, item_count, writes=True,
                identity=True, bias=None, silu=False, single_tokens=False):
    """out[t] = act(h[t] + bias + sum_j w[:, j] * h[t - (taps - 1) + j]) over the tokens of one request, per
    channel; what lies before this step's portion comes from ``state`` [slots, taps - 1, width]
    (fp32, oldest first), which is then moved on by this step's tokens (unless ``writes`` is false).
    ``identity`` false: the input itself is not added (a plain convolution); ``bias`` [width] fp32 or
    None; ``silu``: the activation.  ``h`` and ``out`` may be column ranges of wider buffers.
    ``single_tokens``: every entry brings one token; the state is then moved by the same kernel."""
    _check(out, "causal_taps.out", h.dtype, 2)
    _check(h, "causal_taps.h", None, 2)
    _check(w, "causal_taps.w", torch.float32, 2)
    _check(state, "causal_taps.state", torch.float32, 3)
    for name, t in (("positions", positions), ("token_item", token_item), ("item_slot", item_slot),
                    ("item_start", item_start), ("item_offset", item_offset), ("item_count", item_count)):
        _check(t, f"causal_taps.{name}", torch.int32, 1)
    n, width = h.shape
    taps = w.shape[1]
    if not w.is_contiguous() or w.shape[0] != width or out.shape != h.shape:
        raise KernelError("causal_taps: out, h and w must agree on the width")
    if bias is not None:
        _check(bias, "causal_taps.bias", torch.float32, 1)
        if bias.shape[0] != width:
            raise KernelError("causal_taps: one bias per channel")
    if tuple(state.shape[1:]) != (max(taps - 1, 0), width) or (taps > 1 and state.stride(1) != width):
        raise KernelError(f"causal_taps: the state must be [slots, {taps - 1}, {width}]")
    _causal_taps(out.data_ptr(), out.stride(0), h.data_ptr(), h.stride(0), w.data_ptr(), _ptr(bias), state.data_ptr(),
                 state.stride(0), positions.data_ptr(), token_item.data_ptr(), item_slot.data_ptr(), item_start.data_ptr(),
                 item_offset.data_ptr(), item_count.data_ptr(), n, item_count.shape[0], width, taps,
                 (2 if single_tokens else 1) if writes else 0, int(bool(identity)), int(bool(silu)), dtype_code(h.dtype), _stream())
    return out


_norm_taps_step = Function("sequence", "mllm_sequence_norm_taps_step", [P, P, P, P, P, L, P, P, I, I, I, F, I, I, I, P])


def norm_taps_step(out, x, gain, groups, eps, w, state, token_item, item_slot, writes=True):
    """A step of single tokens (one per entry): ``grouped_rms_norm`` of the fp32 rows ``x``, then
    ``causal_taps`` with every earlier input from ``state``, then the state moved on, in one kernel."""
    _check(out, "norm_taps_step.out", None, 2)
    _check(x, "norm_taps_step.x", torch.float32, 2)
    _check(gain, "norm_taps_step.gain", torch.float32, 1)
    _check(w, "norm_taps_step.w", torch.float32, 2)
    _check(state, "norm_taps_step.state", torch.float32, 3)
    n, width = out.shape
    taps = w.shape[1]
    if (not (out.is_contiguous() and x.is_contiguous() and w.is_contiguous()) or x.shape[0] < n or x.shape[1] != width
            or gain.shape[0] != width or w.shape[0] != width or width % groups != 0):
        raise KernelError("norm_taps_step: sizes do not agree")
    if taps < 2 or tuple(state.shape[1:]) != (taps - 1, width) or state.stride(1) != width:
        raise KernelError(f"norm_taps_step: the state must be [slots, {taps - 1}, {width}]")
    _norm_taps_step(out.data_ptr(), x.data_ptr(), gain.data_ptr(), w.data_ptr(), state.data_ptr(), state.stride(0),
                    token_item.data_ptr(), item_slot.data_ptr(), n, width, int(groups), float(eps), taps, int(bool(writes)),
                    dtype_code(out.dtype), _stream())
    return out


_latent_prepare = Function("sequence", "mllm_sequence_latent_prepare",
                           [P, P, P, P, L, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, P])
ROTARY_LAYOUTS = {"interleaved": 0, "half": 1}


def latent_prepare(pages, q_eff, down, q, gain, inv_freq, positions, token_item, block_table, page_size, rank, rot,
                   rot_dims, heads, dim, eps, writes=True, layout="interleaved"):
    """Per token: the first ``rank`` entries of the fp32 ``down`` row, normed by their root mean square
    and times ``gain``, and its last ``rot`` entries with rotary positions, go into the token's row
    of ``pages`` [n_pages, page_size, 1, rank + rot]; the rotated part of every head's query
    (``q`` [T, heads * (dim + rot)]) gets rotary positions and goes to
    ``q_eff`` [T, heads * (rank + rot)] (fp32), entries rank .. rank + rot of each head.  ``layout``: the
    pairs that turn together are neighbours ("interleaved") or half the rotated entries apart ("half").
    With ``writes`` false only the queries are prepared and ``down`` may be None."""
    _check(pages, "latent_prepare.pages", q.dtype)
    _check(q_eff, "latent_prepare.q_eff", torch.float32, 2)
    if down is None:
        if writes:
            raise KernelError("latent_prepare: an entry that stores its rows needs its projection")
        down = q_eff.new_empty((0, rank + rot))
    _check(down, "latent_prepare.down", torch.float32, 2)
    _check(q, "latent_prepare.q", None, 2)
    _check(gain, "latent_prepare.gain", torch.float32, 1)
    _check(inv_freq, "latent_prepare.inv_freq", torch.float64, 1)
    _check(block_table, "latent_prepare.block_table", torch.int32, 2)
    n = q.shape[0]
    row = rank + rot
    if (not down.is_contiguous() or down.shape[1] != row or not q_eff.is_contiguous() or q_eff.shape[1] != heads * row
            or q.shape[1] != heads * (dim + rot) or gain.shape[0] != rank or inv_freq.shape[0] < rot_dims // 2):
        raise KernelError("latent_prepare: sizes do not agree")
    if not pages.is_contiguous() or pages.numel() % (page_size * row) != 0 or not block_table.is_contiguous():
        raise KernelError("latent_prepare: the pages do not hold whole pages of rows of rank + rot")
    _latent_prepare(pages.data_ptr(), q_eff.data_ptr(), down.data_ptr() if down.numel() else None, q.data_ptr(), q.stride(0), gain.data_ptr(),
                    inv_freq.data_ptr(), positions.data_ptr(), token_item.data_ptr(), block_table.data_ptr(),
                    block_table.shape[1], page_size, n, rank, rot, rot_dims, heads, dim, float(eps), int(bool(writes)),
                    ROTARY_LAYOUTS[layout], dtype_code(q.dtype), _stream())


_head_linear = Function("sequence", "mllm_sequence_head_linear", [P, P, P, I, I, I, I, L, L, L, L, I, I, I, P])


def head_linear(out, a, w, heads, a_head, o_head):
    """out[t, head, :] = w[head] @ a[t, head, :] for every head: ``w`` [heads, N, K]; head ``h`` of
    ``a`` starts at column ``h * a_head`` (K entries), of ``out`` at ``h * o_head`` (N entries)."""
    _check(out, "head_linear.out", None, 2)
    _check(a, "head_linear.a", None, 2)
    _check(w, "head_linear.w", None, 3)
    m = a.shape[0]
    n, k = w.shape[1], w.shape[2]
    if (w.shape[0] != heads or not w.is_contiguous() or out.shape[0] != m or (heads - 1) * a_head + k > a.shape[1]
            or (heads - 1) * o_head + n > out.shape[1]):
        raise KernelError("head_linear: shapes do not agree")
    _head_linear(out.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, heads, a.stride(0), out.stride(0), a_head, o_head,
                 dtype_code(a.dtype), dtype_code(w.dtype), dtype_code(out.dtype), _stream())
    return out


_latent_attention = Function("sequence", "mllm_sequence_latent_attention", [P, P, P, P, I, P, P, I, I, I, I, I, F, I, I, P])


def latent_attention_plain(out, q_eff, pages, block_table, positions, token_item, heads, rank, rot, page_size, scale,
                           window=0):
    """Causal attention of every token of the step over its request's cached rows [rank + rot]:
    score = q_eff[t, head] . row * scale, value = the row's first ``rank`` entries;
    out [T, heads * rank] in 32-bit."""
    _check(out, "latent_attention.out", torch.float32, 2)
    _check(q_eff, "latent_attention.q_eff", torch.float32, 2)
    _check(pages, "latent_attention.pages")
    _check(block_table, "latent_attention.block_table", torch.int32, 2)
    n = q_eff.shape[0]
    if (not out.is_contiguous() or not q_eff.is_contiguous() or out.shape != (n, heads * rank)
            or q_eff.shape[1] != heads * (rank + rot) or not pages.is_contiguous() or not block_table.is_contiguous()):
        raise KernelError("latent_attention: sizes do not agree")
    _latent_attention(out.data_ptr(), q_eff.data_ptr(), pages.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                      positions.data_ptr(), token_item.data_ptr(), n, heads, rank, rot, page_size, float(scale),
                      int(window or 0), dtype_code(pages.dtype), _stream())
    return out


class _LatentTiledParams(ctypes.Structure):
    _fields_ = [("out", P), ("part_out", P), ("part_ml", P), ("q_eff", P), ("pages", P), ("block_table", P),
                ("positions", P), ("token_item", P), ("tiles", P), ("max_blocks", I), ("page_size", I), ("n_tokens", I),
                ("heads", I), ("rank", I), ("rot", I), ("TQ", I), ("HB", I), ("parts", I),
                ("scale", F), ("out_bf16", I), ("key_buffers", I), ("window", I)]


_latent_attention_tiled = Function("sequence", "mllm_sequence_latent_attention_tiled",
                                   [ctypes.POINTER(_LatentTiledParams), I, I, P])
LATENT_TILE_ROWS = 32


def latent_attention_tiled_takes(pages, rank, rot) -> bool:
    """Whether the tiled kernel takes the sizes: rows of a multiple of 4 entries whose latent part is
    a multiple of 8 (at most 1024), and 32 effective queries plus 32 cached rows in shared memory."""
    row = rank + rot
    shared = 32 * (row + 4) * 4 + 32 * 33 * 4 + 64 * 4 + 32 * (row + 4) * pages.element_size()
    return row % 4 == 0 and rank % 8 == 0 and rank <= 1024 and shared <= 220 * 1024


def latent_heads_per_block(heads: int) -> int:
    """Heads of one block of 32 rows in prompt portions: the power of two (32 at most) that leaves
    the fewest rows for heads that do not exist, the larger one on a tie; the block then takes
    32 / that many consecutive tokens.  (12 heads: 4 a block and 8 tokens, no row idle; 16 a block
    would idle a quarter of the rows, and a cached row read thrice costs less than that.)"""
    return min((32, 16, 8, 4, 2, 1), key=lambda block: (-(-heads // block) * block, -block))


def latent_attention_tiled(out, q_eff, pages, block_table, positions, token_item, heads, rank, rot, page_size, scale,
                           tiles=None, n_tiles=0, parts=1, scratch=None, window=0):
    """``latent_attention_plain`` in tiles of 32 query rows that share their keys.  With ``tiles``
    (the step's work list, device int32 records of 8, ``n_tiles`` of them) for prompt portions;
    without, for single tokens, the keys of each in ``parts`` runs (the token's context length over
    ``parts``, in whole blocks of 32) whose results are merged (``scratch``: fp32 (T * heads * parts * rank, T * heads * parts * 2)).
    ``out`` may be bfloat16: the sums are 32-bit either way, the result is rounded once."""
    _check(out, "latent_attention.out", None, 2)
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("latent_attention_tiled: out must be float32 or bfloat16")
    _check(q_eff, "latent_attention.q_eff", torch.float32, 2)
    _check(pages, "latent_attention.pages")
    _check(block_table, "latent_attention.block_table", torch.int32, 2)
    n = q_eff.shape[0]
    if (not out.is_contiguous() or not q_eff.is_contiguous() or out.shape != (n, heads * rank)
            or q_eff.shape[1] != heads * (rank + rot) or not pages.is_contiguous() or not block_table.is_contiguous()):
        raise KernelError("latent_attention: sizes do not agree")
    if not latent_attention_tiled_takes(pages, rank, rot):
        raise KernelError(f"latent_attention_tiled does not take rows of {rank} + {rot}")
    params = _LatentTiledParams()
    params.out, params.q_eff, params.pages = out.data_ptr(), q_eff.data_ptr(), pages.data_ptr()
    params.block_table, params.positions, params.token_item = block_table.data_ptr(), positions.data_ptr(), token_item.data_ptr()
    params.max_blocks, params.page_size, params.n_tokens = block_table.shape[1], page_size, n
    params.heads, params.rank, params.rot, params.scale = heads, rank, rot, float(scale)
    params.out_bf16 = int(out.dtype == torch.bfloat16)
    params.window = int(window or 0)           # (> 0: a query sees the last ``window`` positions only)
    if tiles is not None:
        _check(tiles, "latent_attention.tiles", torch.int32)
        if tiles.numel() < ATTENTION_TILE_RECORD * n_tiles or parts != 1:
            raise KernelError("latent_attention_tiled: the work list is shorter than stated, or parts were asked for")
        params.tiles = tiles.data_ptr()
        params.HB = latent_heads_per_block(heads)
        params.TQ = LATENT_TILE_ROWS // params.HB
        params.parts, units = 1, n_tiles
    else:
        # (a block of 16 rows where that holds every head: no thread then works for a row that is nobody's)
        params.HB, params.TQ, params.parts, units = (16 if heads <= 16 else LATENT_TILE_ROWS), 1, int(parts), n
        if parts > 1:
            part_out, part_ml = scratch
            _check(part_out, "latent_attention.scratch", torch.float32)
            _check(part_ml, "latent_attention.scratch", torch.float32)
            if part_out.numel() < n * heads * parts * rank or part_ml.numel() < n * heads * parts * 2:
                raise KernelError("latent_attention_tiled: scratch too small")
            params.part_out, params.part_ml = part_out.data_ptr(), part_ml.data_ptr()
    _latent_attention_tiled(ctypes.byref(params), units, dtype_code(pages.dtype), _stream())
    return out


class _MemoryScanParams(ctypes.Structure):
    _fields_ = [("out", P), ("ld_out", L), ("q", P), ("k", P), ("v", P), ("ld_q", L), ("ld_k", L), ("ld_v", L),
                ("gates", P), ("ld_gates", L), ("gate_bias", P), ("decay", P), ("state", P), ("state_stride", L),
                ("item_slot", P), ("item_offset", P), ("item_count", P), ("heads", I), ("dim", I), ("vdim", I),
                ("q_scale", F), ("gate_cap", F), ("silu", I), ("writes", I)]


_memory_scan = Function("sequence", "mllm_sequence_memory_scan", [ctypes.POINTER(_MemoryScanParams), I, I, P])
_memory_chunk = Function("sequence", "mllm_sequence_memory_chunk", [ctypes.POINTER(_MemoryScanParams), I, I, P])


class _MemoryPassParams(ctypes.Structure):
    _fields_ = [("base", _MemoryScanParams), ("gate_arrays", P), ("chunk_state", P), ("chunk_norm", P), ("max_chunks", I),
                ("n_items", I)]


_memory_passes = Function("sequence", "mllm_sequence_memory_passes", [ctypes.POINTER(_MemoryPassParams), I, P])


def memory_passes_scratch(n_tokens, n_items, heads, dim, vdim):
    """Floats of scratch ``memory_scan(..., passes=...)`` needs: (gate arrays, chunk states, chunk norms)."""
    chunks = n_tokens // 32 + n_items
    return n_tokens * heads * 5, chunks * heads * dim * vdim, chunks * heads * dim


def memory_chunk_takes(dim) -> bool:
    """Whether the chunked kernel takes the key size: a chunk's q and k and a slice of the state
    lie in shared memory (the launcher's own arithmetic)."""
    padded = (dim + 3) & ~3
    return 4 * (2 * 32 * (padded + 4) + 32 * 32 + padded * 32 + 32 * 36 + padded + 6 * 32 + 33) <= 200 * 1024


def memory_state_floats(heads, dim, vdim, gated) -> int:
    """Floats of a request's matrix-memory state: S [heads, dim, vdim], and, gated, n [heads, dim]
    and m [heads]."""
    return heads * dim * vdim + (heads * dim + heads if gated else 0)


def memory_scan(out, q, k, v, state, item_slot, item_offset, item_count, heads, dim, vdim, q_scale=1.0, silu=False,
                gates=None, gate_bias=None, gate_cap=0.0, decay=None, writes=True, chunked=False, passes=None):
    """The matrix-memory recurrence over each entry's tokens, in order:
    S <- a S + b k v^T, out = S^T q, with a fixed decay per head (``decay`` [heads]; a = decay,
    b = 1) or with ``gates`` [T, 2 * heads] (fp32: input gates then forget gates, ``gate_bias``
    added): capped, exponential, stabilised by a running maximum, the output divided by
    max(|n . q|, exp(-m)) + 1e-6.  q, k [T, heads * dim], v [T, heads * vdim] (any row stride);
    out fp32 [T, heads * vdim]; ``state`` fp32 [slots, memory_state_floats(...)].
    ``chunked``: the kernel for prompt portions, which takes 32 tokens at a time (the same sums in
    another order); without, every token is a step of its own (single decoded tokens).
    ``passes``: three fp32 scratch tensors of ``memory_passes_scratch`` floats: the chunks are then
    taken side by side (their own sums, a scan over the chunks' states, their outputs) instead of
    one after the other."""
    _check(out, "memory_scan.out", torch.float32, 2)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check(t, f"memory_scan.{name}", q.dtype, 2)
    _check(state, "memory_scan.state", torch.float32, 2)
    n = q.shape[0]
    gated = gates is not None
    if (q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * vdim
            or out.shape != (n, heads * vdim) or state.shape[1] != memory_state_floats(heads, dim, vdim, gated)
            or state.stride(1) != 1):
        raise KernelError("memory_scan: sizes do not agree")
    params = _MemoryScanParams()
    params.out, params.ld_out = out.data_ptr(), out.stride(0)
    params.q, params.k, params.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    params.ld_q, params.ld_k, params.ld_v = q.stride(0), k.stride(0), v.stride(0)
    if gated:
        _check(gates, "memory_scan.gates", torch.float32, 2)
        _check(gate_bias, "memory_scan.gate_bias", torch.float32, 1)
        if gates.shape[1] != 2 * heads or gate_bias.shape[0] != 2 * heads or gate_cap <= 0:
            raise KernelError("memory_scan: gates are [T, 2 * heads] with a positive cap")
        params.gates, params.ld_gates, params.gate_bias = gates.data_ptr(), gates.stride(0), gate_bias.data_ptr()
    else:
        _check(decay, "memory_scan.decay", torch.float32, 1)
        if decay.shape[0] != heads:
            raise KernelError("memory_scan: one decay per head")
        params.decay = decay.data_ptr()
    params.state, params.state_stride = state.data_ptr(), state.stride(0)
    params.item_slot, params.item_offset, params.item_count = item_slot.data_ptr(), item_offset.data_ptr(), item_count.data_ptr()
    params.heads, params.dim, params.vdim = heads, dim, vdim
    params.q_scale, params.gate_cap = float(q_scale), float(gate_cap)
    params.silu, params.writes = int(bool(silu)), int(bool(writes))
    if (chunked or passes is not None) and not memory_chunk_takes(dim):
        raise KernelError(f"memory_scan: the chunked kernels do not take a key size of {dim}")
    if passes is not None:
        n_items = item_count.shape[0]
        need = memory_passes_scratch(n, n_items, heads, dim, vdim)
        for t, floats in zip(passes, need):
            _check(t, "memory_scan.passes", torch.float32, 1)
            if t.shape[0] < floats:
                raise KernelError("memory_scan: scratch for the passes over chunks is too small")
        both = _MemoryPassParams()
        both.base = params
        both.gate_arrays, both.chunk_state, both.chunk_norm = (t.data_ptr() for t in passes)
        both.max_chunks, both.n_items = n // 32 + n_items, n_items
        _memory_passes(ctypes.byref(both), dtype_code(q.dtype), _stream())
        return out
    (_memory_chunk if chunked else _memory_scan)(ctypes.byref(params), item_count.shape[0], dtype_code(q.dtype), _stream())
    return out


_depth_mix = Function("sequence", "mllm_sequence_depth_mix", [P, P, P, I, I, I, I, P])


def depth_mix(hidden, kept, weights, index):
    """kept[:, index] = hidden; then, with ``weights`` [index + 1] (fp32), hidden = sum over
    j <= index of weights[j] * kept[:, j].  kept: fp32 [T, planes, width]."""
    _check(hidden, "depth_mix.hidden", torch.float32, 2)
    _check(kept, "depth_mix.kept", torch.float32, 3)
    n, width = hidden.shape
    if not hidden.is_contiguous() or not kept.is_contiguous() or kept.shape[0] != n or kept.shape[2] != width:
        raise KernelError("depth_mix: hidden [T, width] and kept [T, planes, width] must be contiguous")
    if weights is not None:
        _check(weights, "depth_mix.weights", torch.float32, 1)
        if weights.shape[0] != index + 1:
            raise KernelError(f"depth_mix: {weights.shape[0]} weights for {index + 1} results")
    _depth_mix(hidden.data_ptr(), kept.data_ptr(), _ptr(weights), index, kept.shape[1], n, width, _stream())
    return hidden


# ---- rotary positions with a cache store, capped attention, linear recurrences, routed experts ----

_rotary_store = Function("hybrid", "mllm_hybrid_rotary_store",
                         [P, L, I, I, I, I, I, I, I, P, ctypes.c_double, P, P, P, I, I, P, P, I, I, I, P])


def rotary_store(qkv, k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, inv_freq, amplitude, positions, token_item,
                 block_table, page_size, k_pages, v_pages, writes=True):
    """Rows of ``qkv`` hold [q | k | v] (k from column ``k_off``, v from ``v_off``).  The first
    ``rot_dims`` entries of every query and key head turn in interleaved pairs by
    position * ``inv_freq`` [rot_dims / 2] (float64); cosine and sine are multiplied by ``amplitude``.
    Queries and keys are rotated in place; keys and values go to the token's place in the pages."""
    _check(qkv, "rotary_store.qkv", None, 2)
    _check(inv_freq, "rotary_store.inv_freq", torch.float64, 1)
    _check(k_pages, "rotary_store.k_pages", qkv.dtype)
    _check(v_pages, "rotary_store.v_pages", qkv.dtype)
    _check(block_table, "rotary_store.block_table", torch.int32, 2)
    if inv_freq.shape[0] < max(rot_dims // 2, 1) or v_off + kv_heads * vdim > qkv.shape[1] or k_off + kv_heads * dim > qkv.shape[1]:
        raise KernelError("rotary_store: sizes do not agree")
    if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous()
            or k_pages.numel() % (page_size * kv_heads * dim) != 0 or v_pages.numel() % (page_size * kv_heads * vdim) != 0):
        raise KernelError("rotary_store: the pages do not hold whole pages of these rows")
    _rotary_store(qkv.data_ptr(), qkv.stride(0), k_off, v_off, heads, kv_heads, dim, vdim, rot_dims, inv_freq.data_ptr(),
                  float(amplitude), positions.data_ptr(), token_item.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                  page_size, k_pages.data_ptr(), v_pages.data_ptr(), int(bool(writes)), qkv.shape[0], dtype_code(qkv.dtype),
                  _stream())


_capped_attention = Function("hybrid", "mllm_hybrid_capped_attention",
                             [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, I, F, F, I, I, P, L, P, I, I, P])


def capped_attention_tiled_takes(dim, vdim, dtype=torch.bfloat16) -> bool:
    """Whether the tiled kernel takes the sizes: keys and values come in whole 16-byte vectors, and
    a block's queries, 32 keys and 32 values lie in shared memory in 32-bit (the launcher's own
    arithmetic)."""
    vec = 4 if dtype == torch.float32 else 8
    return (0 < dim <= 256 and 0 < vdim <= 256 and dim % vec == 0 and vdim % vec == 0
            and 4 * (16 * dim + 32 * (dim + 4) + 32 * vdim + 512) <= 160 * 1024)


def capped_attention(out, q, k_pages, v_pages, block_table, positions, token_item, n_heads, n_kv_heads, dim, vdim,
                     page_size, scale, cap=0.0, window=0, tiled=False, chunk=0, gate=None, sink=None):
    """Causal attention of every token of the step over its request's pages, keys of ``dim`` and
    values of ``vdim`` entries per head, score = cap * tanh(q . k * scale / cap) (``cap`` 0: no cap);
    scores, weights and the weighted sum in 32-bit.  ``window`` > 0: the last ``window`` positions only;
    ``chunk`` > 0: only keys of the query's own block of ``chunk`` positions (blocks counted from
    position 0).  ``gate`` fp32 [T, >= heads]: head h's result is multiplied by sigmoid(gate[t, h]).
    ``sink`` fp32 [heads]: the softmax's denominator also holds exp(sink[h]), a term with no key and no value.
    ``tiled``: consecutive tokens of a request share the cached rows they read (for steps with prompt
    portions)."""
    _check(out, "capped_attention.out", q.dtype, 2)
    _check(q, "capped_attention.q", None, 2)
    _check(k_pages, "capped_attention.k_pages", q.dtype)
    _check(v_pages, "capped_attention.v_pages", q.dtype)
    _check(block_table, "capped_attention.block_table", torch.int32, 2)
    n = q.shape[0]
    if q.shape[1] != n_heads * dim or out.shape != (n, n_heads * vdim):
        raise KernelError("capped_attention: q / out do not have heads * size columns")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("capped_attention: pages and block table must be contiguous")
    if gate is not None:
        _check(gate, "capped_attention.gate", torch.float32, 2)
        if gate.shape[0] < n or gate.shape[1] < n_heads or gate.stride(1) != 1:
            raise KernelError("capped_attention: one gate per token and head")
    _check_sink(sink, n_heads, "capped_attention")
    _capped_attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                      block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), token_item.data_ptr(), n, n_heads,
                      n_kv_heads, dim, vdim, page_size, float(scale), float(cap or 0.0), int(window or 0), int(chunk or 0),
                      _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(sink), int(bool(tiled)), dtype_code(q.dtype),
                      _stream())
    return out


_head_norm_store = Function("hybrid", "mllm_hybrid_head_norm_store",
                            [P, L, I, I, I, I, I, I, F, P, P, P, I, I, P, P, I, I, I, P])


def head_norm_store(qkv, k_off, v_off, heads, kv_heads, dim, vdim, eps, positions, token_item, block_table, page_size,
                    k_pages, v_pages, writes=True):
    """Rows of ``qkv`` hold [q | k | v] (k from column ``k_off``, v from ``v_off``).  Every query and
    key head is divided by its root mean square, x / sqrt(mean(x^2) + eps), in place (``eps`` < 0: left as
    they are); the keys and the values go to the token's place in the pages."""
    _check(qkv, "head_norm_store.qkv", None, 2)
    _check(k_pages, "head_norm_store.k_pages", qkv.dtype)
    _check(v_pages, "head_norm_store.v_pages", qkv.dtype)
    _check(block_table, "head_norm_store.block_table", torch.int32, 2)
    if (heads * dim > k_off or k_off + kv_heads * dim > v_off or v_off + kv_heads * vdim > qkv.shape[1] or qkv.stride(1) != 1):
        raise KernelError("head_norm_store: sizes do not agree")
    if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous()
            or k_pages.numel() % (page_size * kv_heads * dim) != 0 or v_pages.numel() % (page_size * kv_heads * vdim) != 0):
        raise KernelError("head_norm_store: the pages do not hold whole pages of these rows")
    _head_norm_store(qkv.data_ptr(), qkv.stride(0), k_off, v_off, heads, kv_heads, dim, vdim, float(eps), positions.data_ptr(),
                     token_item.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, k_pages.data_ptr(),
                     v_pages.data_ptr(), int(bool(writes)), qkv.shape[0], dtype_code(qkv.dtype), _stream())


class _RecurrenceParams(ctypes.Structure):
    _fields_ = [("out", P), ("ld_out", L), ("q", P), ("k", P), ("v", P), ("ld_q", L), ("ld_k", L), ("ld_v", L),
                ("gate_a", P), ("gate_b", P), ("ld_gate_a", L), ("ld_gate_b", L), ("log_rate", P), ("step_bias", P),
                ("skip", P), ("state", P), ("state_stride", L), ("item_slot", P), ("item_offset", P), ("item_count", P),
                ("heads", I), ("qk_heads", I), ("dim", I), ("vdim", I), ("q_scale", F), ("delta", I), ("unit_norm", I),
                ("writes", I), ("channel_decay", I)]


_linear_recurrence = Function("hybrid", "mllm_hybrid_linear_recurrence", [ctypes.POINTER(_RecurrenceParams), I, I, I, P])


def linear_recurrence(out, q, k, v, gate_a, gate_b, log_rate, step_bias, state, item_slot, item_offset, item_count, heads,
                      qk_heads, dim, vdim, delta, unit_norm=False, q_scale=1.0, skip=None, writes=True, channel_decay=False):
    """Per entry, its tokens in order, per head with the state S [dim, vdim] (fp32, in ``state``
    [slots, heads * dim * vdim]): step = softplus(gate_a[t, h] + step_bias[h]), a = exp(-exp(log_rate[h]) * step);
    without ``delta``: u = step * v; with: u = sigmoid(gate_b[t, h]) * (v - (a S)^T k); S <- a S + k u^T;
    out[t, h] = S^T q (+ skip[h] * v).  q, k [T, qk_heads * dim] (head h reads h // (heads // qk_heads)),
    v [T, heads * vdim], any row stride; gates fp32 [T, heads]; out fp32 [T, heads * vdim].  ``unit_norm``:
    q and k are divided by sqrt(sum(x^2) + 1e-6) per head first; q is multiplied by ``q_scale``.
    ``channel_decay``: one decay per key channel, a[i] = exp(-exp(log_rate[h]) * softplus(gate_a[t, h, i] + step_bias[h, i]))
    with gate_a [T, heads * dim] and step_bias [heads * dim]; row i of S is multiplied by a[i] before it is read."""
    _check(out, "linear_recurrence.out", torch.float32, 2)
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check(t, f"linear_recurrence.{name}", q.dtype, 2)
    _check(gate_a, "linear_recurrence.gate_a", torch.float32, 2)
    _check(state, "linear_recurrence.state", torch.float32, 2)
    for name, t in (("log_rate", log_rate), ("step_bias", step_bias)):
        _check(t, f"linear_recurrence.{name}", torch.float32, 1)
    n = q.shape[0]
    if (q.shape[1] != qk_heads * dim or k.shape[1] != qk_heads * dim or v.shape[1] != heads * vdim
            or out.shape != (n, heads * vdim) or state.shape[1] != heads * dim * vdim or state.stride(1) != 1
            or gate_a.shape[1] < heads * (dim if channel_decay else 1) or log_rate.shape[0] != heads
            or step_bias.shape[0] != heads * (dim if channel_decay else 1) or gate_a.stride(1) != 1):
        raise KernelError("linear_recurrence: sizes do not agree")
    params = _RecurrenceParams()
    params.out, params.ld_out = out.data_ptr(), out.stride(0)
    params.q, params.k, params.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    params.ld_q, params.ld_k, params.ld_v = q.stride(0), k.stride(0), v.stride(0)
    params.gate_a, params.ld_gate_a = gate_a.data_ptr(), gate_a.stride(0)
    if gate_b is not None:
        _check(gate_b, "linear_recurrence.gate_b", torch.float32, 2)
        params.gate_b, params.ld_gate_b = gate_b.data_ptr(), gate_b.stride(0)
    elif delta:
        raise KernelError("linear_recurrence: the delta rule needs its write gates")
    params.log_rate, params.step_bias = log_rate.data_ptr(), step_bias.data_ptr()
    if skip is not None:
        _check(skip, "linear_recurrence.skip", torch.float32, 1)
        params.skip = skip.data_ptr()
    params.state, params.state_stride = state.data_ptr(), state.stride(0)
    params.item_slot, params.item_offset, params.item_count = item_slot.data_ptr(), item_offset.data_ptr(), item_count.data_ptr()
    params.heads, params.qk_heads, params.dim, params.vdim = heads, qk_heads, dim, vdim
    params.q_scale, params.delta, params.unit_norm, params.writes = float(q_scale), int(bool(delta)), int(bool(unit_norm)), int(bool(writes))
    params.channel_decay = int(bool(channel_decay))
    _linear_recurrence(ctypes.byref(params), item_count.shape[0], n, dtype_code(q.dtype), _stream())
    return out


_route = Function("hybrid", "mllm_hybrid_route", [P, L, P, P, P, I, I, I, I, I, P, P, P, I, I, P])
_experts = Function("hybrid", "mllm_hybrid_experts", [P, L, P, L, P, L, P, P, P, P, P, P, P, L, I, I, I, I, I, I, P])
_expert_combine = Function("hybrid", "mllm_hybrid_expert_combine", [P, L, P, L, P, P, P, I, I, I, I, I, I, I, P])


def route(x, router, shared_gate, top, choice, in_weight, out_weight, bias=None, softmax_of_chosen=False, shared_plain=False):
    """Per row of ``x``: sigmoid scores of ``router`` [experts, width] (sums in 32-bit), the ``top``
    largest with their scores as input weights; with ``shared_gate`` [1, width] one more pair per
    token: expert ``experts``, input weight 1, output weight sigmoid(shared_gate . x); ``shared_plain``:
    that pair with output weight 1 and no gate.  ``softmax_of_chosen``: the logits (plus ``bias`` fp32
    [experts]) rank the experts, and the chosen ones get input weight 1 and, as output weight, the
    softmax over the chosen logits only.  choice int32, in_weight / out_weight fp32: [T * pairs]."""
    _check(x, "route.x", None, 2)
    _check(router, "route.router", x.dtype, 2)
    _check(choice, "route.choice", torch.int32, 1)
    _check(in_weight, "route.in_weight", torch.float32, 1)
    _check(out_weight, "route.out_weight", torch.float32, 1)
    n, width = x.shape
    pairs = top + (1 if shared_gate is not None or shared_plain else 0)
    if router.shape[1] != width or not router.is_contiguous() or min(choice.shape[0], in_weight.shape[0], out_weight.shape[0]) < n * pairs:
        raise KernelError("route: sizes do not agree")
    if bias is not None:
        _check(bias, "route.bias", torch.float32, 1)
        if bias.shape[0] != router.shape[0]:
            raise KernelError("route: one bias per expert")
    if shared_gate is not None:
        _check(shared_gate, "route.shared_gate", x.dtype)
        if shared_gate.numel() != width or not shared_gate.is_contiguous():
            raise KernelError("route: the shared expert's gate is one row of the width")
    _route(x.data_ptr(), x.stride(0), router.data_ptr(), _ptr(bias), _ptr(shared_gate), int(bool(shared_plain)),
           int(bool(softmax_of_chosen)), width, router.shape[0], top, choice.data_ptr(), in_weight.data_ptr(),
           out_weight.data_ptr(), n, dtype_code(x.dtype), _stream())


def experts(hidden, act, x, choice, in_weight, out_weight, gate_of, up_of, down_of, inner_of, max_inner, pairs, ld_down=None,
            assign=False):
    """hidden[t] += sum over the token's ``pairs`` of out_weight * W_down[e] (silu(W_gate[e] x') * (W_up[e] x')),
    x' = in_weight * x[t] rounded to the activations' type; expert e's matrices are named by the
    int64 pointer tables ``gate_of``, ``up_of``, ``down_of`` and its inner size by ``inner_of`` (int32);
    the rows of every down matrix lie ``ld_down`` elements apart (None: ``max_inner``, for experts of
    one size that are stored each by itself).  ``act`` [T * pairs, max_inner] is scratch.  ``assign``: ``hidden`` is set
    to the sum instead of added to."""
    _check(hidden, "experts.hidden", torch.float32, 2)
    _check(x, "experts.x", None, 2)
    _check(act, "experts.act", x.dtype, 2)
    for name, t in (("gate_of", gate_of), ("up_of", up_of), ("down_of", down_of)):
        _check(t, f"experts.{name}", torch.int64, 1)
    _check(inner_of, "experts.inner_of", torch.int32, 1)
    n, width = x.shape
    if hidden.shape != (n, width) or act.shape[0] < n * pairs or act.shape[1] < max_inner:
        raise KernelError("experts: sizes do not agree")
    _experts(hidden.data_ptr(), hidden.stride(0), act.data_ptr(), act.stride(0), x.data_ptr(), x.stride(0), choice.data_ptr(),
             in_weight.data_ptr(), out_weight.data_ptr(), gate_of.data_ptr(), up_of.data_ptr(), down_of.data_ptr(),
             inner_of.data_ptr(), int(ld_down if ld_down is not None else max_inner), int(max_inner), width, int(pairs), n,
             int(bool(assign)), dtype_code(x.dtype), _stream())
    return hidden


def expert_combine(act, gu, choice, in_weight, out_weight, n_experts, inner, top, pairs):
    """For the products over all experts at once: ``gu`` [T, 2 * total] holds every expert's gate and
    up results ([gates | ups], routed expert e in columns [e * inner, (e + 1) * inner), the shared
    expert behind them); act[t, c] = silu(s g) * (s u) * out_weight with s the token's input weight
    for the column's expert, or 0 for an expert it did not choose.  act: [T, total]."""
    _check(act, "expert_combine.act", gu.dtype, 2)
    _check(gu, "expert_combine.gu", None, 2)
    n, total = act.shape
    if gu.shape != (n, 2 * total) or total < n_experts * inner or (pairs == top and total != n_experts * inner):
        raise KernelError("expert_combine: sizes do not agree")
    _expert_combine(act.data_ptr(), act.stride(0), gu.data_ptr(), gu.stride(0), choice.data_ptr(), in_weight.data_ptr(),
                    out_weight.data_ptr(), n_experts, inner, total, top, pairs, n, dtype_code(gu.dtype), _stream())
    return act


_scaled_add = Function("hybrid", "mllm_hybrid_scaled_add", [P, P, F, P, F, L, I, P])


def scaled_add(x, u, a, v=None, b=0.0, assign=False):
    """x += a * u + b * v (fp32, contiguous, equal shapes; ``v`` may be None); ``assign``: x = a * u + b * v."""
    _check(x, "scaled_add.x", torch.float32)
    _check(u, "scaled_add.u", torch.float32)
    if not x.is_contiguous() or not u.is_contiguous() or u.shape != x.shape:
        raise KernelError("scaled_add: x and u must be contiguous and of one shape")
    if v is not None:
        _check(v, "scaled_add.v", torch.float32)
        if not v.is_contiguous() or v.shape != x.shape:
            raise KernelError("scaled_add: v must be contiguous and of x's shape")
    _scaled_add(x.data_ptr(), u.data_ptr(), float(a), _ptr(v), float(b), x.numel(), int(bool(assign)), _stream())
    return x


# ---- residual streams (hyper-connections) and gated feed-forwards --------------------------------------

_streams_fill = Function("streams", "mllm_streams_fill", [P, P, I, I, I, P])
_streams_step = Function("streams", "mllm_streams_step", [P, P, L, P, P, I, P, P, L, P, L, P, F, I, I, I, I, P])
_gated_act = Function("streams", "mllm_streams_gated_act", [P, L, P, L, I, I, I, I, P])
MAX_STREAMS = 16
GATED_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "none": 2}


def streams_fill(streams, hidden):
    """Every stream of ``streams`` [T, s, width] (fp32) becomes the token's row of ``hidden`` [T, width]."""
    _check(streams, "streams_fill.streams", torch.float32, 3)
    _check(hidden, "streams_fill.hidden", torch.float32, 2)
    n, count, width = streams.shape
    if not streams.is_contiguous() or not hidden.is_contiguous() or hidden.shape != (n, width):
        raise KernelError("streams_fill: sizes do not agree")
    _streams_fill(streams.data_ptr(), hidden.data_ptr(), count, width, n, _stream())
    return streams


def streams_step(streams, y=None, mix=None, w_out=None, read=False, w_in=None, u_out=None, normed=None, gain=None, eps=0.0):
    """One pass over ``streams`` [T, s, width] (fp32, changed in place).  With ``y`` [T, width] (fp32), a
    sublayer's result: x_t <- sum_s mix[s, t] x_s + w_out[t] y for all streams at once.  With ``read``: the
    read-out u = sum_s w_in[s] x_s of the streams as they then are (``w_in`` None: their plain sum) goes to
    ``u_out`` (fp32) and / or, divided by its root mean square (eps inside the root) and times ``gain``, to
    ``normed`` (float32 or bfloat16)."""
    _check(streams, "streams_step.streams", torch.float32, 3)
    n, count, width = streams.shape
    if not streams.is_contiguous() or count > MAX_STREAMS:
        raise KernelError(f"streams_step: contiguous streams, at most {MAX_STREAMS}")
    if y is not None:
        _check(y, "streams_step.y", torch.float32, 2)
        _check(mix, "streams_step.mix", torch.float32, 2)
        _check(w_out, "streams_step.w_out", torch.float32, 1)
        if y.shape != (n, width) or y.stride(1) != 1 or tuple(mix.shape) != (count, count) or not mix.is_contiguous() or w_out.shape[0] != count:
            raise KernelError("streams_step: the result or the mixing weights have another shape")
    for name, t, dims in (("w_in", w_in, 1), ("u_out", u_out, 2), ("gain", gain, 1)):
        if t is not None:
            _check(t, f"streams_step.{name}", torch.float32, dims)
    if normed is not None:
        _check(normed, "streams_step.normed", None, 2)
        if gain is None or gain.shape[0] != width or normed.shape != (n, width) or normed.stride(1) != 1 or not read:
            raise KernelError("streams_step: the normed read-out needs a gain of the width")
    if (w_in is not None and w_in.shape[0] != count) or (u_out is not None and (u_out.shape != (n, width) or u_out.stride(1) != 1)):
        raise KernelError("streams_step: the read-out's weights or result have another shape")
    _streams_step(streams.data_ptr(), _ptr(y), y.stride(0) if y is not None else 0, _ptr(mix), _ptr(w_out), int(bool(read)),
                  _ptr(w_in), _ptr(u_out), u_out.stride(0) if u_out is not None else 0, _ptr(normed),
                  normed.stride(0) if normed is not None else 0, _ptr(gain), float(eps), count, width, n,
                  dtype_code(normed.dtype) if normed is not None else DT_F32, _stream())
    return streams


def gated_act(out, gu, activation="silu"):
    """out[t, f] = act(gu[t, f]) * gu[t, inner + f]: ``gu`` [T, 2 * inner] holds a product's gate and up halves."""
    _check(out, "gated_act.out", gu.dtype, 2)
    _check(gu, "gated_act.gu", None, 2)
    n, inner = out.shape
    if gu.shape != (n, 2 * inner) or gu.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gated_act: the product holds two halves of the output's width")
    _gated_act(out.data_ptr(), out.stride(0), gu.data_ptr(), gu.stride(0), inner, GATED_ACTIVATIONS[activation], n,
               dtype_code(gu.dtype), _stream())
    return out


# ---- norms on a sublayer's output, query and key norms with rotary positions, gated linear recurrence ----

_norm_rotary_store = Function("unit", "mllm_unit_norm_rotary_store",
                              [P, L, I, I, I, I, I, I, P, L, P, P, I, F, I, I, P, P, P, P, I, I, P, P, I, I, I, P])
_gated_recurrence = Function("unit", "mllm_unit_gated_recurrence",
                             [P, L, P, L, P, L, P, L, P, P, P, F, P, L, P, P, P, I, I, I, I, I, I, P])
_add_normed_cast = Function("unit", "mllm_unit_add_normed_cast", [P, P, P, F, P, I, I, I, P])
_softcap = Function("unit", "mllm_unit_softcap", [P, F, L, P])
QK_NORMS = {None: 0, "none": 0, "whole": 1, "head": 2}


def norm_rotary_store(qkv, k_off, v_off, heads, kv_heads, dim, vdim, q_out, q_gain, k_gain, norm, eps, rot_dims, layout, inv_freq,
                      positions, token_item, block_table, page_size, k_pages, v_pages, writes=True):
    """Rows of the fp32 ``qkv`` hold the projected [q | k | v] (k from column ``k_off``, v from ``v_off``; ``v_off`` may
    equal ``k_off``: the values are then the keys as projected).  ``norm`` "whole": q and k are divided by the root mean
    square of their whole projection and multiplied by ``q_gain`` [heads * dim] / ``k_gain`` [kv_heads * dim]; "head":
    every head by its own, times a gain of ``dim`` entries shared by the heads; None: no norm.  Then the first
    ``rot_dims`` entries of every head turn by position * ``inv_freq`` [rot_dims / 2] (float64) in pairs that are
    neighbours (``layout`` "interleaved") or half the rotated entries apart ("half").  Queries go to ``q_out``
    [T, heads * dim]; keys and values to the token's place in the pages (unless ``writes`` is false: then only
    the queries are made and the pages may be None)."""
    _check(qkv, "norm_rotary_store.qkv", torch.float32, 2)
    _check(q_out, "norm_rotary_store.q_out", None, 2)
    _check(inv_freq, "norm_rotary_store.inv_freq", torch.float64, 1)
    n = qkv.shape[0]
    mode = QK_NORMS[norm]
    if q_out.shape != (n, heads * dim) or inv_freq.shape[0] < max(rot_dims // 2, 1) or heads * dim > qkv.shape[1]:
        raise KernelError("norm_rotary_store: sizes do not agree")
    gain_size = {0: None, 1: (heads * dim, kv_heads * dim), 2: (dim, dim)}[mode]
    if mode:
        _check(q_gain, "norm_rotary_store.q_gain", torch.float32, 1)
        if q_gain.shape[0] != gain_size[0]:
            raise KernelError(f"norm_rotary_store: the queries' gain has {q_gain.shape[0]} entries, not {gain_size[0]}")
    if writes:
        _check(k_pages, "norm_rotary_store.k_pages", q_out.dtype)
        _check(v_pages, "norm_rotary_store.v_pages", q_out.dtype)
        _check(block_table, "norm_rotary_store.block_table", torch.int32, 2)
        if mode:
            _check(k_gain, "norm_rotary_store.k_gain", torch.float32, 1)
            if k_gain.shape[0] != gain_size[1]:
                raise KernelError(f"norm_rotary_store: the keys' gain has {k_gain.shape[0]} entries, not {gain_size[1]}")
        if v_off + kv_heads * vdim > qkv.shape[1] or k_off + kv_heads * dim > qkv.shape[1]:
            raise KernelError("norm_rotary_store: keys or values lie outside the row")
        if (not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous()
                or k_pages.numel() % (page_size * kv_heads * dim) != 0 or v_pages.numel() % (page_size * kv_heads * vdim) != 0):
            raise KernelError("norm_rotary_store: the pages do not hold whole pages of these rows")
    _norm_rotary_store(qkv.data_ptr(), qkv.stride(0), int(k_off), int(v_off), heads, kv_heads, dim, vdim, q_out.data_ptr(),
                       q_out.stride(0), _ptr(q_gain) if mode else None, _ptr(k_gain) if mode and writes else None, mode, float(eps),
                       int(rot_dims), ROTARY_LAYOUTS[layout], inv_freq.data_ptr(), positions.data_ptr(), token_item.data_ptr(),
                       block_table.data_ptr() if writes else None, block_table.shape[1] if writes else 0, page_size,
                       k_pages.data_ptr() if writes else None, v_pages.data_ptr() if writes else None, int(bool(writes)), n,
                       dtype_code(q_out.dtype), _stream())
    return q_out


def gated_recurrence(out, u, y, gates, bias_r, bias_i, lam, decay_scale, state, item_slot, item_offset, item_count, block_width,
                     writes=True):
    """Per channel c: S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with a_t = exp(-decay_scale * r_t * softplus(lam[c])),
    r_t = sigmoid(gate_r + bias_r[c]), i_t = sigmoid(gate_i + bias_i[c]); out_t = S_t * gelu_tanh(y_t).  ``gates`` fp32
    [T, 2 * inner]: for every block of ``block_width`` channels its r gates, then its i gates.  ``state`` fp32
    [slots, inner] holds S per request and is moved on (unless ``writes`` is false)."""
    _check(out, "gated_recurrence.out", u.dtype, 2)
    _check(u, "gated_recurrence.u", None, 2)
    _check(y, "gated_recurrence.y", u.dtype, 2)
    _check(gates, "gated_recurrence.gates", torch.float32, 2)
    _check(state, "gated_recurrence.state", torch.float32, 2)
    for name, t in (("bias_r", bias_r), ("bias_i", bias_i), ("lam", lam)):
        _check(t, f"gated_recurrence.{name}", torch.float32, 1)
    for name, t in (("item_slot", item_slot), ("item_offset", item_offset), ("item_count", item_count)):
        _check(t, f"gated_recurrence.{name}", torch.int32, 1)
    n, inner = out.shape
    if (u.shape != (n, inner) or y.shape != (n, inner) or gates.shape != (n, 2 * inner) or state.shape[1] != inner
            or min(bias_r.shape[0], bias_i.shape[0], lam.shape[0]) < inner or inner % block_width != 0):
        raise KernelError("gated_recurrence: sizes do not agree")
    _gated_recurrence(out.data_ptr(), out.stride(0), u.data_ptr(), u.stride(0), y.data_ptr(), y.stride(0), gates.data_ptr(),
                      gates.stride(0), bias_r.data_ptr(), bias_i.data_ptr(), lam.data_ptr(), float(decay_scale), state.data_ptr(),
                      state.stride(0), item_slot.data_ptr(), item_offset.data_ptr(), item_count.data_ptr(), inner, int(block_width),
                      int(bool(writes)), item_count.shape[0], n, dtype_code(u.dtype), _stream())
    return out


def add_normed_cast(hidden, y=None, gain=None, eps=0.0, act=None):
    """hidden += y / sqrt(mean(y^2) + eps) * gain on the fp32 stream (``y`` None: nothing is added), and the rows as they
    then are, rounded, to ``act`` (None: not kept)."""
    _check(hidden, "add_normed_cast.hidden", torch.float32, 2)
    n, width = hidden.shape
    if not hidden.is_contiguous():
        raise KernelError("add_normed_cast: the stream must be contiguous")
    if y is not None:
        _check(y, "add_normed_cast.y", torch.float32, 2)
        _check(gain, "add_normed_cast.gain", torch.float32, 1)
        if y.shape[0] < n or y.shape[1] != width or not y.is_contiguous() or gain.shape[0] != width:
            raise KernelError("add_normed_cast: the sublayer's result or the gain has another shape")
    if act is not None:
        _check(act, "add_normed_cast.act", None, 2)
        if act.shape != (n, width) or not act.is_contiguous():
            raise KernelError("add_normed_cast: the rounded rows have another shape")
    _add_normed_cast(hidden.data_ptr(), _ptr(y), _ptr(gain), float(eps), _ptr(act), width, n,
                     dtype_code(act.dtype) if act is not None else DT_F32, _stream())
    return hidden


def softcap(x, cap):
    """x <- cap * tanh(x / cap), fp32, in place."""
    _check(x, "softcap.x", torch.float32)
    if not x.is_contiguous():
        raise KernelError("softcap: the rows must be contiguous")
    _softcap(x.data_ptr(), float(cap), x.numel(), _stream())
    return x

"""Lipulorn's kernels by themselves against the plain functions (``plain_lipulorn``, float64): the pass over
the residual streams, the gated attention within blocks of positions in its three forms, the norm of
query and key heads with the cache store, the delta rule with a decay per key channel over a sequence
cut in pieces, the attention over a latent within a window, the gated activation."""

import numpy as np
import pytest
import torch

import plain_lipulorn as plain

pytestmark = pytest.mark.gpu


def dev(values, dtype=torch.float32):
    return torch.tensor(np.asarray(values), dtype=dtype, device="cuda")


def scattered_table(lengths, page_size, seed=0):
    """A block table whose pages lie scattered over the pool: (table on the device, pages in the pool)."""
    blocks = [-(-n // page_size) for n in lengths]
    order = np.random.default_rng(seed).permutation(sum(blocks))
    table = np.zeros((len(lengths), max(blocks)), dtype=np.int32)
    at = 0
    for i, count in enumerate(blocks):
        table[i, :count] = order[at:at + count]
        at += count
    return dev(table, torch.int32), table, sum(blocks) + 1


# ---- the residual streams ---------------------------------------------------------------------------

@pytest.mark.parametrize("count, width, n", [(1, 24, 5), (3, 100, 33), (4, 768, 70), (8, 40, 2), (6, 64, 9), (13, 52, 7), (16, 20, 3)])
def test_streams_pass(count, width, n):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(count * 100 + width)
    streams = rng.normal(0, 1, (count, n, width))
    y, gain = rng.normal(0, 1, (n, width)), rng.uniform(0.5, 1.5, width)
    w = {"c.in": rng.normal(0, 1, count), "c.out": rng.normal(0, 1, count), "c.mix": rng.normal(0, 1, (count, count))}
    on_device = dev(streams.transpose(1, 0, 2)).contiguous()

    filled = torch.empty_like(on_device)
    ops.streams_fill(filled, dev(y))
    np.testing.assert_array_equal(filled.cpu().numpy(), np.repeat(dev(y).cpu().numpy()[:, None], count, axis=1))

    # the read-out alone, weighted and plain
    u = torch.empty((n, width), device="cuda")
    ops.streams_step(on_device, read=True, w_in=dev(w["c.in"]), u_out=u)
    np.testing.assert_allclose(u.cpu().numpy(), plain.hyper_read(streams, w, "c"), atol=1e-5)
    ops.streams_step(on_device, read=True, u_out=u)
    np.testing.assert_allclose(u.cpu().numpy(), streams.sum(axis=0), atol=1e-5)
    # the write alone: all streams from the old ones
    written = plain.hyper_write(streams, y, w, "c")
    alone = on_device.clone()
    ops.streams_step(alone, y=dev(y), mix=dev(w["c.mix"]), w_out=dev(w["c.out"]))
    np.testing.assert_allclose(alone.cpu().numpy().transpose(1, 0, 2), written, atol=1e-5)
    # write, read-out and norm in one pass
    for dtype, atol in ((torch.float32, 2e-5), (torch.bfloat16, 3e-2)):
        both = on_device.clone()
        normed = torch.empty((n, width), device="cuda", dtype=dtype)
        ops.streams_step(both, y=dev(y), mix=dev(w["c.mix"]), w_out=dev(w["c.out"]), read=True, w_in=dev(w["c.in"]), u_out=u,
                         normed=normed, gain=dev(gain), eps=1e-3)
        np.testing.assert_allclose(both.cpu().numpy().transpose(1, 0, 2), written, atol=1e-5)
        np.testing.assert_allclose(u.cpu().numpy(), plain.hyper_read(written, w, "c"), atol=1e-5)
        np.testing.assert_allclose(normed.float().cpu().numpy(), plain.rms_norm(plain.hyper_read(written, w, "c"), gain, 1e-3), atol=atol)


def test_gated_activation():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(3)
    for n, inner in ((5, 7), (64, 96)):
        gu = rng.normal(0, 2, (n, 2 * inner))
        out = torch.empty((n, inner), device="cuda")
        ops.gated_act(out, dev(gu), "silu")
        np.testing.assert_allclose(out.cpu().numpy(), plain.silu(gu[:, :inner]) * gu[:, inner:], atol=1e-5)


# ---- attention within blocks of positions --------------------------------------------------------------

def plain_block_attention(q, keys, values, positions, block, scale, gate, heads, kv_heads):
    """q [n, heads, dim] at ``positions`` of one sequence whose keys [len, kv_heads, dim] and values are given."""
    out = np.zeros((q.shape[0], heads, values.shape[2]))
    length = keys.shape[0]
    visible = plain.chunk_mask(length, block)[positions]
    for head in range(heads):
        g = head // (heads // kv_heads)
        weights = plain.softmax_rows((q[:, head] @ keys[:, g].T) * scale, visible)
        out[:, head] = (weights @ values[:, g]) * plain.sigmoid(gate[:, head:head + 1])
    return out


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, block", [(4, 2, 16, 24, 40), (6, 1, 64, 64, 7), (2, 2, 32, 32, 128),
                                                               (3, 3, 12, 20, 1), (8, 4, 128, 128, 33)])
def test_gated_attention_within_blocks(heads, kv_heads, dim, vdim, block):
    """A step with a prompt portion of one request, three tokens of a second and one token of a third, pages
    scattered: the tiled kernel and the kernel with one block per (token, head) against the formula; then single
    tokens alone (bfloat16) over split keys against the same formula."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(heads * 100 + block)
    page_size = 8
    lengths, new = [150, 83, 41], [110, 3, 1]
    table, table_host, n_pages = scattered_table(lengths, page_size, seed=block)
    keys = [rng.normal(0, 1, (n, kv_heads, dim)) for n in lengths]
    values = [rng.normal(0, 1, (n, kv_heads, vdim)) for n in lengths]
    k_pages, v_pages = np.zeros((n_pages, page_size, kv_heads, dim)), np.zeros((n_pages, page_size, kv_heads, vdim))
    for i, n in enumerate(lengths):
        for p in range(n):
            k_pages[table_host[i, p // page_size], p % page_size] = keys[i][p]
            v_pages[table_host[i, p // page_size], p % page_size] = values[i][p]
    positions = np.concatenate([np.arange(n - m, n) for n, m in zip(lengths, new)])
    token_item = np.concatenate([np.full(m, i) for i, m in enumerate(new)])
    total = sum(new)
    q, gate = rng.normal(0, 1, (total, heads, dim)), rng.normal(0, 2, (total, 16))
    expected, at = [], 0
    for i, m in enumerate(new):
        expected.append(plain_block_attention(q[at:at + m], keys[i], values[i], positions[at:at + m], block, 0.4, gate[at:at + m],
                                              heads, kv_heads))
        at += m
    expected = np.concatenate(expected).reshape(total, heads * vdim)
    for tiled in (False, True):
        if tiled and not ops.capped_attention_tiled_takes(dim, vdim, torch.float32):
            continue
        out = torch.full((total, heads * vdim), float("nan"), device="cuda")
        ops.capped_attention(out, dev(q.reshape(total, -1)), dev(k_pages), dev(v_pages), table, dev(positions, torch.int32),
                             dev(token_item, torch.int32), heads, kv_heads, dim, vdim, page_size, 0.4, 0.0, 0, tiled=tiled,
                             chunk=block, gate=dev(gate))
        np.testing.assert_allclose(out.cpu().numpy(), expected, atol=2e-5, err_msg=f"tiled {tiled}")
    if dim != vdim or dim not in ops.SPLIT_ATTENTION_HEAD_SIZES:
        return
    # single tokens: the last token of each request, and one at a block's first position
    rows = [new[0] - 1, new[0] + new[1] - 1, total - 1]
    single_q = q[rows]
    single_positions = positions[rows].copy()
    single_positions[0] = (lengths[0] - 1) // block * block        # the first position of a block sees itself alone
    want = np.concatenate([plain_block_attention(single_q[i:i + 1], keys[i], values[i], single_positions[i:i + 1], block, 0.4,
                                                 gate[rows][i:i + 1], heads, kv_heads) for i in range(3)]).reshape(3, heads * vdim)
    span, reach = 64, table.shape[1] * page_size
    spans = -(-reach // span)
    scratch = (torch.empty(3 * heads * spans * dim, device="cuda"), torch.empty(3 * heads * spans * 2, device="cuda"),
               torch.zeros(3 * heads, dtype=torch.int32, device="cuda"))
    got = torch.full((3, heads * vdim), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.split_attention(got, dev(single_q.reshape(3, -1)).bfloat16(), dev(k_pages).bfloat16(), dev(v_pages).bfloat16(), table,
                        dev(single_positions, torch.int32), dev([0, 1, 2], torch.int32), heads, kv_heads, dim, page_size, 0.4, 0, span,
                        spans, *scratch, block=block, gate=dev(gate[rows]))
    np.testing.assert_allclose(got.float().cpu().numpy(), want, atol=5e-2)
    assert int(scratch[2].abs().max()) == 0
    if block == 1:
        # a block of one position: every token sees itself alone, so its result is its own value, gated
        own = np.stack([values[i][single_positions[i]] for i in range(3)])
        np.testing.assert_allclose(want.reshape(3, heads, vdim),
                                   own[:, [h // (heads // kv_heads) for h in range(heads)]] * plain.sigmoid(gate[rows][:, :heads, None]),
                                   atol=1e-12)


def test_head_norms_and_cache_store():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(7)
    heads, kv_heads, dim, vdim, page_size, eps = 3, 1, 10, 6, 4, 1e-3
    positions = np.array([0, 1, 2, 3, 4, 61, 62])
    token_item = np.array([0, 0, 0, 0, 0, 1, 1])
    table = np.zeros((2, 16), dtype=np.int32)
    table[0, :2] = [3, 1]
    table[1, 15] = 2
    width = (heads + kv_heads) * dim + kv_heads * vdim
    qkv = rng.normal(0, 2, (7, width))
    for skip in (False, True):
        on_device = dev(qkv)
        k_pages, v_pages = torch.zeros((5, page_size, kv_heads, dim), device="cuda"), torch.zeros((5, page_size, kv_heads, vdim), device="cuda")
        ops.head_norm_store(on_device, heads * dim, (heads + kv_heads) * dim, heads, kv_heads, dim, vdim, -1.0 if skip else eps,
                            dev(positions, torch.int32), dev(token_item, torch.int32), dev(table, torch.int32), page_size, k_pages, v_pages)
        normed = qkv.copy()
        if not skip:
            both = qkv[:, :(heads + kv_heads) * dim].reshape(7, heads + kv_heads, dim)
            normed[:, :(heads + kv_heads) * dim] = plain.rms_norm(both, None, eps).reshape(7, -1)
        np.testing.assert_allclose(on_device.cpu().numpy(), normed, atol=1e-5)
        for t in range(7):
            page = table[token_item[t], positions[t] // page_size]
            np.testing.assert_allclose(k_pages[page, positions[t] % page_size].cpu().numpy().reshape(-1),
                                       normed[t, heads * dim:(heads + kv_heads) * dim], atol=1e-5)
            np.testing.assert_allclose(v_pages[page, positions[t] % page_size].cpu().numpy().reshape(-1),
                                       normed[t, (heads + kv_heads) * dim:], atol=1e-5)
        assert float(k_pages[0].abs().max()) == 0.0 and float(k_pages[4].abs().max()) == 0.0


# ---- the delta rule with a decay per key channel -----------------------------------------------------------

@pytest.mark.parametrize("heads, qk_heads, dim, vdim", [(2, 1, 8, 8), (3, 3, 20, 12), (4, 2, 64, 64), (1, 1, 128, 40), (60, 4, 12, 16),
                                                        (2, 1, 256, 24), (1, 1, 520, 8)])
def test_channel_decay_recurrence_carries_its_state(heads, qk_heads, dim, vdim):
    """A sequence cut in six (down to one token) against the token-by-token formulas; the decay multiplies
    the rows of the state before the old state is read."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(dim + heads)
    n = 100
    q, k = rng.normal(0, 1, (n, qk_heads * dim)), rng.normal(0, 1, (n, qk_heads * dim))
    v = rng.normal(0, 1, (n, heads * vdim))
    gate_a, gate_b = rng.normal(0, 2, (n, heads * dim)), rng.normal(0, 3, (n, heads))
    log_rate, bias = rng.normal(-1, 1, heads), rng.normal(0, 1, heads * dim)
    expected = np.zeros((n, heads, vdim))
    for head in range(heads):
        g = head // (heads // qk_heads)
        S = np.zeros((dim, vdim))
        for t in range(n):
            qt, kt = q[t, g * dim:(g + 1) * dim], k[t, g * dim:(g + 1) * dim]
            vt = v[t, head * vdim:(head + 1) * vdim]
            a = np.exp(-np.exp(log_rate[head]) * plain.softplus(gate_a[t, head * dim:(head + 1) * dim] + bias[head * dim:(head + 1) * dim]))
            qt = qt / np.sqrt((qt * qt).sum() + 1e-6) * 0.5
            kt = kt / np.sqrt((kt * kt).sum() + 1e-6)
            S = a[:, None] * S
            S = S + np.outer(kt, plain.sigmoid(gate_b[t, head]) * (vt - S.T @ kt))
            expected[t, head] = S.T @ qt
    state = torch.zeros((2, heads * dim * vdim), dtype=torch.float32, device="cuda")
    out = torch.empty((n, heads * vdim), dtype=torch.float32, device="cuda")
    for first, count in ((0, 1), (1, 9), (10, 3), (13, 10), (23, 32), (55, 45)):
        rows = slice(first, first + count)
        ops.linear_recurrence(out[rows], dev(q[rows]), dev(k[rows]), dev(v[rows]), dev(gate_a[rows]), dev(gate_b[rows]), dev(log_rate),
                              dev(bias), state, dev([0, 1], torch.int32), dev([0, 0], torch.int32), dev([0, count], torch.int32), heads,
                              qk_heads, dim, vdim, True, unit_norm=True, q_scale=0.5, channel_decay=True)
    np.testing.assert_allclose(out.cpu().numpy(), expected.reshape(n, heads * vdim), rtol=5e-5,
                               atol=5e-6 * max(4.0, float(np.abs(expected).max())))
    assert float(state[0].abs().max()) == 0.0


# ---- attention over a latent within a window ------------------------------------------------------------------

@pytest.mark.parametrize("heads, rank, rot, window", [(3, 16, 8, 5), (4, 64, 32, 70), (2, 24, 4, 1), (16, 128, 64, 33)])
def test_latent_attention_within_a_window(heads, rank, rot, window):
    """Prompt portions and single tokens over scattered pages: every form the sizes allow against the formula
    (score = effective query . cached row, the weighted sum over the row's first ``rank`` entries)."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(rank + window)
    page_size, row = 8, rank + rot
    for lengths, new in (([150, 83, 41], [110, 3, 1]), ([150, 83, 41], [1, 1, 1])):
        table, table_host, n_pages = scattered_table(lengths, page_size, seed=window)
        rows = [rng.normal(0, 1, (n, row)) for n in lengths]
        pages = np.zeros((n_pages, page_size, 1, row))
        for i, n in enumerate(lengths):
            for p in range(n):
                pages[table_host[i, p // page_size], p % page_size, 0] = rows[i][p]
        starts = [n - m for n, m in zip(lengths, new)]
        positions = np.concatenate([np.arange(s, s + m) for s, m in zip(starts, new)])
        token_item = np.concatenate([np.full(m, i) for i, m in enumerate(new)])
        total = sum(new)
        q_eff = rng.normal(0, 0.5, (total, heads, row))
        expected, at = np.zeros((total, heads, rank)), 0
        for i, m in enumerate(new):
            visible = plain.window_mask(lengths[i], window)[positions[at:at + m]]
            for head in range(heads):
                weights = plain.softmax_rows((q_eff[at:at + m, head] @ rows[i].T) * 0.3, visible)
                expected[at:at + m, head] = weights @ rows[i][:, :rank]
            at += m
        expected = expected.reshape(total, heads * rank)
        common = (dev(q_eff.reshape(total, -1)), None, table, dev(positions, torch.int32), dev(token_item, torch.int32), heads, rank, rot,
                  page_size, 0.3)
        out = torch.full((total, heads * rank), float("nan"), device="cuda")
        ops.latent_attention_plain(out, common[0], dev(pages), *common[2:], window)
        np.testing.assert_allclose(out.cpu().numpy(), expected, atol=2e-5)
        pages_16 = dev(pages).bfloat16()
        if not ops.latent_attention_tiled_takes(pages_16, rank, rot):
            continue
        # the tiled forms read bfloat16 rows: compare with the plain kernel on the same rounded rows
        want = torch.empty_like(out)
        ops.latent_attention_plain(want, common[0], pages_16.float(), *common[2:], window)
        got = torch.full_like(out, float("nan"))
        if max(new) > 1:
            offsets = [sum(new[:i]) for i in range(len(new))]
            tiles, _, _ = ops.attention_tiles(offsets, new, starts, split=False)
            ops.latent_attention_tiled(got, common[0], pages_16, *common[2:], tiles=dev(tiles, torch.int32), n_tiles=len(tiles), window=window)
        else:
            parts = 4
            scratch = (torch.empty(total * heads * parts * rank, device="cuda"), torch.empty(total * heads * parts * 2, device="cuda"))
            ops.latent_attention_tiled(got, common[0], pages_16, *common[2:], parts=parts, scratch=scratch, window=window)
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)

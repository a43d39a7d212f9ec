"""Deluvik on the device against the plain implementation (``plain_deluvik``, float64).

Every test makes its own small configuration and random weights.  32-bit runs must agree within 1e-4 at every
token; bfloat16 runs within 4 % of the logits' spread in the root mean square.  The schedules cut the same requests
in different ways: a request's logits must not depend on the cut, on the rest of the batch, or on which pages and
slots it got."""

import numpy as np
import pytest
import torch

import deluvik_helpers as dv
import plain_deluvik as plain
from engine_helpers import (F32_ATOL, random_tokens, run_schedule, schedule_mixed, schedule_portions, schedule_tail_one_by_one,
                            schedule_whole)

pytestmark = pytest.mark.gpu


def engine_for(folder, dtype="float32", **options):
    from mini_llm_b200.engine import Engine
    options.setdefault("page_size", 8)
    options.setdefault("max_requests", 4)
    options.setdefault("cache_tokens", 1024)
    return Engine(folder, dtype=dtype, **options)


def check(engine, folder, requests, steps, atol=F32_ATOL):
    got = run_schedule(engine, requests, steps)
    for name, tokens in requests.items():
        expected = dv.plain_logits(folder, tokens)
        worst = np.abs(got[name] - expected).max(axis=1)
        assert worst.max() <= atol, f"request {name}: first wrong token {int(np.argmax(worst > atol))} of {len(tokens)}, off by {worst.max():.2e}"
    engine.cache.check()


def dev(values, dtype=torch.float32):
    return torch.tensor(np.asarray(values), dtype=dtype, device="cuda")


# ---- each mechanism alone ----------------------------------------------------------------------

@pytest.mark.parametrize("layer", [
    dv.attention(mlp=None),
    dv.attention(mlp=None, heads=6, kv_heads=1, dim=8, rot_dims=0, scaling=None, softcap=None),
    dv.attention(mlp=None, heads=2, kv_heads=2, dim=24, rot_dims=24, softcap=0.8, scale=2.0),
    dv.attention_2(mlp=None),
    dv.attention_2(mlp=None, heads=3, kv_heads=1, dim=8, vdim=40, taps=1, rot_dims=4, scaling=dv.BANDS),
    dv.attention_2(mlp=None, heads=2, kv_heads=2, dim=40, vdim=8, taps=5, rot_dims=40, scale=1.5),
    dv.parallel(right_scale=0.0, mlp=None),
    dv.parallel(right_scale=0.0, mlp=None, heads=6, kv_heads=1, dim=8, vdim=40, window=1, rot_dims=8),
    dv.parallel(right_scale=0.0, mlp=None, heads=2, kv_heads=2, dim=24, vdim=24, window=100, rot_dims=0),
    dv.parallel(left_scale=0.0, mlp=None),
    dv.parallel(left_scale=0.0, mlp=None, inner=33, blocks=1, taps=1),
    dv.parallel(left_scale=0.0, mlp=None, inner=70, blocks=35, taps=2),
    dv.parallel(),
    dv.attention(mlp=dv.dense(56)),
    dv.attention(mlp=dv.moe(experts=7, top=1, ff=12, shared=None)), dv.attention(mlp=dv.moe(experts=3, top=3, ff=40, shared=8)),
], ids=["attention", "attention_one_kv_head_no_rotation_no_cap", "attention_hard_cap_all_rotated", "convolved",
        "convolved_one_tap_scaled_frequencies", "convolved_five_taps_wide_keys", "window", "window_of_one", "window_never_full",
        "unit", "unit_one_block_one_tap", "unit_blocks_of_two", "both_sides", "dense_feed_forward", "experts_top_one_no_shared",
        "experts_all_chosen"])
def test_one_layer_of_each_kind(tmp_path, layer):
    folder = dv.make_model(str(tmp_path / "m"), dv.config([layer]), seed=3, matrix_scale=3.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(1, 37, 211), "b": random_tokens(2, 1, 211), "c": random_tokens(3, 2, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_portions(requests))


def test_no_cap_on_the_logits(tmp_path):
    folder = dv.make_model(str(tmp_path / "m"), dv.config([dv.attention()], logit_softcap=None), seed=4, matrix_scale=3.0)
    requests = {"a": random_tokens(1, 20, 211)}
    check(engine_for(folder), folder, requests, schedule_whole(requests))


def test_residual_stream_after_every_layer(tmp_path):
    from mini_llm_b200.engine import StepEntry
    folder = dv.make_model(str(tmp_path / "m"), dv.full_stack(), seed=5, matrix_scale=2.0)
    engine = engine_for(folder)
    tokens = random_tokens(4, 29, 211)
    _, streams = dv.plain_logits(folder, tokens, keep_layers=True)
    slot = engine.open_request()
    engine.step([StepEntry(slot, tokens, [28])], dump_hidden=True)
    assert len(engine.hidden_dump) == len(streams) + 1
    for index, expected in enumerate(streams):
        np.testing.assert_allclose(engine.hidden_dump[index + 1].cpu().numpy(), expected, rtol=0,
                                   atol=1e-4 * np.abs(expected).max(), err_msg=f"after layer {index}")
    engine.close_request(slot)


# ---- the same tokens, cut differently -----------------------------------------------------------

def test_prompt_against_token_by_token_and_portions(tmp_path):
    folder = dv.make_model(str(tmp_path / "m"), dv.full_stack(), seed=7, matrix_scale=2.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(11, 45, 211), "b": random_tokens(12, 7, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=45))        # every token alone, from the first
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=5))
    check(engine, folder, requests, schedule_portions(requests))
    check(engine, folder, requests, schedule_portions(requests, sizes=(2, 2, 3, 2, 17)))
    assert engine.step_kinds["replayed"] > 0          # steps of one shape were replayed from a captured graph


def test_mixed_batches_and_reuse_of_pages_and_slots(tmp_path):
    """Six requests through three slots and a page pool that holds less than their sum: pages and slots are given
    back and used again (and poisoned in between), portions run beside single tokens; every request must come out
    as it does alone.  The windowed layers give pages back while their requests still run."""
    folder = dv.make_model(str(tmp_path / "m"), dv.full_stack(), seed=9, matrix_scale=2.0)
    lengths = {"a": 61, "b": 9, "c": 33, "d": 2, "e": 40, "f": 18}
    requests = {name: random_tokens(20 + i, n, 211) for i, (name, n) in enumerate(lengths.items())}
    prompts = {"a": 40, "b": 9, "c": 20, "d": 1, "e": 40, "f": 3}
    engine = engine_for(folder, max_requests=3, cache_tokens=160, debug_poison=True)
    check(engine, folder, requests, schedule_mixed(requests, prompts, max_live=3))
    check(engine, folder, requests, schedule_mixed(requests, prompts, max_live=2, portion_sizes=(2, 11, 3)))
    assert not any(engine.cache.pages_in_use()) and engine.cache.free_slots == 3
    assert engine.cache.freed_by_window > 0


# ---- single keys that decide: far away, and at a window's edge ----------------------------------

def _marked(t, prefix, norm_size):
    """Only tokens 5 and 9 have anything in the first eight channels of the embedding; entry 7 of the one key head
    (not rotated) reads them, and so does entry 7 of query head 0, with the other sign for token 9: token 9's query
    finds token 5's key, whose value stands out."""
    t["embed"][:, :8] = 0.0
    t["embed"][5, :8] = 2.0
    t["embed"][9, :8] = -2.0
    t[f"{prefix}.k"][7] = 0.0
    t[f"{prefix}.k"][7, :8] = 4.0
    t[f"{prefix}.q"][7] = 0.0
    t[f"{prefix}.q"][7, :8] = -4.0
    t[f"{prefix}.q.norm"][:norm_size] = 1.0
    t[f"{prefix}.k.norm"][:norm_size] = 1.0


def _marked_tokens(n, key_at):
    rng = np.random.default_rng(0)
    base = [int(t) for t in rng.integers(10, 64, n)]
    base[-1] = 9
    with_key = list(base)
    with_key[key_at] = 5
    return with_key, base


@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_a_far_key_decides(tmp_path, kind):
    """The logits of the last token hang on one early key among hundreds (behind many page borders), in a prompt, in
    portions and when the last tokens are decoded alone.  The same key one place off (a wrong rotation, a key stored
    in a neighbour's place) would not match; neither would a key whose norm or sink were left out."""
    if kind == "attention":
        layer = dv.attention(heads=2, kv_heads=1, dim=8, rot_dims=4, base=50.0, scaling=dv.BANDS, scale=2.0, softcap=40.0, mlp=None)
    else:
        layer = dv.attention_2(heads=2, kv_heads=1, dim=8, vdim=8, taps=1, rot_dims=4, base=50.0, scale=2.0, mlp=None)
    raw = dv.config([layer], vocab=64, width=32)

    def bend(t):
        _marked(t, "l0.mix", 16)
        t["l0.mix.sink"][:] = [3.0, -1.0]
        if kind == "attention_2":
            for name in ("q", "k", "v"):
                t[f"l0.mix.{name}.conv"][:] = 1.0
    folder = dv.make_model(str(tmp_path / "m"), raw, seed=13, bend=bend, matrix_scale=2.0)
    with_key, without = _marked_tokens(300, 3)
    assert np.abs(dv.plain_logits(folder, with_key)[-1] - dv.plain_logits(folder, without)[-1]).max() > 0.1
    engine = engine_for(folder)
    for tokens in (with_key, without):
        requests = {"r": tokens}
        check(engine, folder, requests, schedule_whole(requests))
        check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=3))
        check(engine, folder, requests, schedule_portions(requests, sizes=(8, 7, 9, 64, 2)))


@pytest.mark.parametrize("window", [13, 16, 40])
def test_keys_just_inside_and_just_outside_the_window(tmp_path, window):
    """The marked key stands ``window - 1`` places before the last token (the oldest key it sees) or ``window`` places
    before it (the newest it does not): in the first case the logits hang on it, in the second they do not notice it.
    Windows shorter than, equal to and longer than two pages, in a prompt, in portions and decoded alone."""
    layer = dv.parallel(heads=2, kv_heads=1, dim=8, vdim=8, window=window, rot_dims=4, base=50.0, scale=2.0, right_scale=0.0, mlp=None)
    raw = dv.config([layer], vocab=64, width=32)
    folder = dv.make_model(str(tmp_path / "m"), raw, seed=15, bend=lambda t: _marked(t, "l0.mix.left", 8), matrix_scale=2.0)
    n = 90
    inside, without = _marked_tokens(n, n - window)
    outside, _ = _marked_tokens(n, n - 1 - window)
    assert np.abs(dv.plain_logits(folder, inside)[-1] - dv.plain_logits(folder, without)[-1]).max() > 0.1
    np.testing.assert_allclose(dv.plain_logits(folder, outside)[-1], dv.plain_logits(folder, without)[-1], atol=1e-12)
    engine = engine_for(folder, cache_tokens=256)
    for tokens in (inside, outside):
        requests = {"r": tokens}
        check(engine, folder, requests, schedule_whole(requests))
        check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=window + 3))
        check(engine, folder, requests, schedule_portions(requests, sizes=(8, 7, 9, 33, 2)))
    assert engine.cache.freed_by_window > 0


def test_a_layer_reads_the_keys_and_values_another_stored(tmp_path):
    """Two readers of one layer's keys and values, with portions cut so that readers meet keys stored in earlier
    steps and in their own; the owner's taps and the readers' own taps carry over the cuts."""
    raw = dv.config([dv.attention_2(taps=4, mlp=None), dv.attention_2(kv_from=0, taps=2, mlp=None), dv.parallel(mlp=None),
                     dv.attention_2(kv_from=0, taps=4, mlp=dv.dense(24))])
    folder = dv.make_model(str(tmp_path / "m"), raw, seed=21, matrix_scale=3.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(71, 50, 211), "b": random_tokens(72, 21, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_mixed(requests, {"a": 30, "b": 11}, max_live=2, portion_sizes=(2, 5, 3)))
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=12))


def test_long_decoding_with_slow_and_fast_decays(tmp_path):
    """The recurrent unit with rates bent so that some channels nearly keep their state (a close to 1, where
    1 - a^2 loses its digits if it is taken carelessly) and others forget at once, and gates at both ends: what an
    early token wrote is still there two hundred tokens later.  Token by token against the whole prompt."""
    raw = dv.config([dv.parallel(left_scale=0.0, inner=32, blocks=2, taps=3, mlp=None), dv.parallel(window=7, mlp=None)], width=32, vocab=97)

    def bend(t):
        t["l0.mix.right.lam"][:] = np.linspace(-12.0, 3.0, 32)
        t["l0.mix.right.ra.b"] *= 100.0
        t["l0.mix.right.ri.b"] *= 100.0
    folder = dv.make_model(str(tmp_path / "m"), raw, seed=17, bend=bend, matrix_scale=2.0)
    engine = engine_for(folder)
    requests = {"long": random_tokens(31, 221, 97)}
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=220))
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_portions(requests, sizes=(16, 17, 15, 2, 33, 100)))


# ---- bfloat16 ------------------------------------------------------------------------------------

def all_experts(raw):
    """The same stack with every expert chosen for every token: no choice hangs on a near tie, which rounding to
    bfloat16 may turn (the 32-bit tests cover the choice itself)."""
    for layer in raw["layers"]:
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


def check_rounding(engine, folder, requests, steps, share=0.04):
    got = run_schedule(engine, requests, steps)
    for name, tokens in requests.items():
        expected = dv.plain_logits(folder, tokens)
        ratio = float(np.sqrt(((got[name] - expected) ** 2).mean()) / expected.std())
        assert ratio <= share, f"request {name}: root mean square of the difference is {ratio:.3f} of the logits' spread"
    engine.cache.check()


def test_bfloat16_follows_within_its_rounding(tmp_path):
    folder = dv.make_model(str(tmp_path / "m"), all_experts(dv.full_stack(width=128)), seed=19, bfloat16_values=True)
    engine = engine_for(folder, dtype="bfloat16")
    requests = {"a": random_tokens(41, 140, 211), "b": random_tokens(42, 12, 211), "c": random_tokens(43, 70, 211)}
    check_rounding(engine, folder, requests, schedule_whole(requests))
    check_rounding(engine, folder, requests, schedule_mixed(requests, {"a": 100, "b": 6, "c": 64}, max_live=3))
    check_rounding(engine, folder, requests, schedule_tail_one_by_one(requests, tail=10))
    chosen = {kernel for key, kernel in engine.kernels.choices.items() if key[0] in ("capped_attention", "linear")}
    assert {"capped_attention_tiled", "split_attention", "gemm_tcgen05"} <= chosen


def test_bfloat16_with_sizes_no_fast_kernel_takes(tmp_path):
    """A width that is no multiple of 8, key sizes of 6 and 10, 35 recurrent channels: every product and the
    attention fall back to kernels that take any size, in bfloat16 too."""
    raw = dv.config([dv.attention_2(heads=3, kv_heads=1, dim=10, vdim=14, rot_dims=6),
                     dv.parallel(heads=2, kv_heads=2, dim=6, vdim=10, rot_dims=2, inner=35, blocks=5, mlp=dv.moe(experts=3, top=2, ff=9, shared=5)),
                     dv.attention(heads=2, kv_heads=1, dim=10, rot_dims=10, mlp=dv.dense(27))], width=100, vocab=203)
    folder = dv.make_model(str(tmp_path / "m"), all_experts(raw), seed=29, bfloat16_values=True)
    requests = {"a": random_tokens(61, 150, 203), "b": random_tokens(62, 3, 203), "c": random_tokens(63, 40, 203)}
    engine = engine_for(folder, dtype="bfloat16")
    check_rounding(engine, folder, requests, schedule_whole(requests))
    check_rounding(engine, folder, requests, schedule_mixed(requests, {"a": 130, "b": 2, "c": 33}, max_live=3))
    chosen = {kernel for key, kernel in engine.kernels.choices.items() if key[0] in ("capped_attention", "linear")}
    assert chosen == {"capped_attention_plain", "linear_plain"}
    check(engine_for(folder), folder, requests, schedule_portions(requests))


def test_greedy_generation_through_the_scheduler(tmp_path):
    from mini_llm_b200.generate import generate
    folder = dv.make_model(str(tmp_path / "m"), dv.full_stack(), seed=23, matrix_scale=3.0)
    model_config, tensors = plain.load_model(folder)
    prompts = [random_tokens(50 + i, n, 211) for i, n in enumerate((3, 19, 1, 30, 8))]
    got = generate(folder, prompts, max_new_tokens=12, temperature=0.0, dtype="float32", page_size=8, max_sessions=3,
                   cache_tokens=256, max_prefill_chunk=7)
    for prompt, generated in zip(prompts, got):
        tokens = list(prompt)
        for index, token in enumerate(generated):
            logits = plain.forward(model_config, tensors, tokens)[-1]
            ordered = np.sort(logits)
            if ordered[-1] - ordered[-2] < 1e-3:
                break                                   # a near tie: either token is right, and the paths part here
            assert token == int(np.argmax(logits)), f"generated token {index}"
            tokens.append(token)


# ---- the mechanisms' kernels by themselves ------------------------------------------------------

def _attention_case(rng, n_tokens, heads, kv_heads, dim, vdim, page_size, dtype, start=0):
    """One request of ``n_tokens`` cached positions; the step's queries are its last ``n_tokens - start``."""
    n_pages = -(-n_tokens // page_size)
    order = rng.permutation(n_pages + 3)[:n_pages]              # the request's pages lie scattered
    k = rng.normal(0, 1, (n_tokens, kv_heads, dim))
    v = rng.normal(0, 1, (n_tokens, kv_heads, vdim))
    q = rng.normal(0, 1, (n_tokens, heads, dim))
    if dtype == torch.bfloat16:
        k, v, q = (dv.to_bfloat16_values(x).astype(np.float64) for x in (k, v, q))
    k_pages = torch.zeros((n_pages + 3, page_size, kv_heads, dim), dtype=dtype, device="cuda")
    v_pages = torch.zeros((n_pages + 3, page_size, kv_heads, vdim), dtype=dtype, device="cuda")
    for p in range(n_tokens):
        k_pages[order[p // page_size], p % page_size] = dev(k[p], dtype)
        v_pages[order[p // page_size], p % page_size] = dev(v[p], dtype)
    table = dev(order[None, :], torch.int32)
    positions = dev(np.arange(start, n_tokens), torch.int32)
    return q, k, v, k_pages, v_pages, table, positions, torch.zeros(n_tokens - start, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, cap", [(4, 2, 16, 24, 0, 0.0), (3, 1, 8, 8, 9, 2.0), (2, 2, 64, 128, 40, 0.0)])
def test_attention_kernels_with_a_sink(heads, kv_heads, dim, vdim, window, cap):
    """Tiles and the plain form against the formula, with sinks from far below to far above the scores."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(dim)
    n = 77
    q, k, v, k_pages, v_pages, table, positions, items = _attention_case(rng, n, heads, kv_heads, dim, vdim, 8, torch.float32)
    sink = np.linspace(-20.0, 12.0, heads)
    expected = plain.attend(q, k, v, 0.4, cap or None, window or None, sink).reshape(n, heads * vdim)
    for tiled in (False, True):
        out = torch.empty((n, heads * vdim), dtype=torch.float32, device="cuda")
        ops.capped_attention(out, dev(q.reshape(n, -1)), k_pages, v_pages, table, positions, items, heads, kv_heads, dim, vdim, 8, 0.4,
                             cap, window, tiled=tiled, sink=dev(sink))
        np.testing.assert_allclose(out.cpu().numpy(), expected, atol=2e-5, err_msg=f"tiled={tiled}")
    assert np.abs(expected - plain.attend(q, k, v, 0.4, cap or None, window or None, None).reshape(n, -1)).max() > 0.05


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, cap, dtype", [
    (4, 2, 64, 64, 0, 0.0, torch.float32), (6, 1, 32, 128, 50, 3.0, torch.float32), (4, 4, 128, 64, 200, 0.0, torch.float32),
    (6, 2, 64, 64, 0, 20.0, torch.bfloat16)])
def test_attention_in_register_tiles(heads, kv_heads, dim, vdim, window, cap, dtype):
    """Steps with thousands of (token, head) rows take the kernel with register tiles: two requests whose border
    falls inside a tile (the second one's portion starts at position 40 of its sequence), against the formula."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(dim + vdim)
    page, n0, n1, start1 = 16, 333, 360, 40
    cases = [_attention_case(rng, n0, heads, kv_heads, dim, vdim, page, dtype), _attention_case(rng, n1, heads, kv_heads, dim, vdim, page, dtype, start=start1)]
    # one pool for both requests: the second one's pages lie behind the first one's
    shift = cases[0][3].shape[0]
    k_pages, v_pages = torch.cat([cases[0][3], cases[1][3]]), torch.cat([cases[0][4], cases[1][4]])
    width = max(cases[0][5].shape[1], cases[1][5].shape[1])
    table = torch.zeros((2, width), dtype=torch.int32, device="cuda")
    table[0, :cases[0][5].shape[1]] = cases[0][5][0]
    table[1, :cases[1][5].shape[1]] = cases[1][5][0] + shift
    positions = torch.cat([cases[0][6], cases[1][6]])
    items = torch.cat([torch.zeros(n0), torch.ones(n1 - start1)]).to(torch.int32).cuda()
    q = np.concatenate([cases[0][0], cases[1][0][start1:]])
    n = q.shape[0]
    assert n * heads >= 2048
    sink = np.linspace(-3.0, 4.0, heads)
    expected = np.concatenate([plain.attend(cases[0][0], cases[0][1], cases[0][2], 0.3, cap or None, window or None, sink),
                               plain.attend(cases[1][0][start1:], cases[1][1], cases[1][2], 0.3, cap or None, window or None, sink,
                                            first_position=start1)]).reshape(n, heads * vdim)
    out = torch.empty((n, heads * vdim), dtype=dtype, device="cuda")
    ops.capped_attention(out, dev(q.reshape(n, -1), dtype), k_pages, v_pages, table, positions, items, heads, kv_heads, dim, vdim, page, 0.3,
                         cap, window, tiled=True, sink=dev(sink))
    np.testing.assert_allclose(out.float().cpu().numpy(), expected, atol=2e-5 if dtype == torch.float32 else 0.02)
    # the same rows through the tiles of few rows (a gate of +40 everywhere opens every head fully and keeps them there)
    gate = torch.full((n, heads), 40.0, device="cuda")
    again = torch.empty_like(out)
    ops.capped_attention(again, dev(q.reshape(n, -1), dtype), k_pages, v_pages, table, positions, items, heads, kv_heads, dim, vdim, page,
                         0.3, cap, window, tiled=True, sink=dev(sink), gate=gate)
    np.testing.assert_allclose(again.float().cpu().numpy(), expected, atol=2e-5 if dtype == torch.float32 else 0.02)


def test_split_attention_with_a_sink():
    """Single tokens over split keys (bfloat16): the sink joins the merge of the chunks."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(5)
    heads, kv_heads, dim, n = 4, 2, 64, 300
    q, k, v, k_pages, v_pages, table, _, _ = _attention_case(rng, n, heads, kv_heads, dim, dim, 16, torch.bfloat16)
    sink = np.array([-30.0, 0.5, 4.0, 25.0])
    for last in (1, 17, 300):
        expected = plain.attend(q[last - 1:last], k[:last], v[:last], 0.2, 3.0, None, sink, first_position=last - 1).reshape(1, -1)
        chunk, max_chunks = 64, -(-table.shape[1] * 16 // 64)
        out = torch.empty((1, heads * dim), dtype=torch.bfloat16, device="cuda")
        acc = torch.empty(heads * max_chunks * dim, dtype=torch.float32, device="cuda")
        ml = torch.empty(heads * max_chunks * 2, dtype=torch.float32, device="cuda")
        counters = torch.zeros(heads, dtype=torch.int32, device="cuda")
        ops.split_attention(out, dev(q[last - 1].reshape(1, -1), torch.bfloat16), k_pages, v_pages, table, dev([last - 1], torch.int32),
                            dev([0], torch.int32), heads, kv_heads, dim, 16, 0.2, 0, chunk, max_chunks, acc, ml, counters, cap=3.0,
                            sink=dev(sink))
        np.testing.assert_allclose(out.float().cpu().numpy(), expected, atol=0.02, err_msg=f"{last} keys")
        assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("norm, layout, values_are_keys, rot_dims", [("whole", "half", True, 12), ("whole", "half", False, 16),
                                                                     ("head", "interleaved", False, 6), (None, "interleaved", False, 0)])
def test_norm_rotation_and_store_in_one_kernel(norm, layout, values_are_keys, rot_dims):
    """Against the formulas, for tokens of two requests on both sides of a page border and at position 900."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(rot_dims)
    heads, kv_heads, dim, page_size = 4, 2, 16, 8
    vdim = dim if values_are_keys else 24
    positions = [6, 7, 8, 9, 900, 0]
    items = [0, 0, 0, 0, 1, 2]
    n = len(positions)
    q_width, k_width, v_width = heads * dim, kv_heads * dim, kv_heads * vdim
    row = rng.normal(0, 1, (n, q_width + k_width + (0 if values_are_keys else v_width) + 5))
    gains = {"whole": (rng.uniform(0.5, 1.5, q_width), rng.uniform(0.5, 1.5, k_width)),
             "head": (rng.uniform(0.5, 1.5, dim), rng.uniform(0.5, 1.5, dim)), None: (None, None)}[norm]
    rot = {"base": 70.0, "dims": rot_dims}
    q, k = row[:, :q_width], row[:, q_width:q_width + k_width]
    v = k if values_are_keys else row[:, q_width + k_width:q_width + k_width + v_width]
    if norm == "whole":
        qn, kn = plain.rms_norm(q, gains[0], 1e-3), plain.rms_norm(k, gains[1], 1e-3)
    elif norm == "head":
        qn = plain.rms_norm(q.reshape(n, heads, dim), gains[0], 1e-3).reshape(n, -1)
        kn = plain.rms_norm(k.reshape(n, kv_heads, dim), gains[1], 1e-3).reshape(n, -1)
    else:
        qn, kn = q, k
    q_expected = plain.rotate(qn.reshape(n, heads, dim), positions, rot, layout).reshape(n, -1)
    k_expected = plain.rotate(kn.reshape(n, kv_heads, dim), positions, rot, layout)
    table = dev([[3, 1, 0] + [0] * 110, [0] * 112 + [4], [2] + [0] * 112], torch.int32)
    k_pages = torch.full((5, page_size, kv_heads, dim), float("nan"), device="cuda")
    v_pages = torch.full((5, page_size, kv_heads, vdim), float("nan"), device="cuda")
    q_out = torch.empty((n, q_width), device="cuda")
    inv_freq = torch.tensor(list(plain.frequencies(rot)) or [0.0], dtype=torch.float64, device="cuda")
    ops.norm_rotary_store(dev(row), q_width, q_width if values_are_keys else q_width + k_width, heads, kv_heads, dim, vdim, q_out,
                          dev(gains[0]) if norm else None, dev(gains[1]) if norm else None, norm, 1e-3, rot_dims, layout, inv_freq,
                          dev(positions, torch.int32), dev(items, torch.int32), table, page_size, k_pages, v_pages)
    np.testing.assert_allclose(q_out.cpu().numpy(), q_expected, atol=1e-5)
    where = {0: (3, 6), 1: (3, 7), 2: (1, 0), 3: (1, 1), 4: (4, 900 % 8), 5: (2, 0)}
    for t, (page, place) in where.items():
        np.testing.assert_allclose(k_pages[page, place].cpu().numpy(), k_expected[t], atol=1e-5, err_msg=f"key of token {t}")
        np.testing.assert_allclose(v_pages[page, place].cpu().numpy(), v[t].reshape(kv_heads, vdim), atol=1e-6, err_msg=f"value of token {t}")
    assert int(torch.isnan(k_pages).all(dim=-1).all(dim=-1).sum()) == 5 * page_size - n       # nothing else was written
    # queries alone, for a layer that reads another's keys and values
    q_only = torch.empty((n, q_width), device="cuda")
    ops.norm_rotary_store(dev(row), 0, 0, heads, kv_heads, dim, vdim, q_only, dev(gains[0]) if norm else None, None, norm, 1e-3, rot_dims,
                          layout, inv_freq, dev(positions, torch.int32), dev(items, torch.int32), None, page_size, None, None, writes=False)
    np.testing.assert_allclose(q_only.cpu().numpy(), q_expected, atol=1e-5)


@pytest.mark.parametrize("inner, blocks, n", [(48, 3, 100), (33, 1, 7), (70, 35, 700)])
def test_recurrent_unit_kernel_carries_its_state(inner, blocks, n):
    """A sequence cut in portions (down to one token), beside another request's tokens, against the token-by-token
    formula; the long sequence makes the kernel fold runs of tokens side by side."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(inner)
    part = inner // blocks
    u, y = rng.normal(0, 1, (n, inner)), rng.normal(0, 1, (n, inner))
    gate_r, gate_i = rng.normal(0, 2, (n, inner)), rng.normal(0, 2, (n, inner))
    bias_r, bias_i, lam = rng.normal(0, 1, inner), rng.normal(0, 1, inner), np.linspace(-12.0, 3.0, inner)
    state, expected = np.zeros(inner), np.zeros((n, inner))
    for t in range(n):
        a = np.exp(-8.0 * plain.sigmoid(gate_r[t] + bias_r) * plain.softplus(lam))
        state = a * state + np.sqrt(1.0 - a * a) * plain.sigmoid(gate_i[t] + bias_i) * u[t]
        expected[t] = state * plain.gelu_tanh(y[t])
    gates = np.zeros((n, 2 * inner))
    for b in range(blocks):
        gates[:, 2 * b * part:(2 * b + 1) * part] = gate_r[:, b * part:(b + 1) * part]
        gates[:, (2 * b + 1) * part:(2 * b + 2) * part] = gate_i[:, b * part:(b + 1) * part]
    held = torch.zeros((3, inner), dtype=torch.float32, device="cuda")
    got, done = [], 0
    cuts = []
    for cut in (1, 2, 1, n // 2, 3, n):
        if sum(cuts) < n:
            cuts.append(min(cut, n - sum(cuts)))
    for cut in cuts:
        rows = slice(done, done + cut)
        other = 2                                           # two tokens of another request come first
        pad = lambda x: dev(np.concatenate([rng.normal(0, 1, (other, x.shape[1])), x[rows]]))
        out = torch.empty((other + cut, inner), device="cuda")
        ops.gated_recurrence(out, pad(u), pad(y), pad(gates), dev(bias_r), dev(bias_i), dev(lam), 8.0, held, dev([0, 2], torch.int32),
                             dev([0, other], torch.int32), dev([other, cut], torch.int32), part)
        got.append(out[other:].cpu().numpy())
        done += cut
    np.testing.assert_allclose(np.concatenate(got), expected, atol=2e-5)
    np.testing.assert_allclose(held[2].cpu().numpy(), state, atol=2e-5)
    assert float(held[1].abs().max()) == 0.0


def test_normed_sum_with_the_rounded_rows_and_the_cap():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(3)
    hidden, y, gain = rng.normal(0, 1, (11, 100)), rng.normal(0, 3, (11, 100)), rng.uniform(0.5, 1.5, 100)
    expected = hidden + plain.rms_norm(y, gain, 1e-3)
    stream, rounded = dev(hidden), torch.empty((11, 100), dtype=torch.bfloat16, device="cuda")
    ops.add_normed_cast(stream, dev(y), dev(gain), 1e-3, rounded)
    np.testing.assert_allclose(stream.cpu().numpy(), expected, atol=3e-6)
    assert torch.equal(rounded, stream.to(torch.bfloat16))
    ops.add_normed_cast(stream, act=rounded)                       # the rounding alone
    np.testing.assert_allclose(stream.cpu().numpy(), expected, atol=3e-6)
    logits = dev(rng.normal(0, 20, (5, 77)))
    before = logits.cpu().numpy().astype(np.float64)
    ops.softcap(logits, 15.0)
    np.testing.assert_allclose(logits.cpu().numpy(), 15.0 * np.tanh(before / 15.0), atol=3e-6)


def test_router_with_the_softmax_of_the_chosen_logits():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(4)
    x, router, bias = rng.normal(0, 1, (9, 40)), rng.normal(0, 1, (6, 40)), rng.normal(0, 3, 6)
    for top, shared in ((1, False), (2, True), (6, True)):
        pairs = top + (1 if shared else 0)
        choice = torch.zeros(9 * pairs, dtype=torch.int32, device="cuda")
        in_weight, out_weight = torch.zeros(9 * pairs, device="cuda"), torch.zeros(9 * pairs, device="cuda")
        ops.route(dev(x), dev(router), None, top, choice, in_weight, out_weight, bias=dev(bias), softmax_of_chosen=True, shared_plain=shared)
        logits = x @ router.T + bias
        for t in range(9):
            chosen = np.argsort(-logits[t], kind="stable")[:top]
            weight = np.exp(logits[t, chosen] - logits[t, chosen].max())
            weight /= weight.sum()
            assert choice[t * pairs:t * pairs + top].tolist() == chosen.tolist()
            np.testing.assert_allclose(out_weight[t * pairs:t * pairs + top].cpu().numpy(), weight, atol=1e-6)
            assert in_weight[t * pairs:(t + 1) * pairs].tolist() == [1.0] * pairs
            if shared:
                assert int(choice[t * pairs + top]) == 6 and float(out_weight[t * pairs + top]) == 1.0

"""Lipulorn on the device against the plain implementation (``plain_lipulorn``, float64).

Every test makes its own small configuration and random weights.  32-bit runs must agree within
1e-4 (of the largest logit, where that is above 1) at every token; bfloat16 runs within 4 % of the
logits' spread in the root mean square.  The schedules cut the same requests in different ways: a
request's logits must not depend on the cut, on the rest of the batch, or on which pages and slots
it got."""

import numpy as np
import pytest
import torch

import lipulorn_helpers as lp
import plain_lipulorn as plain
from engine_helpers import (F32_ATOL, random_tokens, run_schedule, schedule_mixed, schedule_portions,
                            schedule_tail_one_by_one, schedule_whole)

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
        expected = lp.plain_logits(folder, tokens)
        bound = atol * max(1.0, float(np.abs(expected).max()))
        worst = np.abs(got[name] - expected).max(axis=1)
        assert worst.max() <= bound, (f"request {name}: first wrong token {int(np.argmax(worst > bound))} of {len(tokens)}, "
                                      f"off by {worst.max():.2e}")
    engine.cache.check()


def dev(values, dtype=torch.float32):
    return torch.tensor(np.asarray(values), dtype=dtype, device="cuda")


# ---- each mechanism alone ----------------------------------------------------------------------

@pytest.mark.parametrize("layer, streams", [
    (lp.latent(mlp=None), 3),
    (lp.latent(mlp=None, heads=1, dim=8, rot_dim=2, vdim=8, kv_rank=6, q_rank=5, window=1), 1),
    (lp.latent(mlp=None, heads=5, dim=12, rot_dim=20, vdim=4, kv_rank=12, q_rank=44, window=300, base=7.0), 2),
    (lp.attention(mlp=None), 3),
    (lp.attention(mlp=None, heads=6, kv_heads=1, dim=8, vdim=40, chunk=1), 4),
    (lp.attention(mlp=None, heads=2, kv_heads=2, dim=24, vdim=8, chunk=500, scale=2.0), 1),
    (lp.delta(mlp=None), 3),
    (lp.delta(mlp=None, heads=1, kv_heads=1, dim=40, vdim=33, taps=1, a_rank=1, g_rank=1), 2),
    (lp.delta(mlp=None, heads=6, kv_heads=2, dim=4, vdim=70, taps=2, a_rank=9, g_rank=2), 5),
    (lp.delta(mlp=lp.dense(7)), 8),
    (lp.attention(), 1),
    (lp.latent(mlp=lp.dense(16)), 12),
], ids=["latent", "latent_one_head_window_of_one", "latent_wide_window_more_rotated_than_not", "attention",
        "attention_one_kv_head_blocks_of_one", "attention_one_block", "delta", "delta_one_head_one_tap_thin_ranks_of_one",
        "delta_three_heads_a_key", "feed_forward_eight_streams", "feed_forward_one_stream", "feed_forward_twelve_streams"])
def test_one_layer_of_each_kind(tmp_path, layer, streams):
    folder = lp.make_model(str(tmp_path / "m"), lp.config([layer], streams=streams), seed=3, matrix_scale=3.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(1, 37, 211), "b": random_tokens(2, 1, 211), "c": random_tokens(3, 2, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_portions(requests))


def test_residual_stream_after_every_layer(tmp_path):
    from mini_llm_b200.engine import StepEntry
    folder = lp.make_model(str(tmp_path / "m"), lp.full_stack(), seed=5, matrix_scale=2.0)
    engine = engine_for(folder)
    tokens = random_tokens(4, 29, 211)
    results = []
    lp.plain_logits(folder, tokens, results)
    slot = engine.open_request()
    engine.step([StepEntry(slot, tokens, [28])], dump_hidden=True)
    assert len(engine.hidden_dump) == len(results) + 1
    for index, expected in enumerate(results):
        np.testing.assert_allclose(engine.hidden_dump[index + 1].cpu().numpy(), expected, rtol=0,
                                   atol=1e-4 * np.abs(expected).max(), err_msg=f"after layer {index}")
    engine.close_request(slot)


def test_thin_ranks_are_read_off_the_tensors(tmp_path):
    """config.json without the inner sizes of the thin matrix pairs: the stored shapes give them."""
    raw = lp.config([lp.delta(a_rank=7, g_rank=3), lp.delta(heads=2, kv_heads=1, a_rank=2, g_rank=11, mlp=None)])
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=6, matrix_scale=2.0, hide_ranks=True)
    requests = {"a": random_tokens(5, 21, 211)}
    check(engine_for(folder), folder, requests, schedule_portions(requests))


def _random_stack(seed):
    """A stack drawn at random: sizes, layer order, windows, blocks, taps, streams, which layers have a
    feed-forward, and which latent layers read an earlier one's rows."""
    rng = np.random.default_rng(1000 + seed)
    pick = lambda values: values[int(rng.integers(0, len(values)))]
    owners, layers = [], []
    for index in range(int(rng.integers(2, 7))):
        mlp = None if rng.random() < 0.3 else lp.dense(int(rng.integers(3, 50)))
        kind = pick(["latent", "latent", "attention", "delta"])
        if kind == "latent":
            heads, dim, vdim, q_rank = int(rng.integers(1, 6)), pick([4, 8, 12, 20]), pick([4, 8, 12, 28]), int(rng.integers(2, 40))
            window = int(rng.integers(1, 70))
            if owners and rng.random() < 0.5:
                source, kv_rank, rot_dim, base = pick(owners)
                layers.append(lp.latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base, 1.0 / (dim + rot_dim), kv_from=source, mlp=mlp))
            else:
                kv_rank, rot_dim, base = pick([8, 12, 24, 40]), pick([2, 4, 8, 16]), pick([10.0, 500.0, 1e5])
                owners.append((index, kv_rank, rot_dim, base))
                layers.append(lp.latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base, 1.0 / (dim + rot_dim), mlp=mlp))
        elif kind == "attention":
            kv_heads = int(rng.integers(1, 4))
            layers.append(lp.attention(kv_heads * int(rng.integers(1, 4)), kv_heads, pick([4, 8, 16, 20]), pick([4, 8, 16, 36]),
                                       int(rng.integers(1, 70)), float(rng.uniform(0.2, 1.5)), mlp=mlp))
        else:
            kv_heads = int(rng.integers(1, 4))
            layers.append(lp.delta(kv_heads * int(rng.integers(1, 3)), kv_heads, pick([4, 8, 12, 36]), pick([4, 8, 20, 33]), int(rng.integers(1, 6)),
                                   int(rng.integers(1, 10)), int(rng.integers(1, 10)), mlp=mlp))
    return lp.config(layers, width=pick([24, 40, 64, 100]), vocab=int(rng.integers(50, 300)), streams=int(rng.integers(1, 7)),
                     eps=pick([1e-6, 1e-5, 1e-3]))


@pytest.mark.parametrize("seed", range(8))
def test_stacks_drawn_at_random(tmp_path, seed):
    """Whatever the configuration says is what runs: whole prompts, portions and mixed batches of a random stack."""
    raw = _random_stack(seed)
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=seed, matrix_scale=2.5)
    engine = engine_for(folder, max_requests=3, cache_tokens=320, debug_poison=True)
    vocab = raw["vocab"]
    requests = {"a": random_tokens(seed, 90, vocab), "b": random_tokens(seed + 50, 2, vocab), "c": random_tokens(seed + 99, 41, vocab)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_portions(requests, sizes=(2, 9, 17, 3, 31)))
    check(engine, folder, requests, schedule_mixed(requests, {"a": 60, "b": 1, "c": 30}, max_live=3))
    assert not any(engine.cache.pages_in_use()) and engine.cache.free_slots == 3


# ---- the same tokens, cut differently -----------------------------------------------------------

def test_prompt_against_token_by_token_and_portions(tmp_path):
    folder = lp.make_model(str(tmp_path / "m"), lp.full_stack(), seed=7, matrix_scale=3.0)
    engine = engine_for(folder)
    requests = {"a": random_tokens(11, 45, 211), "b": random_tokens(12, 7, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=45))        # every token alone, from the first
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=5))
    check(engine, folder, requests, schedule_portions(requests))
    check(engine, folder, requests, schedule_portions(requests, sizes=(2, 2, 3, 2, 17)))
    assert engine.step_kinds["replayed"] > 0          # steps of one shape were replayed from a captured graph


def test_mixed_batches_and_reuse_of_pages_and_slots(tmp_path):
    """Six requests through three slots and a page pool that holds less than their sum: pages
    and slots are given back and used again (and poisoned in between), the pages a window has
    passed go back while the request lives, portions run beside single tokens; every request must
    come out as it does alone."""
    folder = lp.make_model(str(tmp_path / "m"), lp.full_stack(), seed=9, matrix_scale=3.0)
    lengths = {"a": 61, "b": 9, "c": 33, "d": 2, "e": 40, "f": 18}
    requests = {name: random_tokens(20 + i, n, 211) for i, (name, n) in enumerate(lengths.items())}
    prompts = {"a": 40, "b": 9, "c": 20, "d": 1, "e": 40, "f": 3}
    engine = engine_for(folder, max_requests=3, cache_tokens=160, debug_poison=True)
    check(engine, folder, requests, schedule_mixed(requests, prompts, max_live=3))
    check(engine, folder, requests, schedule_mixed(requests, prompts, max_live=2, portion_sizes=(2, 11, 3)))
    assert engine.cache.freed_by_window > 0
    assert not any(engine.cache.pages_in_use()) and engine.cache.free_slots == 3


# ---- keys at the edges of windows and blocks, and far away ---------------------------------------

def _marked_attention(layer_kind, **sizes):
    """One attention layer bent so that the query of token 9 matches the key of token 5 and nothing
    else: tokens 5 and 9 alone have something in the first eight channels, one query/key entry reads
    them with opposite signs, and the marked key's value stands out.  Whether token 5 is seen by a
    late token 9 then decides that token's logits."""
    layer = (lp.latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=8, q_rank=8, scale=1.0, base=50.0, mlp=None, **sizes)
             if layer_kind == "latent" else lp.attention(heads=2, kv_heads=1, dim=8, vdim=8, scale=6.0, mlp=None, **sizes))
    raw = lp.config([layer], vocab=64, width=32, streams=2)

    def bend(t):
        t["embed"][:, :8] = 0.0
        t["embed"][5, :8] = 2.0
        t["embed"][9, :8] = -2.0
        t["l0.norm1"][:] = 1.0
        t["l0.hc1.in"][:] = 0.5
        if layer_kind == "latent":
            # latent entry 0 reads the marked channels; key entry 7 of every head reads latent entry 0, and
            # so does the query's latent and entry 7 (not rotated) of every head's query, with the other sign
            t["l0.mix.dkv"][0] = 0.0
            t["l0.mix.dkv"][0, :8] = 3.0
            t["l0.mix.dkv.norm"][0] = 1.0
            t["l0.mix.dq"][0] = 0.0
            t["l0.mix.dq"][0, :8] = 3.0
            t["l0.mix.dq.norm"][0] = 1.0
            for head in range(2):
                t["l0.mix.uk"][head * 8 + 7] = 0.0
                t["l0.mix.uk"][head * 8 + 7, 0] = 3.0
                t["l0.mix.uq"][head * 12 + 7] = 0.0
                t["l0.mix.uq"][head * 12 + 7, 0] = -3.0
                t["l0.mix.uv"][head * 8:(head + 1) * 8, 0] = 4.0
        else:
            t["l0.mix.k"][7] = 0.0
            t["l0.mix.k"][7, :8] = 2.0
            t["l0.mix.k.b"][:] = 0.0
            t["l0.mix.v"][:, :8] += 1.0
            for head in range(2):
                t["l0.mix.q"][head * 8 + 7] = 0.0
                t["l0.mix.q"][head * 8 + 7, :8] = -2.0
            t["l0.mix.q.b"][:] = 0.0
            t["l0.mix.g"][:] = np.abs(t["l0.mix.g"])
    return raw, bend


def _edge_cases(engine, folder, length, distances, must_differ):
    """Sequences of ``length`` tokens that end in token 9, with token 5 once, ``distance`` places before
    the end: the engine must follow the plain model for each, as a prompt, in portions and with the
    last tokens decoded alone; ``must_differ`` names pairs of distances whose last logits differ."""
    rng = np.random.default_rng(0)
    base = [int(t) for t in rng.integers(10, 64, length)]
    base[-1] = 9
    last = {}
    for distance in distances:
        tokens = list(base)
        if distance is not None:
            tokens[length - 1 - distance] = 5
        last[distance] = lp.plain_logits(folder, tokens)[-1]
        requests = {"r": tokens}
        check(engine, folder, requests, schedule_whole(requests))
        check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=3))
        check(engine, folder, requests, schedule_portions(requests, sizes=(8, 7, 9, 64, 2)))
    for seen, unseen in must_differ:
        assert np.abs(last[seen] - last[unseen]).max() > 0.1, f"the key at distance {seen} does not show"
        assert np.abs(last[unseen] - last[None]).max() < 1e-9, f"a key at distance {unseen} is outside and must not show"


@pytest.mark.parametrize("window", [37, 290])
def test_latent_window_edges_and_a_far_key(tmp_path, window):
    """The marked key just inside the window (distance window - 1) decides the last logits, also far back
    behind many page borders; one place further (distance window) it is outside and changes nothing."""
    raw, bend = _marked_attention("latent", window=window)
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=13, bend=bend, matrix_scale=2.0)
    engine = engine_for(folder)
    _edge_cases(engine, folder, 300, (None, 1, window - 1, window), [(window - 1, window), (1, window)])


@pytest.mark.parametrize("chunk", [40, 256])
def test_attention_block_edges_and_a_far_key(tmp_path, chunk):
    """A block's first position is seen from its last, the position before it is not; blocks count
    from position 0 whatever the cut."""
    raw, bend = _marked_attention("attention", chunk=chunk)
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=14, bend=bend, matrix_scale=2.0)
    engine = engine_for(folder, debug_poison=True)
    length = 300
    inside = (length - 1) % chunk                  # the distance from the last position to its block's first
    _edge_cases(engine, folder, length, (None, 0 if inside == 0 else 1, inside, inside + 1), [(inside, inside + 1)])
    assert engine.cache.freed_by_window > 0        # the pages of the blocks a request has left went back (and were poisoned)


def test_shared_rows_through_a_wider_and_a_narrower_window(tmp_path):
    """A layer that reads another layer's cached rows has a mask of its own: the rows stay as long as
    the widest window needs them, in long decoding too (pages go back meanwhile)."""
    raw = lp.config([lp.latent(window=6, mlp=None), lp.latent(kv_from=0, window=29, heads=2, q_rank=9, mlp=None),
                     lp.latent(kv_from=0, window=2, heads=4, dim=8, vdim=8)], streams=2)
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=15, matrix_scale=3.0)
    engine = engine_for(folder, debug_poison=True)
    requests = {"a": random_tokens(31, 90, 211), "b": random_tokens(32, 33, 211)}
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=60))
    check(engine, folder, requests, schedule_mixed(requests, {"a": 50, "b": 10}, max_live=2))
    assert engine.cache.freed_by_window > 0


def test_an_old_write_is_read_back_and_replaced(tmp_path):
    """The delta rule with decays bent to almost 1 in some key channels and to a fast fall in others, and
    write gates at both ends: what an early token wrote is still read two hundred tokens later.
    Long decoding, token by token, against the whole prompt."""
    raw = lp.config([lp.delta(heads=2, kv_heads=1, dim=8, vdim=8, taps=2, a_rank=4, g_rank=4, mlp=None),
                     lp.delta(heads=2, kv_heads=2, dim=16, vdim=24, taps=4, a_rank=5, g_rank=6)], width=32, vocab=97)

    def bend(t):
        t["l0.mix.A_log"][:] = [-9.0, 1.5]
        t["l0.mix.dt_bias"][:] = np.tile([-2.0, 1.0, -4.0, 0.0], 4)
        t["l0.mix.b"] *= 30.0                      # write gates at both ends
        t["l1.mix.A_log"][:] = [-6.0, 0.5]
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=17, bend=bend, matrix_scale=2.0)
    engine = engine_for(folder)
    requests = {"long": random_tokens(31, 221, 97)}
    check(engine, folder, requests, schedule_tail_one_by_one(requests, tail=220))
    check(engine, folder, requests, schedule_whole(requests))
    check(engine, folder, requests, schedule_portions(requests, sizes=(16, 17, 15, 2, 33)))


# ---- bfloat16 ---------------------------------------------------------------------------------------

def check_rounding(engine, folder, requests, steps, share=0.04):
    """bfloat16 against the plain model: over a request, the root mean square of the difference stays
    below ``share`` of the logits' standard deviation (the 32-bit runs bound every token)."""
    got = run_schedule(engine, requests, steps)
    for name, tokens in requests.items():
        expected = lp.plain_logits(folder, tokens)
        ratio = float(np.sqrt(((got[name] - expected) ** 2).mean()) / expected.std())
        assert ratio <= share, f"request {name}: root mean square of the difference is {ratio:.3f} of the logits' spread"
    engine.cache.check()


def test_bfloat16_follows_within_its_rounding(tmp_path):
    raw = lp.config([lp.latent(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=48, q_rank=40, window=50, mlp=lp.dense(96)),
                     lp.attention(heads=4, kv_heads=2, dim=32, vdim=64, chunk=48, mlp=lp.dense(96)),
                     lp.delta(heads=4, kv_heads=2, dim=32, vdim=32, taps=4, a_rank=8, g_rank=16, mlp=lp.dense(96)),
                     lp.latent(kv_from=0, heads=2, dim=64, rot_dim=16, vdim=64, kv_rank=48, q_rank=24, window=70, mlp=None)],
                    width=128)
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=19, bfloat16_values=True)
    engine = engine_for(folder, dtype="bfloat16")
    requests = {"a": random_tokens(41, 140, 211), "b": random_tokens(42, 12, 211), "c": random_tokens(43, 70, 211)}
    check_rounding(engine, folder, requests, schedule_whole(requests))
    check_rounding(engine, folder, requests, schedule_mixed(requests, {"a": 100, "b": 6, "c": 64}, max_live=3))
    check_rounding(engine, folder, requests, schedule_tail_one_by_one(requests, tail=10))
    chosen = set(engine.kernels.choices.values())
    assert {"capped_attention_tiled", "latent_attention_tiled", "gemm_tcgen05"} <= chosen


def test_bfloat16_with_sizes_no_fast_kernel_takes(tmp_path):
    """A width that is no multiple of 8 and odd head sizes: every product and the attentions fall back
    to kernels that take any size, in bfloat16 too."""
    raw = lp.config([lp.latent(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=21, q_rank=9, window=33),
                     lp.attention(heads=3, kv_heads=1, dim=10, vdim=14, chunk=21),
                     lp.delta(heads=2, kv_heads=2, dim=6, vdim=10, taps=5, a_rank=3, g_rank=5, mlp=lp.dense(9))],
                    width=100, vocab=203)
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=29, bfloat16_values=True)
    requests = {"a": random_tokens(61, 150, 203), "b": random_tokens(62, 3, 203), "c": random_tokens(63, 40, 203)}
    engine = engine_for(folder, dtype="bfloat16")
    check_rounding(engine, folder, requests, schedule_whole(requests))
    check_rounding(engine, folder, requests, schedule_mixed(requests, {"a": 130, "b": 2, "c": 33}, max_live=3))
    check(engine_for(folder), folder, requests, schedule_portions(requests))


def test_nothing_depends_on_what_fresh_memory_holds(tmp_path):
    """Steps with prompt portions are filled up to round shapes with tokens of no request; the rows of those
    tokens that no attention tile takes are read by the kernels after them.  With every byte the engine gets
    from the allocator full of NaN beforehand, and a first step that makes the buffers larger than the steps
    after it need, no request's logits may change."""
    from mini_llm_b200.engine import StepEntry
    raw = lp.config([lp.latent(heads=3, dim=16, rot_dim=8, vdim=8, kv_rank=40, q_rank=40, window=166, mlp=None),
                     lp.attention(heads=4, kv_heads=2, dim=48, vdim=8, chunk=180),
                     lp.delta(heads=1, kv_heads=1, dim=8, vdim=20, taps=5, a_rank=24, g_rank=7, mlp=lp.dense(24)),
                     lp.attention(heads=4, kv_heads=2, dim=32, vdim=36, chunk=14, mlp=lp.dense(100)),
                     lp.attention(heads=4, kv_heads=2, dim=16, vdim=16, chunk=94, mlp=lp.dense(100))], width=256, vocab=352, streams=1)
    folder = lp.make_model(str(tmp_path / "m"), raw, seed=15, bfloat16_values=True)
    junk = [torch.full((size,), float("nan"), device="cuda") for size in (1 << 26, 1 << 24, 1 << 22, 1 << 20, 1 << 18, 1 << 16)
            for _ in range(2)]
    del junk
    engine = engine_for(folder, dtype="bfloat16", page_size=16, max_requests=3)
    slot = engine.open_request()
    engine.step([StepEntry(slot, random_tokens(15, 300, 352), [299])], dump_hidden=True)       # runs as it is, not filled up
    engine.close_request(slot)
    requests = {"a": random_tokens(15, 300, 352), "b": random_tokens(65, 2, 352), "c": random_tokens(114, 150, 352)}
    check_rounding(engine, folder, requests, schedule_whole(requests), share=0.06)
    check_rounding(engine, folder, requests, schedule_mixed(requests, {"a": 260, "b": 1, "c": 100}, max_live=3), share=0.06)


def test_greedy_generation_through_the_scheduler(tmp_path):
    from mini_llm_b200.generate import generate
    folder = lp.make_model(str(tmp_path / "m"), lp.full_stack(), seed=23, matrix_scale=3.0)
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

"""Lipulorn without a device: the configuration's round trip and its errors, what the layers keep
per request, whose rows a layer reads, and the plain model's own masks, rotation and causality."""

import copy

import numpy as np
import pytest

import lipulorn_helpers as lp
import plain_lipulorn as plain
from mini_llm_b200.config import ConfigError, config_from_dict, describe_model
from mini_llm_b200.engine.model import Model
from mini_llm_b200.parts.spec import FixedState, PagedKV


def test_round_trip():
    raw = lp.full_stack()
    parsed = config_from_dict(raw)
    assert parsed.architecture == "Lipulorn"
    assert parsed.to_dict() == raw
    assert config_from_dict(parsed.to_dict()) == parsed


def _without(raw, path):
    raw = copy.deepcopy(raw)
    node = raw
    for key in path[:-1]:
        node = node[key]
    del node[path[-1]]
    return raw


def _with(raw, path, value):
    raw = copy.deepcopy(raw)
    node = raw
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    return raw


@pytest.mark.parametrize("change, named", [
    (lambda r: _without(r, ["vocab"]), "vocab"),
    (lambda r: _without(r, ["streams"]), "streams"),
    (lambda r: _with(r, ["streams"], 17), "streams"),
    (lambda r: _without(r, ["norm", "eps"]), "norm.eps"),
    (lambda r: _with(r, ["layers", 0, "type"], "hyena"), "layers[0].type"),
    (lambda r: _without(r, ["layers", 0, "mixer", "kv_rank"]), "layers[0].mixer.kv_rank"),
    (lambda r: _with(r, ["layers", 0, "mixer", "rot", "dims"], 7), "layers[0].mixer.rot.dims"),
    (lambda r: _with(r, ["layers", 0, "mixer", "rot", "base"], 1.0), "layers[0].mixer.rot.base"),
    (lambda r: _without(r, ["layers", 0, "mixer", "mask", "size"]), "layers[0].mixer.mask.size"),
    (lambda r: _with(r, ["layers", 1, "mixer", "heads"], 3), "layers[1].mixer.heads"),
    (lambda r: _with(r, ["layers", 1, "mixer", "scale"], "wide"), "layers[1].mixer.scale"),
    (lambda r: _without(r, ["layers", 2, "mixer", "conv"]), "layers[2].mixer.conv"),
    (lambda r: _with(r, ["layers", 3, "mixer", "kv_from"], 1), "layers[3].mixer.kv_from"),
    (lambda r: _with(r, ["layers", 3, "mixer", "kv_from"], 3), "layers[3].mixer.kv_from"),
    (lambda r: _with(r, ["layers", 6, "mixer", "kv_from"], 3), "layers[6].mixer.kv_from"),
    (lambda r: _with(r, ["layers", 3, "mixer", "kv_rank"], 41), "layers[3].mixer.kv_rank"),
    (lambda r: _with(r, ["layers", 0, "mlp", "kind"], "moe"), "layers[0].mlp.kind"),
    (lambda r: _without(r, ["layers", 0, "mlp", "ff"]), "layers[0].mlp.ff"),
])
def test_errors_name_their_key(change, named):
    with pytest.raises(ConfigError) as error:
        config_from_dict(change(lp.full_stack()))
    assert f"'{named}" in str(error.value)


def test_what_the_layers_keep():
    model = Model(describe_model(config_from_dict(lp.full_stack())))
    needs = model.cache_needs()
    # the latent rows stay as long as the widest window of the layers that read them (11, 17 and 4)
    assert needs[0] == PagedKV(1, 40 + 8, 17, has_values=False)
    assert needs[1] == PagedKV(2, 12, None, value_size=20, block=9)       # keys before the newest block are never read again
    assert needs[2] == {"mixer.state": FixedState((4 * 12 * 20,), "float32"), "mixer.taps": FixedState((2, 2 * 2 * 12 + 4 * 20), "float32")}
    assert needs[3] is None and needs[6] is None           # they read layer 0's rows
    assert needs[4] == {"mixer.state": FixedState((2 * 20 * 8,), "float32"), "mixer.taps": FixedState((1, 2 * 2 * 20 + 2 * 8), "float32")}
    assert [entry.cache_of for entry in model.spec.order] == [None, None, None, 0, None, None, 0]
    assert model.spec.residual_streams == 3
    assert model.graph_safe
    # one tap: nothing to keep for the convolution
    lone = Model(describe_model(config_from_dict(lp.config([lp.delta(taps=1)]))))
    assert lone.cache_needs()[0] == {"mixer.state": FixedState((4 * 12 * 20,), "float32")}


def test_declared_tensors():
    """The names and shapes a file must hold; a layer without feed-forward declares no second norm or connection."""
    from mini_llm_b200.weights.loader import collect_specs
    model = Model(describe_model(config_from_dict(lp.config([lp.latent(), lp.latent(kv_from=0, mlp=None), lp.attention(),
                                                              lp.delta(a_rank=None, g_rank=None)], streams=2))))
    specs = collect_specs(model.parts())
    shapes = {name: tuple(spec.shape) for name, spec in specs.items()}
    assert shapes["embed"] == (211, 64) and shapes["head"] == (211, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.hc1.in"] == (2,) and shapes["l0.hc2.mix"] == (2, 2)
    assert shapes["l0.mix.dq"] == (20, 64) and shapes["l0.mix.uq"] == (3 * (16 + 8), 20)
    assert shapes["l0.mix.dkv"] == (40 + 8, 64) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l0.mix.uk"] == (3 * 16, 40) and shapes["l0.mix.uv"] == (3 * 24, 40) and shapes["l0.mix.o"] == (64, 3 * 24)
    assert "l1.mix.dkv" not in shapes and "l1.norm2" not in shapes and "l1.hc2.in" not in shapes and "l1.mlp.up" not in shapes
    assert shapes["l2.mix.q.b"] == (4 * 12,) and shapes["l2.mix.k"] == (2 * 12, 64) and shapes["l2.mix.g"] == (4, 64)
    assert shapes["l3.mix.v.conv"] == (4 * 20, 3) and shapes["l3.mix.A_log"] == (4,) and shapes["l3.mix.dt_bias"] == (4 * 12,)
    assert shapes["l3.mix.a1"] == (None, 64) and shapes["l3.mix.a2"] == (4 * 12, None)       # the file gives the inner size
    assert shapes["l3.mix.g2"] == (4 * 20, None) and shapes["l3.mix.norm"] == (20,)
    assert shapes["l3.mlp.gate.b"] == (40,) and shapes["l3.mlp.down"] == (64, 40)


def test_the_plain_masks():
    window = plain.window_mask(9, 3)
    assert window[5].tolist() == [False] * 3 + [True] * 3 + [False] * 3
    assert window[1].tolist() == [True, True] + [False] * 7
    blocks = plain.chunk_mask(9, 4)
    assert blocks[5].tolist() == [False] * 4 + [True, True] + [False] * 3
    assert blocks[4].tolist() == [False] * 4 + [True] + [False] * 4
    assert blocks[3].tolist() == [True] * 4 + [False] * 5


def test_the_plain_rotation():
    """Entry i turns with entry i + dims/2; what lies beyond ``dims`` passes; the scores depend on the distance alone."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((1, 1, 10))
    turned = plain.rotate_half(np.repeat(x, 4, axis=0), [0, 1, 7, 8], 50.0, 6)
    np.testing.assert_allclose(turned[0], x[0])
    np.testing.assert_allclose(turned[:, :, 6:], np.repeat(x, 4, axis=0)[:, :, 6:])
    angle = 7 * 50.0 ** (-2.0 / 6)
    np.testing.assert_allclose(turned[2, 0, 1], x[0, 0, 1] * np.cos(angle) - x[0, 0, 4] * np.sin(angle))
    np.testing.assert_allclose(turned[2, 0, 4], x[0, 0, 4] * np.cos(angle) + x[0, 0, 1] * np.sin(angle))
    y = rng.standard_normal((1, 1, 10))
    other = plain.rotate_half(np.repeat(y, 4, axis=0), [0, 1, 7, 8], 50.0, 6)
    np.testing.assert_allclose((turned[1] * other[0]).sum(), (turned[3] * other[2]).sum())


def test_the_plain_model_is_causal(tmp_path):
    folder = lp.make_model(str(tmp_path / "m"), lp.full_stack(), seed=1, matrix_scale=2.0)
    config, tensors = plain.load_model(folder)
    tokens = np.random.default_rng(0).integers(0, 211, 40).tolist()
    full = plain.forward(config, tensors, tokens)
    short = plain.forward(config, tensors, tokens[:23])
    np.testing.assert_allclose(full[:23], short, atol=1e-10)
    changed = list(tokens)
    changed[31] = (changed[31] + 1) % 211
    np.testing.assert_allclose(plain.forward(config, tensors, changed)[:31], full[:31], atol=1e-10)
    assert np.abs(plain.forward(config, tensors, changed)[31:] - full[31:]).max() > 1e-6

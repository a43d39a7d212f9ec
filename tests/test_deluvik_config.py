"""Deluvik without a device: the configuration's round trip and its errors, what the layers keep per request (also a
layer that reads another's keys and values), the scaled frequencies, and the plain model's own properties."""

import copy
import math

import numpy as np
import pytest

import deluvik_helpers as dv
import plain_deluvik as plain
from mini_llm_b200.config import ConfigError, config_from_dict, describe_model
from mini_llm_b200.engine.model import Model
from mini_llm_b200.parts.rotary import banded_frequencies
from mini_llm_b200.parts.spec import FixedState, PagedKV


def test_round_trip():
    raw = dv.full_stack()
    parsed = config_from_dict(raw)
    assert parsed.architecture == "Deluvik"
    assert parsed.to_dict() == raw
    assert config_from_dict(parsed.to_dict()) == parsed
    bare = dv.config([dv.attention(softcap=None, scaling=None, mlp=None)], logit_softcap=None)
    assert config_from_dict(bare).to_dict() == bare


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
    (lambda r: _without(r, ["width"]), "width"),
    (lambda r: _without(r, ["norm", "eps"]), "norm.eps"),
    (lambda r: _with(r, ["logit_softcap"], "soft"), "logit_softcap"),
    (lambda r: _with(r, ["layers", 0, "type"], "hyena"), "layers[0].type"),
    (lambda r: _without(r, ["layers", 0, "mixer", "conv"]), "layers[0].mixer.conv"),
    (lambda r: _with(r, ["layers", 1, "mixer", "heads"], 5), "layers[1].mixer.heads"),
    (lambda r: _with(r, ["layers", 1, "mixer", "vdim"], 8), "layers[1].mixer.vdim"),
    (lambda r: _with(r, ["layers", 1, "mixer", "rot", "dims"], 18), "layers[1].mixer.rot.dims"),
    (lambda r: _without(r, ["layers", 1, "mixer", "rot", "scaling", "low"]), "layers[1].mixer.rot.scaling.low"),
    (lambda r: _with(r, ["layers", 1, "mixer", "rot", "scaling", "high"], 0.5), "layers[1].mixer.rot.scaling.high"),
    (lambda r: _with(r, ["layers", 2, "mixer", "kv_from"], 1), "layers[2].mixer.kv_from"),
    (lambda r: _with(r, ["layers", 2, "mixer", "kv_from"], 2), "layers[2].mixer.kv_from"),
    (lambda r: _with(r, ["layers", 4, "mixer", "kv_from"], 2), "layers[4].mixer.kv_from"),
    (lambda r: _with(r, ["layers", 2, "mixer", "kv_heads"], 4), "layers[2].mixer.kv_from"),
    (lambda r: _without(r, ["layers", 3, "mixer", "left", "mask", "size"]), "layers[3].mixer.left.mask.size"),
    (lambda r: _with(r, ["layers", 3, "mixer", "right", "blocks"], 5), "layers[3].mixer.right.blocks"),
    (lambda r: _without(r, ["layers", 3, "mixer", "left_scale"]), "layers[3].mixer.left_scale"),
    (lambda r: _with(r, ["layers", 1, "mlp", "router", "top"], 9), "layers[1].mlp.router.top"),
    (lambda r: _with(r, ["layers", 0, "mlp", "kind"], "sparse"), "layers[0].mlp.kind"),
    (lambda r: _without(r, ["layers", 0, "mlp", "ff"]), "layers[0].mlp.ff"),
])
def test_errors_name_their_key(change, named):
    with pytest.raises(ConfigError) as error:
        config_from_dict(change(dv.full_stack()))
    assert f"'{named}" in str(error.value)


def test_what_the_layers_keep():
    spec = describe_model(config_from_dict(dv.full_stack()))
    assert [entry.cache_of for entry in spec.order] == [None, None, 0, None, 0, None, None, None]
    needs = Model(spec).cache_needs()
    assert needs[0] == {"mixer.kv": PagedKV(2, 16, None, value_size=24), "mixer.taps": FixedState((2, 64 + 32 + 48), "float32")}
    assert needs[1] == {"mixer.kv": PagedKV(2, 16, None, value_size=16)}
    # a layer that reads another's keys and values keeps the last inputs of its own queries' convolution only
    assert needs[2] == {"mixer.taps": FixedState((2, 64), "float32")} and needs[4] == needs[2]
    assert needs[3] == {"mixer.left.kv": PagedKV(2, 16, 11, value_size=8), "mixer.right.state": FixedState((48,), "float32"),
                        "mixer.right.taps": FixedState((3, 48), "float32")}
    assert needs[7] == {"mixer.kv": PagedKV(1, 24, None, value_size=8)}       # one tap: no state
    names = {w.name for part in Model(spec).parts() for w in part.weight_specs()}
    assert "l2.mix.q.conv" in names and "l2.mix.sink" in names and not any(n.startswith(("l2.mix.k", "l2.mix.v")) for n in names)
    assert "l1.mix.k.norm" in names and "l1.mix.v" not in names and "l3.mix.left.sink" not in names
    assert "l2.norm2" not in names and "l1.mlp.router.b" in names and "l1.mlp.shared.sg" not in names


def test_frequencies_by_bands():
    bands = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}
    got = banded_frequencies(300.0, 12, bands)
    for i, f in enumerate(got):
        plain_f = 300.0 ** (-2.0 * i / 12)
        wavelength = 2.0 * math.pi / plain_f
        if wavelength < 16.0:
            assert f == plain_f
        elif wavelength > 48.0:
            assert f == plain_f / 4.0
        else:
            assert plain_f / 4.0 < f < plain_f
    assert any(f == 300.0 ** (-2.0 * i / 12) for i, f in enumerate(got)) and got[-1] == 300.0 ** (-10.0 / 12) / 4.0
    assert len({f / 300.0 ** (-2.0 * i / 12) for i, f in enumerate(got)}) >= 3        # all three bands occur
    np.testing.assert_allclose(got, plain.frequencies({"base": 300.0, "dims": 12, "scaling": bands}), rtol=1e-15)
    assert banded_frequencies(300.0, 12, None) == [300.0 ** (-2.0 * i / 12) for i in range(6)]


def _random_weights(raw, seed=0):
    from mini_llm_b200.weights.random_init import random_tensors
    tensors = random_tensors(describe_model(config_from_dict(raw)), seed, "varied")
    return {name: values.astype(np.float64) * (8.0 if name.endswith("conv") else 1.0) for name, values in tensors.items()}


def test_plain_model_is_causal_and_its_window_and_sink_matter():
    raw = dv.full_stack()
    w = _random_weights(raw)
    rng = np.random.default_rng(0)
    tokens = rng.integers(0, 211, 30).tolist()
    logits = plain.forward(raw, w, tokens)
    changed = list(tokens)
    changed[20] = (changed[20] + 1) % 211
    again = plain.forward(raw, w, changed)
    np.testing.assert_array_equal(logits[:20], again[:20])
    assert np.abs(logits[20:] - again[20:]).max() > 1e-3
    assert np.abs(logits).max() <= raw["logit_softcap"]
    # the window: a key window positions back is the last one seen
    q, k, v = rng.normal(0, 1, (9, 2, 4)), rng.normal(0, 1, (9, 1, 4)), rng.normal(0, 1, (9, 1, 4))
    seen = plain.attend(q, k, v, 1.0, window=3)
    k2, v2 = k.copy(), v.copy()
    k2[5], v2[5] = 9.0, 9.0
    other = plain.attend(q, k2, v2, 1.0, window=3)
    np.testing.assert_array_equal(seen[8], other[8])            # position 8 sees 6, 7, 8
    assert np.abs(seen[7] - other[7]).max() > 1e-3              # position 7 sees 5, 6, 7
    # the sink takes weight and gives nothing back
    with_sink = plain.attend(q, k, v, 1.0, sink=np.array([0.0, 30.0]))
    without = plain.attend(q, k, v, 1.0)
    assert np.abs(with_sink[:, 1]).max() < 1e-6 and np.all(np.abs(with_sink[1:, 0]) < np.abs(without[1:, 0]).max() + 1e-9)
    np.testing.assert_allclose(with_sink[0, 0], without[0, 0] * (math.exp((q[0, 0] @ k[0, 0])) / (math.exp(q[0, 0] @ k[0, 0]) + 1.0)))


def test_plain_recurrent_unit_against_its_closed_form():
    """With gates that do not depend on the input (zero gate matrices), S_t is a geometric sum."""
    sizes = {"width": 6, "blocks": 2, "conv": 1}
    rng = np.random.default_rng(1)
    w = {"p.y": rng.normal(0, 1, (6, 5)), "p.y.b": rng.normal(0, 1, 6), "p.x": rng.normal(0, 1, (6, 5)), "p.x.b": rng.normal(0, 1, 6),
         "p.conv": np.ones((6, 1)), "p.conv.b": np.zeros(6), "p.ra": np.zeros((2, 3, 3)), "p.ra.b": rng.normal(0, 1, (2, 3)),
         "p.ri": np.zeros((2, 3, 3)), "p.ri.b": rng.normal(0, 1, (2, 3)), "p.lam": rng.normal(0, 1, 6), "p.o": np.eye(6)}
    x = rng.normal(0, 1, (7, 5))
    got = plain.gated_linear_unit(x, sizes, w, "p")
    u = x @ w["p.x"].T + w["p.x.b"]
    a = np.exp(-8.0 * plain.sigmoid(w["p.ra.b"].reshape(-1)) * plain.softplus(w["p.lam"]))
    gain = np.sqrt(1.0 - a * a) * plain.sigmoid(w["p.ri.b"].reshape(-1))
    state = sum(a ** (6 - t) * gain * u[t] for t in range(7))
    np.testing.assert_allclose(got[6], state * plain.gelu_tanh(x[6] @ w["p.y"].T + w["p.y.b"]), rtol=1e-12)

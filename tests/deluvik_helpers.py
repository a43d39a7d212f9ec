"""Shared by the Deluvik tests: small configurations (none with the sizes of any released model), model folders
with random weights that a test may then bend, and the plain logits."""

import json
import os

import numpy as np

import plain_deluvik as plain
from mini_llm_b200.config import config_from_dict, describe_model
from mini_llm_b200.weights.random_init import random_tensors
from mini_llm_b200.weights.safetensors_io import write_safetensors

BANDS = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 48}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=24, shared=40):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": None if shared is None else {"ff": shared}}


def rotation(dims, base=300.0, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(scaling)
    return rot


def attention(heads=4, kv_heads=2, dim=16, rot_dims=12, base=300.0, scaling=BANDS, scale=0.3, softcap=5.0, mlp="default"):
    """The values are the keys as projected: one size for both."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rotation(rot_dims, base, scaling)}
    if softcap is not None:
        mixer["softcap"] = softcap
    return {"type": "attention", "mixer": mixer, "mlp": moe() if mlp == "default" else mlp}


def attention_2(heads=4, kv_heads=2, dim=16, vdim=24, taps=3, rot_dims=8, base=300.0, scaling=None, scale=0.3, kv_from=None,
                mlp="default"):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps, "scale": scale,
             "rot": rotation(rot_dims, base, scaling)}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": mixer, "mlp": moe() if mlp == "default" else mlp}


def parallel(heads=4, kv_heads=2, dim=16, vdim=8, window=11, rot_dims=6, base=300.0, scaling=None, scale=0.3, inner=48, blocks=3,
             taps=4, left_scale=0.7, right_scale=1.2, mlp="default"):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                               "mask": {"size": window}, "rot": rotation(rot_dims, base, scaling)},
                      "right": {"width": inner, "blocks": blocks, "conv": taps},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": moe() if mlp == "default" else mlp}


def config(layers, width=96, vocab=211, eps=1e-5, logit_softcap=9.0):
    raw = {"architecture": "Deluvik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": list(layers)}
    if logit_softcap is not None:
        raw["logit_softcap"] = logit_softcap
    return raw


def full_stack(**kw):
    """Every layer type, with and without feed-forward, two layers that read an earlier layer's keys and values
    (one of them not the layer before), other sizes in the later layers."""
    return config([attention_2(mlp=dense()),
                   attention(),
                   attention_2(kv_from=0, mlp=None),
                   parallel(),
                   attention_2(kv_from=0, mlp=moe(experts=3, top=1, ff=16, shared=None)),
                   attention(heads=3, kv_heads=3, dim=8, rot_dims=8, scaling=None, softcap=None, scale=0.5, mlp=dense(24)),
                   parallel(heads=2, kv_heads=1, dim=8, vdim=24, window=5, rot_dims=0, inner=40, blocks=1, taps=2,
                            mlp=moe(experts=4, top=4, ff=8, shared=8)),
                   attention_2(heads=2, kv_heads=1, dim=24, vdim=8, taps=1, rot_dims=24, scaling=BANDS, mlp=None)],
                  **kw)


def to_bfloat16_values(values):
    """The nearest values that bfloat16 holds (ties to even), still as float32."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(np.shape(values))


def make_model(folder, raw, seed=0, bend=None, matrix_scale=1.0, bfloat16_values=False):
    """Write config.json and model.safetensors (32-bit) with random weights: matrices N(0, 0.05) times
    ``matrix_scale``, gains U(0.5, 1.5), biases N(0, 0.02); taps of about 0.4, sinks N(0, 1.5), decay rates
    N(0, 2): every tap, sink and rate matters.  ``bend(tensors)`` may change them before they are written.
    ``bfloat16_values``: every value is one that bfloat16 holds, as in a model that was stored in that type."""
    parsed = config_from_dict(raw)
    tensors = random_tensors(describe_model(parsed), seed, "varied")
    for name, values in tensors.items():
        if values.ndim >= 2 and not name.endswith("conv") and name != "embed":
            values *= matrix_scale
        if name.endswith("conv"):
            values *= 8.0
        if name.endswith(".sink"):
            values *= 15.0
        if name.endswith(".lam"):
            values *= 20.0
        if name.endswith("router.b"):
            values *= 10.0
    if bend is not None:
        bend(tensors)
    if bfloat16_values:
        tensors = {name: to_bfloat16_values(values) for name, values in tensors.items()}
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(raw, handle)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, {name: "F32" for name in tensors})
    return folder


_cache = {}


def plain_logits(folder, tokens, keep_layers=False):
    key = (folder, tuple(tokens))
    if keep_layers:
        model_config, tensors = plain.load_model(folder)
        return plain.forward(model_config, tensors, list(tokens), keep_layers=True)
    if key not in _cache:
        model_config, tensors = plain.load_model(folder)
        _cache[key] = plain.forward(model_config, tensors, list(tokens))
    return _cache[key]

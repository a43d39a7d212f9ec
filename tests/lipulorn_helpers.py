"""Shared by the Lipulorn tests: small configurations (none with the sizes of any released model),
model folders with random weights that a test may then bend, and the plain logits."""

import json
import os

import numpy as np

import plain_lipulorn as plain
from mini_llm_b200.config import config_from_dict, describe_model
from mini_llm_b200.weights.random_init import random_tensors
from mini_llm_b200.weights.safetensors_io import write_safetensors
from sumozen_helpers import to_bfloat16_values

DENSE = "default"


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def _mlp(mlp):
    return dense() if mlp == DENSE else mlp


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=20, window=11, base=100.0, scale=0.3, kv_from=None,
           mlp=DENSE):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": scale, "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": _mlp(mlp)}


def attention(heads=4, kv_heads=2, dim=12, vdim=20, chunk=9, scale=0.4, mlp=DENSE):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": chunk}}, "mlp": _mlp(mlp)}


def delta(heads=4, kv_heads=2, dim=12, vdim=20, taps=3, a_rank=6, g_rank=5, mlp=DENSE):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps,
                                               "a_rank": a_rank, "g_rank": g_rank}, "mlp": _mlp(mlp)}


def config(layers, width=64, vocab=211, streams=3, eps=1e-5):
    return {"architecture": "Lipulorn", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps},
            "layers": list(layers)}


def full_stack(**kw):
    """Every layer type, with and without feed-forward, a layer that reads another's rows through a wider
    window and one through a narrower, and other sizes in the second half."""
    return config([latent(), attention(), delta(mlp=None), latent(kv_from=0, window=17, heads=2, dim=8, vdim=8, q_rank=12),
                   delta(heads=2, kv_heads=2, dim=20, vdim=8, taps=2, a_rank=3, g_rank=9, mlp=dense(24)),
                   attention(heads=3, kv_heads=3, dim=8, vdim=8, chunk=5, mlp=None),
                   latent(kv_from=0, window=4, heads=4, dim=8, vdim=16, q_rank=8, mlp=None)], **kw)


def make_model(folder, raw, seed=0, bend=None, matrix_scale=1.0, bfloat16_values=False, hide_ranks=False):
    """Write config.json and model.safetensors (32-bit) with random weights: matrices N(0, 0.05)
    times ``matrix_scale``, gains U(0.5, 1.5), biases N(0, 0.02); the streams' mixing matrices near the
    identity (off the diagonal within 0.3).  ``bend(tensors)`` may change them before they are written.
    ``bfloat16_values``: every value is one that bfloat16 holds.  ``hide_ranks``: the inner sizes of the
    thin matrix pairs are left out of config.json (the engine then reads them off the tensors)."""
    parsed = config_from_dict(raw)
    tensors = random_tensors(describe_model(parsed), seed, "varied")
    for name, values in tensors.items():
        if values.ndim == 2 and not name.endswith("conv") and name != "embed" and ".hc" not in name:
            values *= matrix_scale
        if name.endswith("conv"):
            values *= 8.0                   # taps of about 0.4: every tap matters
        if name.endswith(".mix") and ".hc" in name:
            values[:] = (values - 1.0) * 0.6 + np.eye(values.shape[0])
        if name.endswith("dt_bias") or name.endswith("A_log"):
            values *= 30.0                  # decays spread between slow and fast
    if bend is not None:
        bend(tensors)
    if bfloat16_values:
        tensors = {name: to_bfloat16_values(values) for name, values in tensors.items()}
    if hide_ranks:
        raw = json.loads(json.dumps(raw))
        for layer in raw["layers"]:
            layer["mixer"].pop("a_rank", None)
            layer["mixer"].pop("g_rank", None)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(raw, handle)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, {name: "F32" for name in tensors})
    return folder


_plain_cache = {}


def plain_logits(folder, tokens, layer_results=None):
    """Logits [len, vocab] of the plain implementation (float64)."""
    key = (folder, tuple(tokens))
    if key not in _plain_cache or layer_results is not None:
        model_config, tensors = plain.load_model(folder)
        _plain_cache[key] = plain.forward(model_config, tensors, list(tokens), layer_results)
    return _plain_cache[key]

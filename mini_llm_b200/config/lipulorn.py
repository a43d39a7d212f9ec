"""Configuration of Lipulorn: a stack over several residual streams whose layers each name their mixer.

``config.json`` is nested: ``vocab``, ``width``, ``streams`` (the number of residual streams of the
hyper-connections), ``norm`` (``eps``) and ``layers``, a list whose entries give ``type``
("latent_attention": attention over a shared latent within a sliding window; "attention": attention
within blocks of positions, with normed queries and keys and a gate per head; "channel_delta": a
gated delta rule with a decay per key channel), ``mixer`` (its sizes and constants) and ``mlp``
(``kind`` "dense" with ``ff``; or null for a layer without feed-forward).  A latent-attention layer may
name an earlier one with ``kv_from``: it then reads that layer's cached rows and has no down
projection of its own.  Every size and constant is read from there; a missing or ill-typed key is an
error that names its path.  The inner sizes of a channel_delta mixer's thin matrix pairs are not
in the file: they are read off the stored tensors (``a_rank`` / ``g_rank`` may give them for models
with random weights).
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ModelConfig
from .sumozen import _plain, _section, _sizes, _take, _multiple

LATENT_KEYS = {"heads": int, "dim": int, "rot_dim": int, "vdim": int, "kv_rank": int, "q_rank": int, "scale": float}
ATTENTION_KEYS = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float}
DELTA_KEYS = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int}
LAYER_TYPES = ("attention", "channel_delta", "latent_attention")


def _mask(raw, where):
    return {"size": _take(_section(raw, "mask", where), "size", int, where + "mask.")}


def read_mixer(kind, raw, where, index, earlier):
    if kind == "latent_attention":
        sizes = _sizes(raw, LATENT_KEYS, where)
        rot = _section(raw, "rot", where)
        sizes["rot"] = {"base": _take(rot, "base", float, where + "rot."), "dims": _take(rot, "dims", int, where + "rot.")}
        if sizes["rot"]["base"] <= 1.0:
            raise ConfigError(f"config key '{where}rot.base': must be larger than 1, got {sizes['rot']['base']!r}")
        if sizes["rot"]["dims"] % 2 or sizes["rot"]["dims"] > sizes["rot_dim"]:
            raise ConfigError(f"config key '{where}rot.dims': an even number of at most rot_dim = {sizes['rot_dim']} entries "
                              f"is rotated, got {sizes['rot']['dims']}")
        sizes["mask"] = _mask(raw, where)
        if raw.get("kv_from") is not None:
            source = _take(raw, "kv_from", int, where, positive=False)
            if not 0 <= source < index or earlier[source]["type"] != "latent_attention" or "kv_from" in earlier[source]["mixer"]:
                raise ConfigError(f"config key '{where}kv_from': layer {source} is not an earlier latent_attention layer with a "
                                  f"down projection of its own")
            theirs = earlier[source]["mixer"]
            for key in ("kv_rank", "rot_dim", "rot"):
                if theirs[key] != sizes[key]:
                    raise ConfigError(f"config key '{where}{key}': {sizes[key]!r} differs from layer {source}'s {theirs[key]!r}, "
                                      f"whose cached rows this layer reads")
            sizes["kv_from"] = source
        return sizes
    if kind == "attention":
        sizes = _sizes(raw, ATTENTION_KEYS, where)
        _multiple(sizes, "heads", "kv_heads", where)
        sizes["mask"] = _mask(raw, where)
        return sizes
    sizes = _sizes(raw, DELTA_KEYS, where)
    _multiple(sizes, "heads", "kv_heads", where)
    for key in ("a_rank", "g_rank"):
        if raw.get(key) is not None:
            sizes[key] = _take(raw, key, int, where)
    return sizes


def read_mlp(raw, where):
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"config key '{where[:-1]}': expected an object or null, got {raw!r}")
    kind = _take(raw, "kind", str, where, positive=False)
    if kind != "dense":
        raise ConfigError(f"config key '{where}kind': unknown feed-forward '{kind}' (known: dense)")
    return {"kind": kind, "ff": _take(raw, "ff", int, where)}


def read_layer(raw, index: int, earlier) -> dict:
    where = f"layers[{index}]."
    if not isinstance(raw, dict):
        raise ConfigError(f"config key 'layers[{index}]': expected an object, got {raw!r}")
    kind = _take(raw, "type", str, where, positive=False)
    if kind not in LAYER_TYPES:
        raise ConfigError(f"config key '{where}type': unknown layer type '{kind}' (known: {', '.join(LAYER_TYPES)})")
    return {"type": kind, "mixer": read_mixer(kind, _section(raw, "mixer", where), where + "mixer.", index, earlier),
            "mlp": read_mlp(raw.get("mlp"), where + "mlp.")}


@dataclass(frozen=True)
class LipulornConfig(ModelConfig):
    vocab: int = field(default=0, metadata={"kind": int})
    width: int = field(default=0, metadata={"kind": int})
    streams: int = field(default=0, metadata={"kind": int})
    norm_eps: float = field(default=0.0, metadata={"kind": float})
    layers: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict, architecture: str | None = None) -> "LipulornConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError(f"config key 'layers': expected a list of layers, got {listed!r}")
        layers = []
        for index, layer in enumerate(listed):
            layers.append(read_layer(layer, index, layers))
        streams = _take(raw, "streams", int, "")
        if streams > 16:
            raise ConfigError(f"config key 'streams': at most 16 residual streams, got {streams}")
        return cls(architecture=architecture or raw.get("architecture") or "Lipulorn",
                   vocab=_take(raw, "vocab", int, ""), width=_take(raw, "width", int, ""), streams=streams,
                   norm_eps=_take(_section(raw, "norm"), "eps", float, "norm.", positive=False), layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "streams": self.streams,
                "norm": {"eps": self.norm_eps}, "layers": [_plain(layer) for layer in self.layers]}

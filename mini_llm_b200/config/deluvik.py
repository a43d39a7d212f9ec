"""Configuration of Deluvik: a stack whose layers each name their mixer, with the norm on every sublayer's output.

``config.json`` is nested: ``vocab``, ``width``, ``norm`` (``eps``), ``logit_softcap`` (optional) and ``layers``, a list
whose entries give ``type``, ``mixer`` (its sizes and constants) and ``mlp``:

* ``type`` "attention": ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` (``base``, ``dims``, optional ``scaling``
  with ``factor``, ``low``, ``high``, ``original``), optional ``softcap``; the values are the keys as projected, so
  ``vdim`` equals ``dim``;
* ``type`` "attention_2": the same keys, plus ``conv`` (taps of the short convolution on q, k and v) and optionally
  ``kv_from`` (an earlier attention layer whose keys and values this layer reads instead of its own);
* ``type`` "parallel": ``left`` (an attention with ``mask.size``, the sliding window), ``right`` (``width``, ``blocks``,
  ``conv``: the gated linear recurrence), ``left_scale`` and ``right_scale``;
* ``mlp``: null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"},
  "shared": {"ff"} or null}``.

Every size and constant is read from there; a missing or ill-typed key is an error that names its path.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ModelConfig
from .sumozen import _multiple, _plain, _section, _sizes, _take

ATTENTION_KEYS = {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float}
RIGHT_KEYS = {"width": int, "blocks": int, "conv": int}
SCALING_KEYS = ("factor", "low", "high", "original")
LAYER_TYPES = ("attention", "attention_2", "parallel")


def _optional(raw, key, kind, where):
    return _take(raw, key, kind, where) if raw.get(key) is not None else None


def read_rotation(raw, where, dim):
    rot = {"base": _take(raw, "base", float, where), "dims": _take(raw, "dims", int, where, positive=False)}
    if rot["base"] <= 1.0:
        raise ConfigError(f"config key '{where}base': must be larger than 1, got {rot['base']!r}")
    if rot["dims"] < 0 or rot["dims"] % 2 or rot["dims"] > dim:
        raise ConfigError(f"config key '{where}dims': an even number of at most dim = {dim} entries is rotated, "
                          f"got {rot['dims']}")
    scaling = raw.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, dict):
            raise ConfigError(f"config key '{where}scaling': expected an object or null, got {scaling!r}")
        rot["scaling"] = {key: _take(scaling, key, float, where + "scaling.") for key in SCALING_KEYS}
        if rot["scaling"]["high"] <= rot["scaling"]["low"]:
            raise ConfigError(f"config key '{where}scaling.high': must lie above scaling.low = {rot['scaling']['low']!r}")
    else:
        rot["scaling"] = None
    return rot


def read_attention(raw, where):
    """The keys every attention of the design has; ``softcap``, ``conv``, ``mask`` and ``kv_from`` where given."""
    sizes = _sizes(raw, ATTENTION_KEYS, where)
    _multiple(sizes, "heads", "kv_heads", where)
    sizes["rot"] = read_rotation(_section(raw, "rot", where), where + "rot.", sizes["dim"])
    sizes["softcap"] = _optional(raw, "softcap", float, where)
    sizes["conv"] = _optional(raw, "conv", int, where)
    mask = raw.get("mask")
    if mask is not None:
        sizes["mask"] = {"size": _take(_section(raw, "mask", where), "size", int, where + "mask.")}
    else:
        sizes["mask"] = None
    if raw.get("kv_from") is not None:
        sizes["kv_from"] = _take(raw, "kv_from", int, where, positive=False)
    return sizes


def read_mixer(kind, raw, where):
    if kind == "parallel":
        left = read_attention(_section(raw, "left", where), where + "left.")
        right = _sizes(_section(raw, "right", where), RIGHT_KEYS, where + "right.")
        if right["width"] % right["blocks"] != 0:
            raise ConfigError(f"config key '{where}right.blocks': {right['width']} channels do not split into "
                              f"{right['blocks']} equal parts")
        return {"left": left, "right": right,
                "left_scale": _take(raw, "left_scale", float, where, positive=False),
                "right_scale": _take(raw, "right_scale", float, where, positive=False)}
    sizes = read_attention(raw, where)
    if kind == "attention" and sizes["vdim"] != sizes["dim"]:
        raise ConfigError(f"config key '{where}vdim': the values of this mixer are its keys, so vdim must equal dim = "
                          f"{sizes['dim']}, got {sizes['vdim']}")
    if kind == "attention_2" and sizes["conv"] is None:
        raise ConfigError(f"config key '{where}conv' is missing")
    return sizes


def read_mlp(raw, where):
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"config key '{where[:-1]}': expected an object or null, got {raw!r}")
    kind = _take(raw, "kind", str, where, positive=False)
    if kind == "dense":
        return {"kind": kind, "ff": _take(raw, "ff", int, where)}
    if kind != "moe":
        raise ConfigError(f"config key '{where}kind': unknown feed-forward '{kind}' (known: dense, moe)")
    router = _section(raw, "router", where)
    mlp = {"kind": kind,
           "router": {"experts": _take(router, "experts", int, where + "router."), "top": _take(router, "top", int, where + "router.")},
           "expert": {"ff": _take(_section(raw, "expert", where), "ff", int, where + "expert.")}}
    if mlp["router"]["top"] > mlp["router"]["experts"]:
        raise ConfigError(f"config key '{where}router.top': {mlp['router']['top']} of {mlp['router']['experts']} experts")
    shared = raw.get("shared")
    if shared is not None:
        if not isinstance(shared, dict):
            raise ConfigError(f"config key '{where}shared': expected an object or null, got {shared!r}")
        mlp["shared"] = {"ff": _take(shared, "ff", int, where + "shared.")}
    else:
        mlp["shared"] = None
    return mlp


def read_layer(raw, index: int) -> dict:
    where = f"layers[{index}]."
    if not isinstance(raw, dict):
        raise ConfigError(f"config key 'layers[{index}]': expected an object, got {raw!r}")
    kind = _take(raw, "type", str, where, positive=False)
    if kind not in LAYER_TYPES:
        raise ConfigError(f"config key '{where}type': unknown layer type '{kind}' (known: {', '.join(LAYER_TYPES)})")
    return {"type": kind, "mixer": read_mixer(kind, _section(raw, "mixer", where), where + "mixer."),
            "mlp": read_mlp(raw.get("mlp"), where + "mlp.")}


def check_shared_rows(layers) -> None:
    """A layer with ``kv_from`` names an earlier attention layer that has keys and values of its own, with the same
    key/value heads and sizes (what the shared pages must agree on)."""
    for index, layer in enumerate(layers):
        source = layer["mixer"].get("kv_from") if layer["type"] != "parallel" else None
        if source is None:
            continue
        where = f"layers[{index}].mixer.kv_from"
        if not 0 <= source < index:
            raise ConfigError(f"config key '{where}': {source} is not an earlier layer")
        other = layers[source]
        if other["type"] == "parallel" or other["mixer"].get("kv_from") is not None:
            raise ConfigError(f"config key '{where}': layer {source} is not an attention layer with keys and values of its own")
        for key in ("kv_heads", "dim", "vdim"):
            if other["mixer"][key] != layer["mixer"][key]:
                raise ConfigError(f"config key '{where}': layer {source} has another '{key}' ({other['mixer'][key]!r}) than this "
                                  f"layer ({layer['mixer'][key]!r})")


@dataclass(frozen=True)
class DeluvikConfig(ModelConfig):
    vocab: int = field(default=0, metadata={"kind": int})
    width: int = field(default=0, metadata={"kind": int})
    norm_eps: float = field(default=0.0, metadata={"kind": float})
    logit_softcap: float | None = None
    layers: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict, architecture: str | None = None) -> "DeluvikConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"config key 'layers': expected a list of layers, got {layers!r}")
        read = tuple(read_layer(layer, index) for index, layer in enumerate(layers))
        check_shared_rows(read)
        return cls(architecture=architecture or raw.get("architecture") or "Deluvik",
                   vocab=_take(raw, "vocab", int, ""), width=_take(raw, "width", int, ""),
                   norm_eps=_take(_section(raw, "norm"), "eps", float, "norm.", positive=False),
                   logit_softcap=_optional(raw, "logit_softcap", float, ""), layers=read)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [_drop_absent(_plain(layer)) for layer in self.layers]}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out


def _drop_absent(value):
    """Optional keys that the file did not give are not written back (``mlp`` and ``shared`` may be null by themselves)."""
    if isinstance(value, dict):
        return {key: _drop_absent(one) for key, one in value.items() if one is not None or key in ("mlp", "shared")}
    return value

"""Deluvik as a model description.

A decoder-only stack with the norm on every sublayer's output: ``x <- x + norm1(mixer(x))``, then, if the layer has
one, ``x <- x + norm2(ff(x))``; the sublayers read the stream itself, and every norm divides by the root mean square
and multiplies by its weight.  A layer names its mixer.  "attention": queries and keys normed over their whole
projection, rotary positions on pairs half apart (frequencies scaled by bands of their wavelength where the
configuration says so), capped scores, a sink in the softmax, and the keys as projected for values.  "attention_2":
projections of q, k and v through a short causal convolution, the same norm and rotation, a sink; with ``kv_from``
the layer reads an earlier such layer's cached keys and values with queries of its own.  "parallel": a sliding-window
attention (queries and keys normed per head, neighbouring pairs rotated) beside a real-gated linear recurrent unit,
added with a scale each.  The feed-forward is ``W_down (gelu(W_gate x) * (W_up x))`` or a mixture of experts whose
chosen experts' outputs are weighed by the softmax over the chosen logits, with a shared expert.  The logits are capped.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*`` (``left.*`` /
``right.*`` in a parallel layer) and ``l<i>.mlp.*``; matrices are stored [out, in].
"""

from __future__ import annotations

from ..config.deluvik import DeluvikConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

DECAY_SCALE = 8.0          # log a = -8 * r * softplus(lam) in the recurrent unit


def _attention(sizes: dict, prefix: str, width: int, eps: float, norm: str, layout: str, values: str, sink: bool) -> PartSpec:
    rot = sizes["rot"]
    rotation = PartSpec("banded_rotary", prefix, {
        "base": rot["base"], "dims": rot["dims"], "layout": layout,
        "scaling": tuple(sorted(rot["scaling"].items())) if rot["scaling"] else None})
    return PartSpec("normed_attention", prefix, {
        "width": width, "n_heads": sizes["heads"], "n_kv_heads": sizes["kv_heads"], "key_size": sizes["dim"],
        "value_size": sizes["vdim"], "score_scale": sizes["scale"], "eps": eps, "position": rotation, "norm": norm,
        "values": values, "taps": sizes["conv"], "softcap": sizes["softcap"],
        "window": sizes["mask"]["size"] if sizes["mask"] else None, "sink": sink, "own_kv": sizes.get("kv_from") is None})


def _mixer(layer: dict, prefix: str, width: int, eps: float) -> PartSpec:
    kind, sizes = layer["type"], layer["mixer"]
    if kind == "attention":
        return _attention(sizes, prefix, width, eps, "whole", "half", "keys", True)
    if kind == "attention_2":
        return _attention(sizes, prefix, width, eps, "whole", "half", "projected", True)
    right = sizes["right"]
    left = _attention(sizes["left"], f"{prefix}.left", width, eps, "head", "interleaved", "projected", False)
    unit = PartSpec("gated_linear_recurrence", f"{prefix}.right", {
        "width": width, "inner": right["width"], "blocks": right["blocks"], "taps": right["conv"], "decay_scale": DECAY_SCALE})
    return PartSpec("parallel_mixers", prefix, {
        "branches": (("left", left, sizes["left_scale"]), ("right", unit, sizes["right_scale"]))})


def _feed_forward(mlp: dict, prefix: str, width: int) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", prefix, {"width": width, "inner": mlp["ff"], "activation": "gelu_tanh", "bias": False})
    return PartSpec("routed_experts", prefix, {
        "width": width, "n_experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "expert_inner": mlp["expert"]["ff"],
        "shared_inner": mlp["shared"]["ff"] if mlp["shared"] else None, "weights": "softmax_of_chosen", "router_bias": True,
        "shared_gate": False})


def describe(config: DeluvikConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps

    def norm(prefix, name):
        return PartSpec("grouped_rms_norm", prefix, {"width": width, "eps": eps, "groups": 1, "name": name})

    layers, order = [], []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}"
        parts = {"mixer": _mixer(layer, f"{prefix}.mix", width, eps), "norm_1": norm(prefix, "norm1")}
        if layer["mlp"] is not None:
            parts["feed_forward"] = _feed_forward(layer["mlp"], f"{prefix}.mlp", width)
            parts["norm_2"] = norm(prefix, "norm2")
        layers.append(LayerSpec("output_norm", parts))
        order.append(RunEntry(index, layer["mixer"].get("kv_from") if layer["type"] != "parallel" else None))
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=None,
        embedding=PartSpec("token_embedding", "", {"vocab_size": config.vocab, "width": width, "name": "embed"}),
        position=None,
        layers=tuple(layers),
        order=tuple(order),
        final_norm=norm("final", "norm"),
        head=PartSpec("linear_head", "", {"vocab_size": config.vocab, "width": width, "weight_name": "head",
                                          "softcap": config.logit_softcap}),
        # a layer without feed-forward has no use for a second norm, should a file hold one
        ignored_weights=tuple(rf"l{index}\.norm2" for index, layer in enumerate(config.layers) if layer["mlp"] is None),
    )


register_architecture("Deluvik", DeluvikConfig, describe)

"""Lipulorn as a model description.

A decoder-only pre-norm stack over ``streams`` residual streams (hyper-connections): every sublayer
reads a weighted sum of the streams through its RMS norm (``x / sqrt(mean(x^2) + eps) * w``) and writes
its result back onto all streams through a mixing matrix; the model's residual is the sum of the
streams.  A layer names its mixer: "latent_attention" (attention over a shared latent, queries through
a latent of their own, rotary positions on halves-apart pairs of the shared key part, a sliding
window; with ``kv_from`` it reads an earlier layer's cached rows), "attention" (biased projections,
queries and keys over their root mean square per head, no positions, a mask of blocks of positions,
a sigmoid gate per head) or "channel_delta" (a gated delta rule with a decay per key channel).  The
feed-forward is ``W_down (silu(W_gate x) * (W_up x))`` with biases.  The head has a matrix of its own.

Tensor names: ``embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.hc1.*`` / ``l<i>.hc2.*`` (``in``, ``out``, ``mix``), ``l<i>.mix.*`` and ``l<i>.mlp.*``; matrices
are stored [out, in].
"""

from __future__ import annotations

from ..config.lipulorn import LipulornConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer(layer: dict, prefix: str, width: int, eps: float, keep: int | None) -> PartSpec:
    kind, sizes = layer["type"], layer["mixer"]
    if kind == "latent_attention":
        return PartSpec("latent_attention", prefix, {
            "width": width, "n_heads": sizes["heads"], "head_size": sizes["dim"], "rotated_size": sizes["rot_dim"],
            "value_size": sizes["vdim"], "latent_size": sizes["kv_rank"], "score_scale": sizes["scale"],
            "rotary_base": sizes["rot"]["base"], "rotary_dims": sizes["rot"]["dims"], "eps": eps,
            "window": sizes["mask"]["size"], "keep": keep, "rotary_layout": "half", "query_rank": sizes["q_rank"],
            "own_rows": "kv_from" not in sizes})
    if kind == "attention":
        return PartSpec("gated_attention", prefix, {
            "width": width, "n_heads": sizes["heads"], "n_kv_heads": sizes["kv_heads"], "key_size": sizes["dim"],
            "value_size": sizes["vdim"], "score_scale": sizes["scale"], "head_norm_eps": eps,
            "chunk": sizes["mask"]["size"], "gate": True, "bias": True})
    return PartSpec("channel_delta_memory", prefix, {
        "width": width, "n_heads": sizes["heads"], "n_qk_heads": sizes["kv_heads"], "key_size": sizes["dim"],
        "value_size": sizes["vdim"], "taps": sizes["conv"], "eps": eps, "step_rank": sizes.get("a_rank"),
        "gate_rank": sizes.get("g_rank")})


def describe(config: LipulornConfig) -> ModelSpec:
    width, eps, streams = config.width, config.norm_eps, config.streams

    def norm(prefix, name):
        return PartSpec("grouped_rms_norm", prefix, {"width": width, "eps": eps, "groups": 1, "name": name})

    # a layer whose rows other layers read keeps them as long as the widest of their windows
    keep = {}
    for index, layer in enumerate(config.layers):
        if layer["type"] == "latent_attention":
            owner = layer["mixer"].get("kv_from", index)
            keep[owner] = max(keep.get(owner, 0), layer["mixer"]["mask"]["size"])
    layers, order = [], []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}"
        parts = {"streams_1": PartSpec("stream_connection", f"{prefix}.hc1", {"n_streams": streams}),
                 "norm_1": norm(prefix, "norm1"),
                 "mixer": _mixer(layer, f"{prefix}.mix", width, eps, keep.get(index))}
        mlp = layer["mlp"]
        if mlp is not None:
            parts["streams_2"] = PartSpec("stream_connection", f"{prefix}.hc2", {"n_streams": streams})
            parts["norm_2"] = norm(prefix, "norm2")
            parts["feed_forward"] = PartSpec("gated_mlp", f"{prefix}.mlp", {"width": width, "inner": mlp["ff"],
                                                                          "activation": "silu", "bias": True})
        layers.append(LayerSpec("hyper_connections", parts))
        order.append(RunEntry(index, layer["mixer"].get("kv_from")))
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab,
        max_positions=None,
        embedding=PartSpec("token_embedding", "", {"vocab_size": config.vocab, "width": width, "name": "embed"}),
        position=None,
        layers=tuple(layers),
        order=tuple(order),
        final_norm=norm("final", "norm"),
        head=PartSpec("linear_head", "", {"vocab_size": config.vocab, "width": width, "weight_name": "head"}),
        residual_streams=streams,
        # a layer without feed-forward has no use for a second norm or connection, should a file hold them
        ignored_weights=tuple(rf"l{index}\.(norm2|hc2\..*)" for index, layer in enumerate(config.layers) if layer["mlp"] is None),
    )


register_architecture("Lipulorn", LipulornConfig, describe)

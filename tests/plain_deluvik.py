"""A plain, slow Deluvik in numpy float64: one function per mechanism, token by token where the
mechanism is a recurrence.  It shares nothing with the package: the tests compare the engine
with it.  ``config`` is the nested dictionary of the model's ``config.json``; ``weights`` maps
tensor names to float64 arrays."""

from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, w, eps):
    """Rows over their root mean square (eps inside the root), times w."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def causal_taps(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    n, taps = u.shape[0], w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u])
    y = np.zeros_like(u)
    for j in range(taps):
        y += padded[j:j + n] * w[:, j]
    return y if bias is None else y + bias


def frequencies(rot):
    """f_i = base^(-2i/dims); with ``scaling`` (factor, low, high, original) a pair whose wavelength
    is shorter than original/high keeps f, one longer than original/low gets f / factor, and between
    the two the frequencies are blended."""
    dims, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    scaling = rot.get("scaling")
    if not scaling:
        return f
    factor, low, high, original = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out[i] = fi
        elif wavelength > original / low:
            out[i] = fi / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x, positions, rot, layout):
    """x [T, heads, size]: among the first rot.dims entries of every head, pair i turns by
    position * f_i; the pair is (i, i + dims/2) in the "half" layout and (2i, 2i+1) in the
    "interleaved" one."""
    dims = rot["dims"]
    if dims == 0:
        return x
    half = dims // 2
    angle = np.asarray(positions, dtype=np.float64)[:, None] * frequencies(rot)[None, :]
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    out = x.copy()
    if layout == "half":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half], out[..., half:dims] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * c - v * s, v * c + u * s
    return out


def attend(q, k, v, scale, softcap=None, window=None, sink=None, first_position=0):
    """q [T, H, dim], k [S, G, dim], v [S, G, vdim]; query t stands at position first_position + t
    and key j at position j.  Head h reads key/value head h // (H / G).  The softmax's denominator
    also holds exp(sink[h]) if there is a sink."""
    n, heads, _ = q.shape
    group = heads // k.shape[1]
    out = np.zeros((n, heads, v.shape[2]))
    for t in range(n):
        p = first_position + t
        lo = 0 if window is None else max(0, p - window + 1)
        for h in range(heads):
            score = k[lo:p + 1, h // group] @ q[t, h] * scale
            if softcap:
                score = softcap * np.tanh(score / softcap)
            top = score.max() if sink is None else max(score.max(), sink[h])
            e = np.exp(score - top)
            denominator = e.sum() + (np.exp(sink[h] - top) if sink is not None else 0.0)
            out[t, h] = (e / denominator) @ v[lo:p + 1, h // group]
    return out


def whole_norm_attention(x, sizes, w, prefix, eps, kv=None, convolved=False):
    """The mixers "attention" and "attention_2": query and key norm over the whole projection, pairs
    half apart, a sink.  "attention": values are the keys as projected; a cap on the scores.
    "attention_2" (``convolved``): projections of q, k and v, each through a short convolution;
    with ``kv`` (another layer's rotated keys and its values) no keys and values of its own.
    Returns (output [T, width], keys, values)."""
    n = x.shape[0]
    heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    positions = np.arange(n)
    q = x @ w[f"{prefix}.q"].T
    if convolved:
        q = causal_taps(q, w[f"{prefix}.q.conv"])
    q = rms_norm(q, w[f"{prefix}.q.norm"], eps).reshape(n, heads, dim)
    q = rotate(q, positions, sizes["rot"], "half")
    if kv is None:
        k = x @ w[f"{prefix}.k"].T
        if convolved:
            k = causal_taps(k, w[f"{prefix}.k.conv"])
            v = causal_taps(x @ w[f"{prefix}.v"].T, w[f"{prefix}.v.conv"])
        else:
            v = k
        v = v.reshape(n, groups, vdim)
        k = rms_norm(k, w[f"{prefix}.k.norm"], eps).reshape(n, groups, dim)
        k = rotate(k, positions, sizes["rot"], "half")
    else:
        k, v = kv
    mixed = attend(q, k, v, sizes["scale"], sizes.get("softcap"), None, w[f"{prefix}.sink"])
    return mixed.reshape(n, heads * vdim) @ w[f"{prefix}.o"].T, k, v


def windowed_attention(x, sizes, w, prefix, eps):
    """The left side of a parallel layer: q, k, v projections, query and key norm per head with one
    weight of the head's size, neighbouring pairs, a sliding window, ordinary softmax."""
    n = x.shape[0]
    heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    positions = np.arange(n)
    q = rms_norm((x @ w[f"{prefix}.q"].T).reshape(n, heads, dim), w[f"{prefix}.q.norm"], eps)
    k = rms_norm((x @ w[f"{prefix}.k"].T).reshape(n, groups, dim), w[f"{prefix}.k.norm"], eps)
    v = (x @ w[f"{prefix}.v"].T).reshape(n, groups, vdim)
    q, k = rotate(q, positions, sizes["rot"], "interleaved"), rotate(k, positions, sizes["rot"], "interleaved")
    window = sizes["mask"]["size"] if sizes.get("mask") else None
    mixed = attend(q, k, v, sizes["scale"], None, window, None)
    return mixed.reshape(n, heads * vdim) @ w[f"{prefix}.o"].T


def gated_linear_unit(x, sizes, w, prefix):
    """The right side: y = gelu(W_y x + b), u = conv(W_x x + b); per block of channels
    r = sigmoid(ra u + b), i = sigmoid(ri u + b); a = exp(-8 r softplus(lam));
    S_t = a S_(t-1) + sqrt(1 - a^2) i u, from S = 0; output W_o (S y)."""
    n, blocks, width = x.shape[0], sizes["blocks"], sizes["width"]
    y = gelu_tanh(x @ w[f"{prefix}.y"].T + w[f"{prefix}.y.b"])
    u = causal_taps(x @ w[f"{prefix}.x"].T + w[f"{prefix}.x.b"], w[f"{prefix}.conv"], w[f"{prefix}.conv.b"])
    part = width // blocks
    r, i = np.zeros_like(u), np.zeros_like(u)
    for b in range(blocks):
        cut = slice(b * part, (b + 1) * part)
        r[:, cut] = sigmoid(u[:, cut] @ w[f"{prefix}.ra"][b].T + w[f"{prefix}.ra.b"][b])
        i[:, cut] = sigmoid(u[:, cut] @ w[f"{prefix}.ri"][b].T + w[f"{prefix}.ri.b"][b])
    state = np.zeros(width)
    out = np.zeros_like(u)
    for t in range(n):
        a = np.exp(-8.0 * r[t] * softplus(w[f"{prefix}.lam"]))
        state = a * state + np.sqrt(1.0 - a * a) * i[t] * u[t]
        out[t] = state
    return (out * y) @ w[f"{prefix}.o"].T


def gated_expert(x, w, prefix, act):
    return (act(x @ w[f"{prefix}.gate"].T) * (x @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


def feed_forward(x, mlp, w, prefix):
    if mlp["kind"] == "dense":
        return gated_expert(x, w, prefix, gelu_tanh)
    top = mlp["router"]["top"]
    logits = x @ w[f"{prefix}.router"].T + w[f"{prefix}.router.b"]
    out = np.zeros_like(x)
    for t in range(x.shape[0]):
        chosen = np.argsort(-logits[t], kind="stable")[:top]
        weight = np.exp(logits[t, chosen] - logits[t, chosen].max())
        weight /= weight.sum()
        for e, g in zip(chosen, weight):
            out[t] += g * gated_expert(x[t:t + 1], w, f"{prefix}.e{e}", silu)[0]
    if mlp.get("shared"):
        out += gated_expert(x, w, f"{prefix}.shared", silu)
    return out


def forward(config, w, tokens, keep_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer)."""
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    kept, cached = [], {}
    for index, layer in enumerate(config["layers"]):
        prefix, sizes, kind = f"l{index}", layer["mixer"], layer["type"]
        if kind == "parallel":
            mixed = (sizes["left_scale"] * windowed_attention(x, sizes["left"], w, f"{prefix}.mix.left", eps)
                     + sizes["right_scale"] * gated_linear_unit(x, sizes["right"], w, f"{prefix}.mix.right"))
        else:
            source = sizes.get("kv_from")
            mixed, k, v = whole_norm_attention(x, sizes, w, f"{prefix}.mix", eps, cached[source] if source is not None else None,
                                               convolved=kind == "attention_2")
            cached[index] = (k, v)
        x = x + rms_norm(mixed, w[f"{prefix}.norm1"], eps)
        if layer["mlp"] is not None:
            x = x + rms_norm(feed_forward(x, layer["mlp"], w, f"{prefix}.mlp"), w[f"{prefix}.norm2"], eps)
        kept.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, kept) if keep_layers else logits


def load_model(folder):
    """(config dictionary, {name: float64 array}) of a model folder; its own small safetensors reader."""
    import json
    import os
    import struct

    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    with open(os.path.join(folder, "model.safetensors"), "rb") as handle:
        data = handle.read()
    (length,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + length])
    body = data[8 + length:]
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        if info["dtype"] == "F32":
            values = np.frombuffer(body[begin:end], dtype="<f4").astype(np.float64)
        elif info["dtype"] == "BF16":
            values = (np.frombuffer(body[begin:end], dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        else:
            raise ValueError(f"{name}: element type {info['dtype']}")
        tensors[name] = values.reshape(info["shape"])
    return config, tensors

"""A plain, slow Lipulorn in numpy float64: one function per mechanism, token by token where the
mechanism is a recurrence.  It shares nothing with the package: the tests compare the engine
with it.  ``config`` is the nested dictionary of the model's ``config.json``; ``weights`` maps
tensor names to float64 arrays."""

from __future__ import annotations

import json
import os
import struct

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, w, eps):
    """Rows over their root mean square (eps inside the root), times w."""
    y = x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def softmax_rows(score, visible):
    score = np.where(visible, score, -np.inf)
    p = np.exp(score - score.max(axis=1, keepdims=True))
    return p / p.sum(axis=1, keepdims=True)


def causal_taps(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    n, taps = u.shape[0], w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u])
    y = np.zeros_like(u)
    for j in range(taps):
        y += padded[j:j + n] * w[:, j]
    return y


def rotate_half(x, positions, base, dims):
    """x [T, heads, size]: entry i and entry i + dims/2 (i < dims/2) turn by position * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half, dtype=np.float64) / dims)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


def window_mask(n, size):
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    return (i - j >= 0) & (i - j < size)


def chunk_mask(n, size):
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    return (j <= i) & (i // size == j // size)


def latent_kv(h, sizes, w, prefix, eps):
    """What a latent-attention layer caches: the normed latent [T, rank] and the rotated shared key part [T, rot]."""
    n, rank, rot = h.shape[0], sizes["kv_rank"], sizes["rot_dim"]
    down = h @ w[f"{prefix}.dkv"].T
    c = rms_norm(down[:, :rank], w[f"{prefix}.dkv.norm"], eps)
    shared = rotate_half(down[:, None, rank:rank + rot], np.arange(n), sizes["rot"]["base"], sizes["rot"]["dims"])[:, 0]
    return c, shared


def latent_attention(h, sizes, w, prefix, eps, kv):
    n = h.shape[0]
    heads, dim, rot, vdim, rank = sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"]
    c, shared = kv
    cq = rms_norm(h @ w[f"{prefix}.dq"].T, w[f"{prefix}.dq.norm"], eps)
    q = (cq @ w[f"{prefix}.uq"].T).reshape(n, heads, dim + rot)
    q_plain = q[..., :dim]
    q_rot = rotate_half(q[..., dim:], np.arange(n), sizes["rot"]["base"], sizes["rot"]["dims"])
    k_plain = (c @ w[f"{prefix}.uk"].T).reshape(n, heads, dim)
    v = (c @ w[f"{prefix}.uv"].T).reshape(n, heads, vdim)
    visible = window_mask(n, sizes["mask"]["size"])
    out = np.zeros((n, heads, vdim))
    for head in range(heads):
        score = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ shared.T) * sizes["scale"]
        out[:, head] = softmax_rows(score, visible) @ v[:, head]
    return out.reshape(n, heads * vdim) @ w[f"{prefix}.o"].T


def chunked_attention(h, sizes, w, prefix, eps):
    n = h.shape[0]
    heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    q = (h @ w[f"{prefix}.q"].T + w[f"{prefix}.q.b"]).reshape(n, heads, dim)
    k = (h @ w[f"{prefix}.k"].T + w[f"{prefix}.k.b"]).reshape(n, groups, dim)
    v = (h @ w[f"{prefix}.v"].T + w[f"{prefix}.v.b"]).reshape(n, groups, vdim)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    gate = sigmoid(h @ w[f"{prefix}.g"].T)
    visible = chunk_mask(n, sizes["mask"]["size"])
    out = np.zeros((n, heads, vdim))
    for head in range(heads):
        g = head // (heads // groups)
        score = (q[:, head] @ k[:, g].T) * sizes["scale"]
        out[:, head] = (softmax_rows(score, visible) @ v[:, g]) * gate[:, head:head + 1]
    return out.reshape(n, heads * vdim) @ w[f"{prefix}.o"].T


def channel_delta(h, sizes, w, prefix, eps):
    """S <- g S (g per key channel); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    n = h.shape[0]
    heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    q = silu(causal_taps(h @ w[f"{prefix}.q"].T, w[f"{prefix}.q.conv"])).reshape(n, groups, dim)
    k = silu(causal_taps(h @ w[f"{prefix}.k"].T, w[f"{prefix}.k.conv"])).reshape(n, groups, dim)
    v = silu(causal_taps(h @ w[f"{prefix}.v"].T, w[f"{prefix}.v.conv"])).reshape(n, heads, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[f"{prefix}.b"].T)
    step = softplus((h @ w[f"{prefix}.a1"].T) @ w[f"{prefix}.a2"].T + w[f"{prefix}.dt_bias"]).reshape(n, heads, dim)
    decay = np.exp(-np.exp(w[f"{prefix}.A_log"])[None, :, None] * step)
    gate = sigmoid((h @ w[f"{prefix}.g1"].T) @ w[f"{prefix}.g2"].T).reshape(n, heads, vdim)
    state = np.zeros((heads, dim, vdim))
    out = np.zeros((n, heads, vdim))
    for t in range(n):
        for head in range(heads):
            g = head // (heads // groups)
            s = state[head] * decay[t, head][:, None]
            u = beta[t, head] * (v[t, head] - s.T @ k[t, g])
            s = s + np.outer(k[t, g], u)
            state[head] = s
            out[t, head] = s.T @ q[t, g]
    out = rms_norm(out, w[f"{prefix}.norm"], eps) * gate
    return out.reshape(n, heads * vdim) @ w[f"{prefix}.o"].T


def gated_mlp(h, w, prefix):
    gate = h @ w[f"{prefix}.gate"].T + w[f"{prefix}.gate.b"]
    up = h @ w[f"{prefix}.up"].T + w[f"{prefix}.up.b"]
    return (silu(gate) * up) @ w[f"{prefix}.down"].T + w[f"{prefix}.down.b"]


def hyper_read(streams, w, prefix):
    """streams [s, T, width] -> sum_s in[s] x_s."""
    return np.tensordot(w[f"{prefix}.in"], streams, axes=(0, 0))


def hyper_write(streams, y, w, prefix):
    """All streams at once from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y."""
    mixed = np.tensordot(w[f"{prefix}.mix"].T, streams, axes=(1, 0))
    return mixed + w[f"{prefix}.out"][:, None, None] * y[None]


def forward(config, w, tokens, layer_results=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layer_results``: a list that gets the
    sum of the streams after every layer."""
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    streams = np.repeat(x[None], config["streams"], axis=0)
    kept = {}
    for index, layer in enumerate(config["layers"]):
        p, sizes = f"l{index}", layer["mixer"]
        h = rms_norm(hyper_read(streams, w, f"{p}.hc1"), w[f"{p}.norm1"], eps)
        if layer["type"] == "latent_attention":
            source = sizes.get("kv_from")
            if source is None:
                kept[index] = latent_kv(h, sizes, w, f"{p}.mix", eps)
                source = index
            y = latent_attention(h, sizes, w, f"{p}.mix", eps, kept[source])
        elif layer["type"] == "attention":
            y = chunked_attention(h, sizes, w, f"{p}.mix", eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta(h, sizes, w, f"{p}.mix", eps)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        streams = hyper_write(streams, y, w, f"{p}.hc1")
        if layer.get("mlp") is not None:
            h = rms_norm(hyper_read(streams, w, f"{p}.hc2"), w[f"{p}.norm2"], eps)
            streams = hyper_write(streams, gated_mlp(h, w, f"{p}.mlp"), w, f"{p}.hc2")
        if layer_results is not None:
            layer_results.append(streams.sum(axis=0))
    x = rms_norm(streams.sum(axis=0), w["final.norm"], eps)
    return x @ w["head"].T


def read_safetensors(path):
    """name -> float64 array (F32, BF16 and I32 tensors)."""
    with open(path, "rb") as handle:
        (size,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(size))
        data = handle.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            values = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            values = np.frombuffer(raw, dtype="<f4")
        elif info["dtype"] == "I32":
            values = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{name}: element type {info['dtype']} is not read here")
        out[name] = values.astype(np.float64).reshape(info["shape"])
    return out


def load_model(folder):
    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    return config, read_safetensors(os.path.join(folder, "model.safetensors"))

"""Rotary positions in the interleaved layout, with optional YaRN scaling of the frequencies.

Among the first ``dims`` entries of every query and key head, entries 2i and 2i+1 form a pair that
turns by ``position * f_i``, ``f_i = base^(-2i/dims)``; the rest pass unchanged.  With ``scaling``
(``factor``, ``original``, ``fast``, ``slow``) the frequencies are blended: with
``at(t) = dims * ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(at(fast)), 0)``,
``hi = min(ceil(at(slow)), dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``
the frequency is ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``, and cosine and sine are both
multiplied by ``0.1 * ln(factor) + 1``.  The table of frequencies is 64-bit, made once; the angle
and its cosine and sine are taken in 64-bit per token and rounded to 32-bit once.

The encoding is a parameter of a mixer.  ``rotate_store`` turns the queries and keys of a step in
place and writes the keys and values into their cache pages in the same pass.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_part


def rotary_frequencies(base: float, dims: int, scaling: dict | None = None):
    """(frequencies as a list of dims / 2 floats, amplitude)."""
    half = dims // 2
    plain = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return plain, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def at(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(at(float(scaling["fast"]))), 0)
    hi = min(math.ceil(at(float(scaling["slow"]))), dims - 1)
    span = max(hi - lo, 0.001)
    blended = []
    for i, f in enumerate(plain):
        ramp = min(max((i - lo) / span, 0.0), 1.0)
        blended.append(f / factor * ramp + f * (1.0 - ramp))
    return blended, 0.1 * math.log(factor) + 1.0


class InterleavedRotary(PositionEncoding):
    graph_safe = True

    def __init__(self, prefix, base: float, dims: int, scaling: dict | None = None):
        super().__init__(prefix)
        self.base, self.dims = float(base), int(dims)
        self.scaling = dict(scaling) if scaling else None
        if self.dims < 0 or self.dims % 2 != 0:
            raise ValueError(f"{prefix}: an even number of entries is rotated, got {self.dims}")
        if self.base <= 1.0:
            raise ValueError(f"{prefix}: the rotary base must be larger than 1")
        if self.scaling is not None:
            for key in ("factor", "original", "fast", "slow"):
                if key not in self.scaling or float(self.scaling[key]) <= 0:
                    raise ValueError(f"{prefix}: the scaling needs a positive '{key}'")
        self.frequencies, self.amplitude = rotary_frequencies(self.base, self.dims, self.scaling) if self.dims else ([], 1.0)
        self.inv_freq = None

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        device = runtime.device if runtime is not None else "cuda"
        self.inv_freq = torch.tensor(self.frequencies or [0.0], dtype=torch.float64, device=device)

    def rotate_store(self, ctx, cache, qkv, k_off, v_off, n_heads, n_kv_heads, key_size, value_size):
        if self.dims > key_size:
            raise ValueError(f"{self.prefix}: {self.dims} rotated entries do not fit a head of {key_size}")
        ctx.kernels.rotary_store(ctx, cache, qkv, k_off, v_off, n_heads, n_kv_heads, key_size, value_size, self.dims,
                                 self.inv_freq, self.amplitude)


def banded_frequencies(base: float, dims: int, scaling: dict | None = None):
    """dims / 2 frequencies ``f_i = base^(-2i/dims)``; with ``scaling`` (``factor``, ``low``, ``high``, ``original``)
    by bands of the wavelength ``l = 2 pi / f`` (the rule of Llama 3.1): ``f`` stays where ``l < original / high``,
    becomes ``f / factor`` where ``l > original / low``, and between the two, with
    ``s = (original / l - low) / (high - low)``, ``(1 - s) f / factor + s f``."""
    plain = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return plain
    factor, low, high, original = (float(scaling[key]) for key in ("factor", "low", "high", "original"))
    out = []
    for f in plain:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


class BandedRotary(PositionEncoding):
    """Rotary positions on the first ``dims`` entries of every query and key head, pair i turning by
    ``position * f_i``; ``layout`` says which entries form pair i: 2i and 2i+1 ("interleaved") or i and
    i + dims/2 ("half"); the frequencies may be scaled by bands of their wavelength
    (``banded_frequencies``).  A mixer that norms its queries and keys first calls ``norm_rotate_store``:
    norm, rotation and the cache store are one kernel."""

    graph_safe = True

    def __init__(self, prefix, base: float, dims: int, layout: str = "half", scaling: dict | None = None):
        super().__init__(prefix)
        self.base, self.dims, self.layout = float(base), int(dims), layout
        self.scaling = dict(scaling) if scaling else None
        if self.dims < 0 or self.dims % 2 != 0:
            raise ValueError(f"{prefix}: an even number of entries is rotated, got {self.dims}")
        if self.base <= 1.0:
            raise ValueError(f"{prefix}: the rotary base must be larger than 1")
        if layout not in ("interleaved", "half"):
            raise ValueError(f"{prefix}: unknown layout of the rotated pairs '{layout}' (known: half, interleaved)")
        if self.scaling is not None:
            for key in ("factor", "low", "high", "original"):
                if key not in self.scaling or float(self.scaling[key]) <= 0:
                    raise ValueError(f"{prefix}: the scaling needs a positive '{key}'")
            if float(self.scaling["high"]) <= float(self.scaling["low"]):
                raise ValueError(f"{prefix}: the scaling's 'high' must lie above its 'low'")
        self.frequencies = banded_frequencies(self.base, self.dims, self.scaling) if self.dims else []
        self.inv_freq = None

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        device = runtime.device if runtime is not None else "cuda"
        self.inv_freq = torch.tensor(self.frequencies or [0.0], dtype=torch.float64, device=device)

    def norm_rotate_store(self, ctx, cache, qkv, q_out, k_off, v_off, n_heads, n_kv_heads, key_size, value_size, q_gain, k_gain,
                          norm, eps):
        if self.dims > key_size:
            raise ValueError(f"{self.prefix}: {self.dims} rotated entries do not fit a head of {key_size}")
        return ctx.kernels.norm_rotary_store(ctx, cache, qkv, q_out, k_off, v_off, n_heads, n_kv_heads, key_size, value_size,
                                             q_gain, k_gain, norm, eps, self.dims, self.layout, self.inv_freq)


register_part("interleaved_rotary", InterleavedRotary)
register_part("banded_rotary", BandedRotary)

"""Position encodings a mixer can apply to q and k.

"rope": rotary encoding with per-pair frequencies theta_d = theta^(-2d/D), optionally rescaled by the
llama3 rule; frequencies are computed on the host in float32 exactly as the reference does
(src/engine/llama4_cpu_engine.cpp:446-464), the angle float(p) * theta_d and its sine and cosine on
the device (the reference tabulates them, :466-470).  "none": q and k are used as projected.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import Position, RotaryEncoding, register_position


def llama3_frequencies(head_dim: int, theta: float, scaling) -> np.ndarray:
    f32 = np.float32
    half = head_dim // 2
    out = np.empty(half, dtype=np.float32)
    for d in range(half):
        expo = f32(-2.0) * f32(d) / f32(head_dim)
        t = f32(np.power(f32(theta), expo, dtype=np.float32))
        if scaling is not None:
            orig = f32(scaling["original_max_position_embeddings"])
            low, high = f32(scaling["low_freq_factor"]), f32(scaling["high_freq_factor"])
            factor = f32(scaling["factor"])
            wavelen = f32(2.0) * f32(3.14159265358979323846) / t
            if wavelen > orig / low:
                t = t / factor
            elif wavelen >= orig / high:
                smooth = (orig / wavelen - low) / (high - low)
                t = (f32(1.0) - smooth) * (t / factor) + smooth * t
        out[d] = t
    return out


def llama3_frequencies_f64(dims: int, theta: float, scaling) -> np.ndarray:
    """The same rule in double precision, rounded to float32 once: a frequency whose wavelength is shorter than
    original / high is kept, one longer than original / low is divided by `factor`, and between the two
    s = (original / wavelength - low) / (high - low) blends them, (1 - s) f / factor + s f."""
    f = np.float64(theta) ** (-2.0 * np.arange(dims // 2, dtype=np.float64) / dims)
    if scaling is not None:
        orig, factor = float(scaling["original_max_position_embeddings"]), float(scaling["factor"])
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        wavelength = 2.0 * np.pi / f
        s = (orig / wavelength - low) / (high - low)
        blended = (1.0 - s) * f / factor + s * f
        f = np.where(wavelength < orig / high, f, np.where(wavelength > orig / low, f / factor, blended))
    return f.astype(np.float32)


def yarn_frequencies(dims: int, theta: float, scaling) -> tuple:
    """(frequencies, amplitude) of the YaRN rule in double precision, rounded once.  With f_i = theta^(-2i / dims) and
    d(t) = dims * ln(original / (2 pi t)) / (2 ln theta), the pair index whose wave makes t turns over `original`
    positions: lo = max(floor(d(beta_fast)), 0), hi = min(ceil(d(beta_slow)), dims - 1), ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1); pair i turns at f_i (1 - ramp_i) + f_i / factor * ramp_i, so fast pairs keep their
    frequency and slow pairs are stretched by `factor`; sines and cosines are multiplied by 0.1 ln(factor) + 1."""
    factor, original = float(scaling["factor"]), float(scaling["original_max_position_embeddings"])
    fast, slow = float(scaling["beta_fast"]), float(scaling["beta_slow"])
    if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and theta > 1):
        raise ValueError("rope: the yarn rule needs positive factor, original length, beta_fast and beta_slow")
    i = np.arange(dims // 2, dtype=np.float64)
    f = np.float64(theta) ** (-2.0 * i / dims)
    turn = lambda t: dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(theta))
    lo, hi = max(math.floor(turn(fast)), 0), min(math.ceil(turn(slow)), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).astype(np.float32), 0.1 * math.log(factor) + 1.0


@register_position("rope")
class RotaryPosition(Position):
    """params: head_dim, theta, pairing ("half_split" pairs (d, d+D/2); "interleaved" pairs (2d, 2d+1)),
    scaling (None, the llama3 dictionary, {"rope_type": "linear", "factor": f}: every frequency divided by f, or
    {"rope_type": "yarn", "factor", "original_max_position_embeddings", "beta_fast", "beta_slow"}: see
    `yarn_frequencies`), rotary_dims (None: the whole head; n: only the first n elements of a
    head turn, as pairs (d, d + n/2) with frequencies theta^(-2d/n), the rest pass unchanged), frequency_math
    ("float32": the powers as the reference computes them; "float64": in double precision, rounded once, the
    llama3 rule included)."""
    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        sc = spec.get("scaling")
        linear, yarn = None, None
        if sc is not None and sc.get("rope_type", "llama3") == "yarn":
            yarn, sc = sc, None
        if sc is not None and sc.get("rope_type", "llama3") == "linear":
            linear, sc = float(sc["factor"]), None         # every frequency divided by one factor
            if not linear > 0:
                raise ValueError(f"rope: a linear scaling factor must be positive, not {linear}")
        if sc is not None and sc.get("rope_type", "llama3") != "llama3":
            raise ValueError(f"rope scaling of type '{sc.get('rope_type')}' is not supported")
        if spec["pairing"] not in ("half_split", "interleaved"):
            raise ValueError(f"unknown rope pairing '{spec['pairing']}'")
        self.interleaved = spec["pairing"] == "interleaved"
        dims = spec.get("rotary_dims")
        dims = int(spec["head_dim"]) if dims is None else int(dims)
        if dims < 2 or dims % 2 or dims > int(spec["head_dim"]):
            raise ValueError(f"rope: {dims} rotated elements of a head of {spec['head_dim']}")
        self.amplitude = 1.0
        if yarn is not None:
            self.frequencies, self.amplitude = yarn_frequencies(dims, float(spec["theta"]), yarn)
        elif spec.get("frequency_math", "float32") == "float64" and sc is not None:
            self.frequencies = llama3_frequencies_f64(dims, float(spec["theta"]), sc)
        elif spec.get("frequency_math", "float32") == "float64":
            # theta^(-2d/n) / factor in double precision, rounded once
            f = np.float64(spec["theta"]) ** (-2.0 * np.arange(dims // 2, dtype=np.float64) / dims)
            self.frequencies = (f / (linear or 1.0)).astype(np.float32)
        else:
            self.frequencies = llama3_frequencies(dims, float(spec["theta"]), sc)
            if linear is not None:
                self.frequencies = (self.frequencies.astype(np.float64) / linear).astype(np.float32)
        self.inv_freq = None

    def prepare(self, device):
        self.inv_freq = torch.from_numpy(self.frequencies).to(device)

    def encoding(self):
        return RotaryEncoding(self.inv_freq, self.interleaved, self.amplitude)


@register_position("none")
class NoPosition(Position):
    graph_safe = True

"""Rotary position encoding part.

Frequencies: f_j = theta^(-2j/rotary_dim) (batchspec/models/modules/rope.py:27-31),
optionally rescaled by the llama3 rule whose constants the reference forwards
(rope.py:33-44), divided by a plain factor (``rope_scale``), or blended by the YaRN
rule (``yarn``: factor, original, fast, slow; cosine and sine then carry a magnitude).  The table is built
in float64 on the host and held as two float32 numbers per frequency; the kernels form
the angle position * f_j in float64 and reduce it to [-pi, pi] there, so that it is
right to 2e-7 rad at any position; sine, cosine and the rotation are float32.

Pairing: the reference rotates adjacent pairs after permuting Wq/Wk rows offline
(tools/prepare_model/convert_weights.py:112-128); this part keeps the
checkpoint's row order and rotates (j, j + rotary_dim/2), which gives the same
scores.  ``interleaved=True`` rotates adjacent pairs for checkpoints that were
permuted.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import POSITION_ENCODINGS, PositionEncoding, Runtime, register_part


def rope_inv_freq(rotary_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    j = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * j / rotary_dim)
    if scaling:
        kind = scaling["rope_type"]
        factor = float(scaling["factor"])
        if kind == "linear":
            f = f / factor
        elif kind == "llama3":
            low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
            old = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            smooth = ((old / wavelen) - low) / (high - low)
            mid = (1.0 - smooth) * f / factor + smooth * f
            f = torch.where(wavelen > old / low, f / factor, torch.where(wavelen < old / high, f, mid))
        elif kind == "yarn":
            f = yarn_blend(f, rotary_dim, float(theta), factor, float(scaling["original"]), float(scaling["fast"]),
                           float(scaling["slow"]))
        else:
            raise ValueError(f"rope scaling {kind!r} is not supported")
    return f


def yarn_blend(f: torch.Tensor, rotary_dim: int, theta: float, factor: float, original: float, fast: float,
               slow: float) -> torch.Tensor:
    """YaRN: frequency i becomes f_i / factor * ramp_i + f_i * (1 - ramp_i).  The ramp rises linearly from 0 at index
    lo to 1 at index hi, where index(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta) is the (fractional)
    index of the frequency that makes t turns over ``original`` positions, lo = max(floor(index(fast)), 0) and
    hi = min(ceil(index(slow)), rotary_dim - 1); a ramp of no width is given the width 0.001."""
    def index(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(index(fast)), 0)
    hi = min(math.ceil(index(slow)), rotary_dim - 1)
    i = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp)


def yarn_magnitude(factor: float) -> float:
    """What YaRN multiplies cosine and sine by: 0.1 ln(factor) + 1."""
    return 0.1 * math.log(factor) + 1.0


@register_part(POSITION_ENCODINGS, "rope")
class RotaryEmbedding(PositionEncoding):
    graph_safe = True
    def __init__(self, runtime: Runtime, head_dim: int, theta: float, scaling: Optional[dict] = None,
                 rotary_dim: Optional[int] = None, interleaved: bool = False):
        self.runtime = runtime
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim {self.head_dim}")
        self.interleaved = bool(interleaved)
        self.frequencies = rope_inv_freq(self.rotary_dim, theta, scaling)            # float64, on the host
        self.inv_freq = ops.rope_frequency_table(self.frequencies, runtime.device)
        # cosine and sine times this (YaRN); the fused rotate-and-append kernels know no magnitude
        self.magnitude = yarn_magnitude(float(scaling["factor"])) if scaling and scaling["rope_type"] == "yarn" else 1.0

    def rope_table(self):
        if self.magnitude != 1.0:
            return None
        return self.inv_freq, self.rotary_dim, self.interleaved

    def apply(self, q, k, ctx):
        ops.rope_inplace(q, ctx.positions, self.inv_freq, self.rotary_dim, self.interleaved, self.magnitude)
        if k is not None:
            ops.rope_inplace(k, ctx.positions, self.inv_freq, self.rotary_dim, self.interleaved, self.magnitude)


@register_part(POSITION_ENCODINGS, "none")
class NoPositionEncoding(PositionEncoding):
    graph_safe = True
    def __init__(self, runtime: Runtime):
        self.runtime = runtime

    def apply(self, q, k, ctx):
        return None

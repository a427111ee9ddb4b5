"""Position encodings.

``rope``: non-interleaved ("rotate half") rotary positions over the whole head size. The tables
are built once in float64 and stored in float32, as the reference does
(src/llmserve/models/layers.py:47-63); they stay float32 in the bfloat16 path too, so rotation
angles are never rounded to 16 bits. Frequency scaling ``linear`` and ``llama3`` follow
src/llmserve/models/layers.py:24-58.

Frequency scaling ``yarn``: with ``d(t) = dims * ln(original / (2 pi t)) / (2 ln theta)``, ``lo =
max(floor(d(yarn_fast)), 0)``, ``hi = min(ceil(d(yarn_slow)), dims - 1)`` and ``ramp_i = clamp((i -
lo) / max(hi - lo, 0.001), 0, 1)``, frequency i becomes ``f_i / factor * ramp_i + f_i * (1 -
ramp_i)`` (fast-turning pairs keep their frequency, slow ones are stretched by ``factor``), and
both tables are multiplied by ``0.1 ln(factor) + 1``.

``head_dim`` is the number of rotated dims: a mixer whose heads are larger rotates the first
``head_dim`` dims of each head (pairs ``(i, i + head_dim/2)``) and passes the rest.

``none``: no position information (for mixers that carry order in their own state).

``sinusoid``: an absolute encoding added to the embedded tokens: entry 2i of the vector of
position p is ``sin(p * base^(-2i/width))`` and entry 2i+1 the cosine of the same angle. The
frequencies are made once in float64 and stored in float32; the angle is the float32 product of
the position and the frequency.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .base import POSITION_ENCODINGS, PositionEncoding


@dataclass(frozen=True)
class RotarySpec:
    head_dim: int
    theta: float
    scaling_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_positions: int = 0
    yarn_fast: float = 32.0  # turns over the original length above which a pair keeps its frequency
    yarn_slow: float = 1.0  # turns below which a pair is stretched by the whole factor
    kind: str = "rope"


def rotary_table_factor(spec: RotarySpec) -> float:
    """What cos and sin are multiplied by (one, except under ``yarn``)."""
    return 0.1 * math.log(spec.factor) + 1.0 if spec.scaling_type == "yarn" else 1.0


@dataclass(frozen=True)
class NoPositionSpec:
    kind: str = "none"


def rotary_inverse_frequencies(spec: RotarySpec) -> torch.Tensor:
    """float64 ``[head_dim/2]``."""
    d = spec.head_dim
    inv = 1.0 / (spec.theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    if spec.scaling_type == "linear":
        inv = inv / spec.factor
    elif spec.scaling_type == "llama3":
        old = spec.original_max_positions
        low_wavelen = old / spec.low_freq_factor
        high_wavelen = old / spec.high_freq_factor
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > low_wavelen, inv / spec.factor, inv)
        smooth = (old / wavelen - spec.low_freq_factor) / (
            spec.high_freq_factor - spec.low_freq_factor
        )
        mid = (1 - smooth) * scaled / spec.factor + smooth * scaled
        is_mid = (wavelen >= high_wavelen) & (wavelen <= low_wavelen)
        inv = torch.where(is_mid, mid, scaled)
    elif spec.scaling_type == "yarn":
        def pair_of(turns: float) -> float:
            return d * math.log(spec.original_max_positions / (2.0 * math.pi * turns)) / (2.0 * math.log(spec.theta))

        lo = max(math.floor(pair_of(spec.yarn_fast)), 0)
        hi = min(math.ceil(pair_of(spec.yarn_slow)), d - 1)
        ramp = ((torch.arange(d // 2, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        inv = inv / spec.factor * ramp + inv * (1.0 - ramp)
    elif spec.scaling_type != "default":
        raise NotImplementedError(f"rope scaling {spec.scaling_type!r}")
    return inv


@POSITION_ENCODINGS.register("rope")
class RotaryPositionEncoding(PositionEncoding):
    def __init__(self, spec: RotarySpec, env) -> None:
        super().__init__(spec, env)
        if spec.head_dim % 2:
            raise ValueError(f"rotary positions need an even head size, got {spec.head_dim}")
        inv = rotary_inverse_frequencies(spec)
        ang = torch.outer(torch.arange(env.max_positions, dtype=torch.float64), inv)
        mag = rotary_table_factor(spec)
        self.cos = (ang.cos() * mag).float().contiguous().to(env.device)
        self.sin = (ang.sin() * mag).float().contiguous().to(env.device)

    def rotary_tables(self):
        return self.cos, self.sin


@dataclass(frozen=True)
class SinusoidSpec:
    hidden_size: int
    base: float = 10000.0
    kind: str = "sinusoid"


@POSITION_ENCODINGS.register("sinusoid")
class SinusoidPositionEncoding(PositionEncoding):
    def __init__(self, spec: SinusoidSpec, env) -> None:
        super().__init__(spec, env)
        w = spec.hidden_size
        i = torch.arange((w + 1) // 2, dtype=torch.float64)
        self.freq = (spec.base ** (-2.0 * i / w)).float().contiguous().to(env.device)

    def embed(self, x, positions) -> None:
        self.ops.sinusoid_add(x, positions, self.freq)


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    pass

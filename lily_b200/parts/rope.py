"""Rotary position encoding as float32 cos / sin tables.

A position encoding of the "rotation table" sort gives the mixer ``rotary_dim`` and
``tables() -> (cos, sin)``, each float32 ``[positions, rotary_dim / 2]``; the attention mixer hands
them to the fused norm + rotation + cache-write kernel, which rotates the first ``rotary_dim``
features of each head in rotate-half order and passes the rest through.

Frequencies ``base^(-2j/rotary_dim)`` and angles ``position * frequency`` are float32, as in
lily/layers/rotary.py:49-56; Llama-3 scaling follows rotary.py:99-119; "yarn" scaling blends each frequency with
its slowed value by a ramp over the feature index and stretches both tables (``_yarn``, ``table_stretch``).  The tables stay float32
in both precisions (the reference casts them to the model dtype, rotary.py:46-47).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from lily_b200.config.model_config import RopeScaling
from lily_b200.parts.base import BuildContext, Part, register_part


@dataclass(frozen=True)
class RopeSpec:
    head_dim: int
    rotary_dim: int
    theta: float
    scaling: RopeScaling = field(default_factory=RopeScaling)
    kind: str = "rope"
    # True: feature 2i is paired with feature 2i + 1 (the interleaved layout) instead of i with i + rotary_dim / 2.
    # A score q . k does not change when the features of q and k are reordered alike, so a mixer serves this layout
    # by reordering the rows of its q and k projections once, when it loads them (``pairing_order``), and the kernels
    # rotate halves as ever.
    interleaved: bool = False
    # True: the frequencies are worked out in float64 and then rounded to float32 (a float32 power is up to a few
    # units in the last place off, which a position of a thousand turns into 1e-4 of a radian); the angles are
    # float32 products either way
    exact_frequencies: bool = False


def inverse_frequencies(spec: RopeSpec) -> torch.Tensor:
    work = torch.float64 if spec.exact_frequencies else torch.float32
    inv = 1.0 / (spec.theta ** (torch.arange(0, spec.rotary_dim, 2, dtype=work) / spec.rotary_dim))
    return _scaled(inv, spec).to(torch.float32)


def _scaled(inv: torch.Tensor, spec: RopeSpec) -> torch.Tensor:
    s = spec.scaling
    if s.rope_type == "default":
        return inv
    if s.rope_type == "yarn":
        return _yarn(inv, spec)
    if s.rope_type != "llama3":
        raise ValueError(f"Unsupported rope scaling type {s.rope_type!r}")
    low_wavelen = s.original_max_position_embeddings / s.low_freq_factor
    high_wavelen = s.original_max_position_embeddings / s.high_freq_factor
    wavelen = 2 * math.pi / inv
    if s.low_freq_factor != s.high_freq_factor:
        smooth = (s.original_max_position_embeddings / wavelen - s.low_freq_factor) / (
            s.high_freq_factor - s.low_freq_factor)
    else:
        smooth = torch.zeros_like(inv)
    mid = (1 - smooth) * inv / s.factor + smooth * inv
    return torch.where(wavelen < high_wavelen, inv, torch.where(wavelen > low_wavelen, inv / s.factor, mid))


def _yarn(inv: torch.Tensor, spec: RopeSpec) -> torch.Tensor:
    """Frequencies blended between their own value and a ``factor``-th of it by a ramp over the feature index: the index
    at which a wave makes t turns over the original length L is ``dims ln(L / (2 pi t)) / (2 ln theta)``; the ramp
    rises from 0 at the (floored, at least 0) index of ``fast_turns`` to 1 at the (ceiled, at most dims - 1) index of
    ``slow_turns``."""
    s, dims = spec.scaling, spec.rotary_dim

    def index(turns: float) -> float:
        return dims * math.log(s.original_max_position_embeddings / (2.0 * math.pi * turns)) / (2.0 * math.log(spec.theta))
    lo = max(math.floor(index(s.fast_turns)), 0)
    hi = min(math.ceil(index(s.slow_turns)), dims - 1)
    i = torch.arange(dims // 2, dtype=inv.dtype)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return inv / s.factor * ramp + inv * (1.0 - ramp)


def table_stretch(spec: RopeSpec) -> float:
    """The factor both tables are multiplied by (1 unless the scaling stretches them)."""
    s = spec.scaling
    return s.table_stretch_slope * math.log(s.factor) + 1.0 if s.rope_type == "yarn" and s.factor > 0 else 1.0


def pairing_order(head_dim: int, rotary_dim: int) -> torch.Tensor:
    """For each feature of a head in the order the kernels rotate (first halves, second halves, the rest), the
    feature of the interleaved layout that stands there: [0, 2, 4, ..., 1, 3, 5, ..., rotary_dim, ...]."""
    return torch.cat([torch.arange(0, rotary_dim, 2), torch.arange(1, rotary_dim, 2), torch.arange(rotary_dim, head_dim)])


_TABLES = {}      # (spec, positions, device) -> (cos, sin): layers with the same encoding share one pair of tables


@register_part("position", "rope")
class RotaryTable(Part):
    def __init__(self, spec: RopeSpec, prefix: str, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.rotary_dim = spec.rotary_dim
        self.interleaved = spec.interleaved
        key = (spec.rotary_dim, spec.theta, spec.scaling, spec.exact_frequencies, ctx.max_position, str(ctx.device))
        if key not in _TABLES:
            if len(_TABLES) > 16:
                _TABLES.clear()
            t = torch.arange(ctx.max_position, dtype=torch.float32)
            freqs = torch.outer(t, inverse_frequencies(spec))          # float32 on the host
            stretch = table_stretch(spec)
            cos, sin = (freqs.cos(), freqs.sin()) if stretch == 1.0 else (freqs.cos() * stretch, freqs.sin() * stretch)
            _TABLES[key] = (cos.contiguous().to(ctx.device), sin.contiguous().to(ctx.device))
        self._cos, self._sin = _TABLES[key]

    def tables(self):
        return self._cos, self._sin

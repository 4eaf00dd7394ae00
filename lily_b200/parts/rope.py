"""Rotary position encoding as float32 cos / sin tables.

A position encoding of the "rotation table" sort gives the mixer ``rotary_dim`` and
``tables() -> (cos, sin)``, each float32 ``[positions, rotary_dim / 2]``; the attention mixer hands
them to the fused norm + rotation + cache-write kernel, which rotates the first ``rotary_dim``
features of each head in rotate-half order and passes the rest through.

Frequencies ``base^(-2j/rotary_dim)`` and angles ``position * frequency`` are float32, as in
lily/layers/rotary.py:49-56; Llama-3 scaling follows rotary.py:99-119.  The tables stay float32
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


def inverse_frequencies(spec: RopeSpec) -> torch.Tensor:
    inv = 1.0 / (spec.theta ** (torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim))
    s = spec.scaling
    if s.rope_type == "default":
        return inv
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


@register_part("position", "rope")
class RotaryTable(Part):
    def __init__(self, spec: RopeSpec, prefix: str, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.rotary_dim = spec.rotary_dim
        t = torch.arange(ctx.max_position, dtype=torch.float32)
        freqs = torch.outer(t, inverse_frequencies(spec))          # float32 on the host
        self._cos = freqs.cos().contiguous().to(ctx.device)
        self._sin = freqs.sin().contiguous().to(ctx.device)

    def tables(self):
        return self._cos, self._sin

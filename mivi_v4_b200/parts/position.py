"""Position encodings.  A mixer that rotates its queries and keys asks its
position part for ``rotary()``; a part that encodes nothing returns None.  A part may
also define ``score_scale()``: a constant factor on the attention scores (an encoding
that stretches its frequencies and makes up for it by sharpening the softmax); the
mixer multiplies its 1/sqrt(head_dim) by it."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import Part
from .registry import register

ROPE_STYLES = ("interleaved", "half_split")


@register("position", "rope")
class Rope(Part):
    """Rotary encoding: pair i of a head turns by pos * theta^(-2i/head_dim)
    (crates/mivi-core/src/rope.rs:59-61, 116-121).  ``interleaved`` pairs the
    elements (2i, 2i+1) as the reference does (rope.rs:219-229);
    ``half_split`` pairs (i, i + head_dim/2).  The frequencies are worked out
    in float64 and rounded once to float32; the angle is a float32 product."""

    def __init__(self, head_dim: int, theta: float, style: str = "interleaved"):
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {head_dim}")
        if style not in ROPE_STYLES:
            raise ValueError(f"rope style {style!r}; known: {', '.join(ROPE_STYLES)}")
        self.head_dim, self.theta, self.style = int(head_dim), float(theta), style
        self._inv_freq: Optional[torch.Tensor] = None

    def rotary(self, device) -> Optional[Tuple[torch.Tensor, bool]]:
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            i = torch.arange(self.head_dim // 2, dtype=torch.float64)
            inv = 1.0 / (torch.tensor(self.theta, dtype=torch.float64) ** (2.0 * i / self.head_dim))
            self._inv_freq = inv.to(torch.float32).to(device)
        return self._inv_freq, self.style == "half_split"

    def score_scale(self) -> float:
        return 1.0

    def amplitude(self) -> float:
        """A factor on cos and sin (1: a pure rotation)."""
        return 1.0


@register("position", "none")
class NoPosition(Part):
    """No position encoding inside the mixer."""

    def rotary(self, device):
        return None


@register("position", "rope_yarn")
class YarnRope(Rope):
    """Rotary encoding whose low frequencies are stretched so that a model reaches ``factor`` times its original
    context (YaRN; Peng et al., "YaRN: Efficient Context Window Extension of Large Language Models").  With
    f_i = theta^(-2i/dims) and turns(t) = dims ln(original / (2 pi t)) / (2 ln theta), the pairs from
    lo = max(floor(turns(fast)), 0) to hi = min(ceil(turns(slow)), dims - 1) are blended by
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1): frequency f_i / factor * ramp_i + f_i (1 - ramp_i).
    Cos and sin are multiplied by ``amplitude()`` = 0.1 ln(factor) + 1.  Pairs are (i, i + dims/2)."""

    def __init__(self, head_dim: int, theta: float, factor: float, original: float, fast: float, slow: float,
                 style: str = "half_split"):
        super().__init__(head_dim, theta, style)
        if factor < 1.0 or original <= 0 or fast <= 0 or slow <= 0:
            raise ValueError(f"rope scaling: factor {factor} (>= 1), original {original}, fast {fast}, slow {slow} (> 0)")
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)

    def _turn_dim(self, turns: float) -> float:
        return self.head_dim * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

    def rotary(self, device) -> Optional[Tuple[torch.Tensor, bool]]:
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            i = torch.arange(self.head_dim // 2, dtype=torch.float64)
            f = 1.0 / (torch.tensor(self.theta, dtype=torch.float64) ** (2.0 * i / self.head_dim))
            lo = max(math.floor(self._turn_dim(self.fast)), 0)
            hi = min(math.ceil(self._turn_dim(self.slow)), self.head_dim - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            inv = f / self.factor * ramp + f * (1.0 - ramp)
            self._inv_freq = inv.to(torch.float32).to(device)
        return self._inv_freq, self.style == "half_split"

    def amplitude(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0

"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from ..ops.linear import linear, norm_link_ok
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("embedding", "table")
class Embedding(Part):
    """x_t = E[token_t], no scaling (crates/mivi-model/src/model.rs:355-366)."""

    emits_norm = True            # forward(step, emit=link) can write the norm that follows it

    def __init__(self, vocab: int, hidden: int):
        self.vocab, self.hidden = int(vocab), int(hidden)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def forward(self, step, emit=None) -> torch.Tensor:
        """``emit``: the first layer's first norm as a link (steps of few tokens); its rows and sums
        are then written here and that norm is no kernel of its own."""
        x = step.ws.get("resid", (step.n_tokens, self.hidden), torch.float32)
        return K.embed(self.weight, step.tokens, x, emit)


@register("embedding", "table_scaled_positions")
class ScaledEmbeddingWithPositions(Part):
    """x_t = E[token_t] * scale + P[position_t]: a scaled token embedding plus a learned position vector
    (``positions`` False: no position table; ``max_positions`` None: as many rows as the checkpoint has).  With ``hand_rounded`` the rows are also written in the model's
    dtype and handed to the first block through ``step.handed`` as ("stream", rows): a block whose first
    sublayer reads the stream itself then needs no rounding pass."""

    def __init__(self, vocab: int, hidden: int, scale: float = 1.0, max_positions: Optional[int] = None,
                 hand_rounded: bool = False, positions: bool = True):
        self.vocab, self.hidden, self.scale = int(vocab), int(hidden), float(scale)
        self.max_positions = None if max_positions is None else int(max_positions)
        self.hand_rounded, self.has_positions = bool(hand_rounded), bool(positions)

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"weight": ParamSpec((self.vocab, self.hidden))}
        if self.has_positions:
            specs["positions"] = ParamSpec((self.max_positions, self.hidden))
        return specs

    def load(self, t) -> None:
        self.weight, self.positions = t["weight"], t.get("positions")
        if self.positions is not None and self.positions.dtype != self.weight.dtype:
            self.weight, self.positions = self.weight.float(), self.positions.float()

    def forward(self, step) -> torch.Tensor:
        N = step.n_tokens
        x = step.ws.get("resid", (N, self.hidden), torch.float32)
        rounded = None
        if self.hand_rounded and step.dtype != torch.float32:
            rounded = step.ws.get("stream_rounded", (N, self.hidden), step.dtype)
        if self.positions is not None and step.max_context > self.positions.shape[0]:
            raise K.KernelError(f"a sequence reaches position {step.max_context - 1}; the position table has "
                                f"{self.positions.shape[0]} rows")
        K.embed_scaled_pos(self.weight, step.tokens, self.scale, self.positions, step.positions, x, rounded)
        step.handed = ("stream", rounded) if rounded is not None else None
        return x


@register("head", "linear")
class LMHead(Part):
    """logits = f W^T in float32; W is the embedding table when ``tied``
    (crates/mivi-model/src/model.rs:455-473).  ``softcap`` c > 0: logits <- c tanh(logits / c)."""

    def __init__(self, vocab: int, hidden: int, tied: bool, softcap: float = 0.0):
        self.vocab, self.hidden, self.tied, self.softcap = int(vocab), int(hidden), bool(tied), float(softcap or 0.0)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {} if self.tied else {"weight": ParamSpec((self.vocab, self.hidden))}

    def carries_norm(self, step, embedding) -> bool:
        """Whether the product can apply the final norm's scale itself (steps of few rows)."""
        w = embedding.weight if self.tied else self.weight
        return norm_link_ok(step.n_out, w, step.dtype)

    def forward(self, f, step, embedding, scale=None) -> torch.Tensor:
        w = embedding.weight if self.tied else self.weight
        logits = step.ws.get("logits", (f.shape[0], self.vocab), torch.float32)
        linear(f, w, logits, scale=scale)
        return K.softcap_(logits, self.softcap) if self.softcap > 0 else logits

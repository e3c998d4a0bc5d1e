"""Per-layer inputs that depend on the token ids: something a layer adds to the residual stream from a
table row of the token at that place, beside the embedding at the model's entry."""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("token_input", "gated_table")
class GatedTableInput(Part):
    """x += rmsnorm(P (gelu_tanh(G x) * e)) with e the columns [index * dim, (index + 1) * dim) of the
    token's row in a table [vocab, table_width] that all layers share, G [dim, hidden], P [hidden, dim], and
    the norm a root-mean-square norm with a plain weight.  The residual stream is rounded to the model's
    dtype for the product with G; gelu, the norm and the sum are float32."""

    takes_norm = True            # forward(..., then_norm=...) runs the layer norm that follows inside its last kernel

    def __init__(self, hidden: int, vocab: int, dim: int, index: int, table_width: int, eps: float):
        self.hidden, self.vocab, self.dim = int(hidden), int(vocab), int(dim)
        self.index, self.table_width, self.eps = int(index), int(table_width), float(eps)
        if (self.index + 1) * self.dim > self.table_width:
            raise ValueError(f"columns {self.index * self.dim}..{(self.index + 1) * self.dim} lie outside a table "
                             f"of width {self.table_width}")

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"table": ParamSpec((self.vocab, self.table_width)),
                "gate": ParamSpec((self.dim, self.hidden)), "proj": ParamSpec((self.hidden, self.dim)),
                "norm": ParamSpec((self.hidden,), "vector", "norm")}

    def load(self, t) -> None:
        self.table, self.w_gate, self.w_proj, self.norm = t["table"], t["gate"], t["proj"], t["norm"]

    def forward(self, resid, step, then_norm=None) -> None:
        """``then_norm``: (layer norm part, out) of the norm that follows at once on the finished rows (the next
        layer's first one): it then runs inside this part's last kernel and ``out`` holds its result."""
        N, H = resid.shape
        g = self.scratch(step, "g", (N, self.dim), step.dtype)
        if K.table_gate_proj_ok(N, self.w_gate, self.table, step.dtype):
            # a few tokens: rounding, the narrow product and the gate in one kernel
            K.table_gate_proj(resid, self.w_gate, self.table, self.index * self.dim, step.tokens, g)
        else:
            x = resid
            if step.dtype != torch.float32:
                x = K.round_rows(resid, self.scratch(step, "x", (N, H), step.dtype))
            p = self.scratch(step, "p", (N, self.dim), torch.float32)
            linear(x, self.w_gate, p)
            K.table_gate(p, self.table, self.index * self.dim, step.tokens, g)
        y = self.scratch(step, "y", (N, H), torch.float32)
        linear(g, self.w_proj, y)
        if then_norm is not None:
            K.rmsnorm_add_layernorm(y, self.norm, self.eps, resid, then_norm[0].weight, then_norm[0].eps, then_norm[1])
        else:
            K.rmsnorm_add(y, self.norm, self.eps, resid)

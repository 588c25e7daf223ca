"""LayerNorm: mean and biased variance in two passes, rstd = 1/sqrt(var + eps), then
scale and shift (reference: crates/core/src/kernels/reference.rs:42-51).  The eps is a
parameter; the reference has it as a constant (crates/core/src/config.rs:20-21)."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import INIT_NORMAL, INIT_ONE_PLUS_NORMAL, VECTOR, Norm, ParamSpec, register_norm


@register_norm("layernorm")
class LayerNorm(Norm):
    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)

    def param_specs(self) -> List[ParamSpec]:
        return [
            ParamSpec("weight", (self.width,), VECTOR, INIT_ONE_PLUS_NORMAL),
            ParamSpec("bias", (self.width,), VECTOR, INIT_NORMAL),
        ]

    def reserve(self, workspace, limits) -> None:
        # where a product cannot fold the norm into its own kernel it normalises into this buffer
        workspace.reserve("norm.fallback", limits.max_rows * self.width, limits.dtype)

    def as_input(self, x: torch.Tensor, ctx, dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
        """This norm applied to the residual stream, in the form a matrix product can take as its
        activations (the product then normalises the rows itself where it can)."""
        return ops.NormInput(x, self.params["weight"], self.params["bias"], self.eps, ctx.workspace, dtype,
                             rows=rows, max_rows=0 if rows is not None else ctx.max_rows)

    def forward(self, x: torch.Tensor, out: torch.Tensor, n_rows: int,
                rows: Optional[torch.Tensor] = None) -> None:
        ops.layernorm(x, self.params["weight"], self.params["bias"], self.eps, out, n_rows, rows)

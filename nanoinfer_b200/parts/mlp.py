"""The dense feed-forward: x += act(xn . W_fc^T + b_fc) . W_proj^T + b_proj
(reference: crates/core/src/stages/blocks.rs:113-137).  The reference fixes the inner width
at 4C (crates/core/src/weights.rs:95-98) and the activation at tanh-GELU
(crates/core/src/kernels/reference.rs:53-61); both are parameters here, and the exact
erf-GELU is offered beside the tanh form."""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from .base import MATRIX, VECTOR, FeedForward, ParamSpec, StepContext, register_feed_forward


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    takes_norm_input = True

    def __init__(self, width: int, inner: int, activation: str, bias: bool = True):
        if activation not in ("tanh", "erf"):
            raise ValueError(f"activation {activation!r} is not one of 'tanh', 'erf' (the two GELU forms)")
        self.width, self.inner, self.activation, self.bias = int(width), int(inner), activation, bool(bias)

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec("fc_weight", (self.inner, self.width), MATRIX),
                 ParamSpec("proj_weight", (self.width, self.inner), MATRIX)]
        if self.bias:
            specs += [ParamSpec("fc_bias", (self.inner,), VECTOR), ParamSpec("proj_bias", (self.width,), VECTOR)]
        return specs

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("mlp.fc", limits.max_rows * self.inner, self.dtype)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> None:
        T, p = ctx.n_rows, self.params
        fc = ctx.workspace.get("mlp.fc", (ctx.max_rows, self.inner), self.dtype)
        xn, norm = (None, xn) if isinstance(xn, ops.NormInput) else (xn, None)
        ops.trace_scope(ctx.layer, "fc")
        ops.linear(xn, p["fc_weight"], p.get("fc_bias"), fc, T, act=ops.ACT_CODES[self.activation], norm=norm)
        ops.trace_scope(ctx.layer, "fc_proj")
        ops.linear(fc, p["proj_weight"], p.get("proj_bias"), x, T, residual=True)

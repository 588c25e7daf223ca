"""Token embedding: x[t] = table[token_t], written to the 32-bit residual stream; a position
encoding that is a plain table is added in the same kernel
(reference: crates/core/src/stages/blocks.rs:19-27)."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import TABLE, Embedding, ParamSpec, PositionEncoding, StepContext, register_embedding


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, width: int):
        self.vocab_size, self.width = int(vocab_size), int(width)

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("table", (self.vocab_size, self.width), TABLE)]

    def forward(self, ctx: StepContext, x: torch.Tensor, position: Optional[PositionEncoding]) -> None:
        table = position.additive_table() if position is not None else None
        ops.embed(ctx.tokens[:ctx.n_rows], self.params["table"], x, table,
                  ctx.positions if table is not None else None, feedback=ctx.token_feedback)
        if position is not None and table is None:
            position.on_embedding(x, ctx)

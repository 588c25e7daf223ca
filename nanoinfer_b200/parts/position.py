"""Learned absolute positions: a table row per position, added to the token embedding
(reference: crates/core/src/kernels/reference.rs:86-94).  The table's length bounds the
context (crates/core/src/stages/mod.rs:516-519)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .base import TABLE, ParamSpec, PositionEncoding, register_position


@register_position("learned_absolute")
class LearnedAbsolutePositions(PositionEncoding):
    def __init__(self, n_positions: int, width: int):
        self.n_positions, self.width = int(n_positions), int(width)

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("table", (self.n_positions, self.width), TABLE)]

    def additive_table(self) -> Optional[torch.Tensor]:
        return self.params["table"]

    def max_positions(self) -> Optional[int]:
        return self.n_positions

"""How the parts of a layer are arranged.  The pre-norm block is the reference's
(crates/core/src/stages/blocks.rs:4-8):
    x = x + mixer(norm_1(x));   x = x + feed_forward(norm_2(x))
Another arrangement is another class registered under another name."""
from __future__ import annotations

from typing import Callable, Dict, Optional, Type

import torch

from .base import FeedForward, KVCacheView, Mixer, Norm, StepContext

BLOCKS: Dict[str, Type["Block"]] = {}


def register_block(name: str) -> Callable[[Type["Block"]], Type["Block"]]:
    def deco(cls):
        BLOCKS[name] = cls
        return cls
    return deco


class Block:
    def __init__(self, width: int, norm_1: Norm, mixer: Mixer, norm_2: Norm, feed_forward: FeedForward):
        self.width = int(width)
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward

    def parts(self):
        return {"norm_1": self.norm_1, "mixer": self.mixer, "norm_2": self.norm_2,
                "feed_forward": self.feed_forward}

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool, dtype: torch.dtype) -> None:
        raise NotImplementedError


@register_block("pre_norm")
class PreNormBlock(Block):
    def _normed(self, norm, part, x, ctx, dtype):
        """The part's input: a foldable norm input where both the norm and the part can do that,
        else the norm's output in scratch."""
        if part.takes_norm_input:
            folded = norm.as_input(x, ctx, dtype)
            if folded is not None:
                return folded
        xn = ctx.workspace.get("block.normed", (ctx.max_rows, self.width), dtype)
        norm.forward(x, xn, ctx.n_rows)
        return xn

    def forward(self, x, ctx, cache, state, writes_cache, dtype) -> None:
        self.mixer.forward(self._normed(self.norm_1, self.mixer, x, ctx, dtype), x, ctx, cache, state, writes_cache)
        self.feed_forward.forward(self._normed(self.norm_2, self.feed_forward, x, ctx, dtype), x, ctx)

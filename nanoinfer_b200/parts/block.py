"""How the parts of a layer are arranged.  The pre-norm block is the reference's
(crates/core/src/stages/blocks.rs:4-8):
    x = x + mixer(norm_1(x));   x = x + feed_forward(norm_2(x))
Another arrangement is another class registered under another name.  An arrangement names the
parts it is made of and the registry each comes from (``slots``); a layer's specification gives a
part for each of these names, and the model builds them."""
from __future__ import annotations

from typing import Callable, ClassVar, Dict, Optional, Type

import torch

from .base import FEED_FORWARDS, MIXERS, NORMS, KVCacheView, Mixer, Part, Registry, StepContext, StepLimits, Workspace

BLOCKS: Dict[str, Type["Block"]] = {}


def register_block(name: str) -> Callable[[Type["Block"]], Type["Block"]]:
    def deco(cls):
        BLOCKS[name] = cls
        return cls
    return deco


class Block:
    #: part name -> the registry it is built from.  At most one of them may be a mixer: the cache
    #: manager gives a run of the layer one set of pages or one state slot tensor.
    slots: ClassVar[Dict[str, Registry]] = {}

    def __init__(self, width: int, parts: Dict[str, Part]):
        missing, unknown = set(self.slots) - set(parts), set(parts) - set(self.slots)
        if missing or unknown:
            raise ValueError(f"{type(self).__name__} is made of {sorted(self.slots)}: missing {sorted(missing)}, "
                             f"unknown {sorted(unknown)}")
        self.width = int(width)
        self._parts = dict(parts)
        for name, part in parts.items():
            setattr(self, name, part)
        mixers = [p for p in parts.values() if isinstance(p, Mixer)]
        if len(mixers) > 1:
            raise ValueError("a block holds at most one mixer")
        #: the part that mixes across positions (None: the layer has none)
        self.mixer: Optional[Mixer] = mixers[0] if mixers else None

    def parts(self) -> Dict[str, Part]:
        return dict(self._parts)

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        """Size the arrangement's own scratch (the parts size theirs themselves)."""

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool, dtype: torch.dtype) -> None:
        raise NotImplementedError


@register_block("pre_norm")
class PreNormBlock(Block):
    slots = {"norm_1": NORMS, "mixer": MIXERS, "norm_2": NORMS, "feed_forward": FEED_FORWARDS}

    def reserve(self, workspace, limits) -> None:
        workspace.reserve("block.normed", limits.max_rows * self.width, limits.dtype)

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

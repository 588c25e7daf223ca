"""The parts a model is put together from.  Importing this package registers the built-in
parts under their names."""
from . import attention, block, embedding, head, mlp, norm, position  # noqa: F401  (registration)
from .base import (FEED_FORWARDS, HEADS, EMBEDDINGS, MIXERS, NORMS, POSITIONS, Embedding, FeedForward, Head,
                   KVCacheSpec, KVCacheView, Mixer, Norm, ParamSpec, Part, PositionEncoding, StateSpec,
                   StepContext, TensorRef, Workspace, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position)
from .block import BLOCKS, Block, register_block

__all__ = [n for n in dir() if not n.startswith("_")]

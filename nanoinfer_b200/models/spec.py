"""A model as data: which part stands where, which checkpoint tensor feeds which parameter,
and in which order the layers run.

An architecture's builder turns its configuration into a ``ModelSpec``; ``Model`` (model.py)
builds the parts from it through the part registries.  The run order is a list too: a
``ScheduleEntry`` names a layer (the same layer may be named twice: shared weights, but each
run has keys and values of its own) and may say that it reads the cache of an earlier entry
instead of writing one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..parts.base import TensorRef


@dataclass
class PartSpec:
    kind: str                                   # registered name of the part
    args: Dict[str, Any]                        # constructor arguments (sizes and constants)
    tensors: Dict[str, TensorRef] = field(default_factory=dict)   # parameter key -> checkpoint tensor


class LayerSpec:
    """One layer: the registered name of its arrangement and a part for each of the names that
    arrangement is made of (for the pre-norm block: ``norm_1``, ``mixer``, ``norm_2``,
    ``feed_forward``), given as keywords or as the ``parts`` dictionary."""

    def __init__(self, arrangement: str, parts: Optional[Dict[str, PartSpec]] = None,
                 mixer_position: Optional[PartSpec] = None, **named: PartSpec):
        self.arrangement = arrangement              # registered name of the block arrangement
        self.parts: Dict[str, PartSpec] = {**(parts or {}), **named}
        #: a position encoding that acts inside the mixer (on queries and keys), if any
        self.mixer_position = mixer_position

    def __getattr__(self, name: str) -> PartSpec:
        parts = self.__dict__.get("parts", {})
        if name in parts:
            return parts[name]
        raise AttributeError(name)

    def __repr__(self) -> str:
        return f"LayerSpec({self.arrangement!r}, {self.parts!r}, mixer_position={self.mixer_position!r})"


@dataclass
class ScheduleEntry:
    layer: int                                  # index into ModelSpec.layers
    #: index of an EARLIER schedule entry whose keys and values this run reads; None: its own
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    width: int
    embedding: PartSpec
    position: Optional[PartSpec]                # position encoding applied at the embedding, if any
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    #: the longest sequence the model takes (None: bounded by the cache only)
    max_positions: Optional[int] = None
    #: prefixes a checkpoint may put before every name
    name_prefixes: List[str] = field(default_factory=lambda: [""])
    #: regular expressions of tensors a checkpoint may hold that the model does not use
    ignorable: List[str] = field(default_factory=list)
    eos_token_id: Optional[int] = None

"""A model built from a ModelSpec: the parts, the run order, and the forward pass over the
rows of one step.

The forward pass is the reference's (crates/core/src/stages/kv_cache.rs:25-74): embed the new
tokens at their positions, run the layers (each appends its keys and values to the cache and
attends over it), then the final norm and the head on the rows whose logits are wanted only
(crates/metal/src/shaders/batch.metal:430-452 gathers them the same way).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..parts import base as P
from ..parts.block import BLOCKS, Block
from .spec import ModelSpec, PartSpec


@dataclass
class Binding:
    """One parameter of one part and the checkpoint tensor that feeds it."""
    part: P.Part
    spec: P.ParamSpec
    ref: P.TensorRef
    where: str          # for messages, e.g. "layers[3].mixer"


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class Model:
    def __init__(self, spec: ModelSpec, config=None):
        self.spec, self.config = spec, config
        self.width = spec.width
        self._bindings: List[Binding] = []
        self.embedding = self._build(P.EMBEDDINGS, spec.embedding, "embedding")
        self.position = self._build(P.POSITIONS, spec.position, "position") if spec.position else None
        self.layers: List[Block] = []
        for i, ls in enumerate(spec.layers):
            if ls.arrangement not in BLOCKS:
                raise KeyError(f"unknown block arrangement {ls.arrangement!r}; registered: {sorted(BLOCKS)}")
            w = f"layers[{i}]"
            cls = BLOCKS[ls.arrangement]
            built: Dict[str, P.Part] = {}
            for name, ps in ls.parts.items():
                if name not in cls.slots:
                    raise ValueError(f"{w}: the {ls.arrangement!r} arrangement has no part {name!r} "
                                     f"(it is made of {sorted(cls.slots)})")
                registry = cls.slots[name]
                if registry is P.MIXERS and ls.mixer_position is not None:
                    args = dict(ps.args)
                    args["position"] = self._build(P.POSITIONS, ls.mixer_position, f"{w}.mixer_position")
                    ps = PartSpec(ps.kind, args, ps.tensors)
                built[name] = self._build(registry, ps, f"{w}.{name}")
            self.layers.append(cls(spec.width, built))
        self.final_norm = self._build(P.NORMS, spec.final_norm, "final_norm")
        self.head = self._build(P.HEADS, spec.head, "head")
        self.schedule = list(spec.schedule)
        self._check_schedule()
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # ------------------------------------------------------------------ construction
    def _build(self, registry: P.Registry, ps: PartSpec, where: str) -> P.Part:
        part = registry.build(ps.kind, **ps.args)
        wanted = {s.key: s for s in part.param_specs()}
        unknown = set(ps.tensors) - set(wanted)
        unmapped = set(wanted) - set(ps.tensors)
        if unknown or unmapped:
            raise ValueError(f"{where} ({ps.kind}): tensors mapped to unknown parameters {sorted(unknown)}, "
                             f"parameters without a tensor {sorted(unmapped)}")
        for key, s in wanted.items():
            self._bindings.append(Binding(part, s, ps.tensors[key], where))
        return part

    def _check_schedule(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {e.layer}, but there are {len(self.layers)} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i or self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{i}].cache_of must name an earlier entry that owns a cache")
                a = self._kv_spec(e.layer)
                b = self._kv_spec(self.schedule[e.cache_of].layer)
                if a is None or a != b:
                    raise ValueError(f"schedule[{i}] cannot read the cache of entry {e.cache_of}: "
                                     f"their key/value needs differ ({a} vs {b})")

    def _kv_spec(self, layer: int) -> Optional[P.KVCacheSpec]:
        mixer = self.layers[layer].mixer
        return mixer.kv_spec() if mixer is not None else None

    def bindings(self) -> List[Binding]:
        return list(self._bindings)

    def parts(self) -> List[P.Part]:
        seen, out = set(), []
        for b in self._bindings:
            if id(b.part) not in seen:
                seen.add(id(b.part))
                out.append(b.part)
        return out

    def all_parts(self) -> List[P.Part]:
        out: List[P.Part] = [self.embedding]
        if self.position is not None:
            out.append(self.position)
        for blk in self.layers:
            out.extend(blk.parts().values())
            pos = getattr(blk.mixer, "position", None)
            if pos is not None:
                out.append(pos)
        out += [self.final_norm, self.head]
        return out

    def prepare(self, dtype: torch.dtype, device: torch.device) -> None:
        self.dtype, self.device = dtype, device
        for part in self.all_parts():
            part.prepare(dtype, device)

    # ------------------------------------------------------------------ what the cache manager must provide
    def kv_needs(self) -> List[Tuple[int, P.KVCacheSpec]]:
        """(schedule index, need) for every run that owns paged keys and values."""
        out = []
        for i, e in enumerate(self.schedule):
            spec = self._kv_spec(e.layer)
            if spec is not None and e.cache_of is None:
                out.append((i, spec))
        return out

    def state_needs(self) -> List[Tuple[int, P.StateSpec]]:
        """(schedule index, need) for every run whose mixer keeps per-request state of fixed size."""
        out = []
        for i, e in enumerate(self.schedule):
            mixer = self.layers[e.layer].mixer
            spec = mixer.state_spec() if mixer is not None else None
            if spec is not None:
                out.append((i, spec))
        return out

    def capture_safe(self) -> bool:
        """Whether a step of this model may be captured in a CUDA graph: every mixer says so."""
        return all(getattr(blk.mixer, "capture_safe", True) for blk in self.layers if blk.mixer is not None)

    def step_planners(self) -> Dict[str, object]:
        """name -> factory of the per-step plans that the model's parts ask for (parts that give the
        same name share one plan a step)."""
        out: Dict[str, object] = {}
        for part in self.all_parts():
            got = part.step_planner()
            if got is not None:
                out.setdefault(got[0], got[1])
        return out

    def reserve(self, workspace: P.Workspace, limits: P.StepLimits) -> None:
        """Size the scratch of the forward pass and of every part for the largest step.  Logits are
        sized for one row per batch entry (what generation asks for); a step that wants more (a
        replay that asks for every position) makes them grow, which drops captured graphs."""
        workspace.reserve("model.residual", limits.max_rows * self.width, torch.float32)
        n = max(limits.max_entries, 1)
        workspace.reserve("model.final", n * self.width, limits.dtype)
        workspace.reserve("model.logits", n * _round_up(self.vocab_size, 16), torch.float32)
        for part in self.all_parts():
            part.reserve(workspace, limits)
        for blk in self.layers:
            blk.reserve(workspace, limits)

    @property
    def vocab_size(self) -> int:
        return self.head.vocab_size

    @property
    def max_positions(self) -> Optional[int]:
        return self.spec.max_positions

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: P.StepContext, caches: Dict[int, P.KVCacheView], states: Dict[int, torch.Tensor],
                logit_rows: Optional[torch.Tensor], n_logits: int) -> Optional[torch.Tensor]:
        """Run the rows of ``ctx`` through the model; return float32 logits [n_logits, vocab] of the
        rows listed in ``logit_rows`` (None if none are wanted)."""
        ws = ctx.workspace
        x = ws.get("model.residual", (ctx.max_rows, self.width), torch.float32)
        self.embedding.forward(ctx, x, self.position)
        for i, e in enumerate(self.schedule):
            owner = i if e.cache_of is None else e.cache_of
            ctx.layer = i
            self.layers[e.layer].forward(x, ctx, caches.get(owner), states.get(i), e.cache_of is None, self.dtype)
        ctx.layer = -1
        if n_logits <= 0:
            return None
        # the final norm runs on the wanted rows only; the head folds it into its product where it can
        h = self.final_norm.as_input(x, ctx, self.dtype, rows=logit_rows) if getattr(
            self.head, "takes_norm_input", False) else None
        if h is None:
            h = ws.get("model.final", (n_logits, self.width), self.dtype)
            self.final_norm.forward(x, h, n_logits, rows=logit_rows)
        pitch = _round_up(self.vocab_size, 16)
        logits = ws.get("model.logits", (n_logits, pitch), torch.float32)
        self.head.forward(h, logits[:, :self.vocab_size], n_logits, ctx)
        return logits[:, :self.vocab_size]

"""Byte and FLOP counts of a step, taken from the built model and its cache, never from a
configuration's field names: another architecture is measured by the same code.

The counting rules are the reference's (crates/cli/src/bench.rs:261-271,
crates/cli/src/metal_batch.rs:113-114,157-160, crates/core/src/config.rs:29-48):
  * a decode step has to read every weight it uses once, plus the cached keys and values of the
    live requests; tables that are touched one row per token (token and position embeddings) are
    left out unless the same tensor is also the head's matrix;
  * matrix FLOPs are 2 per weight element and row for every run of a layer, the head counted per
    logits row, plus what each mixer says it spends per visible key.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence

import torch

from .parts import base as P


def _unique_tensors(model) -> Dict[int, tuple]:
    """data_ptr -> (tensor, streamed): every bound parameter once (a tied tensor is one tensor);
    ``streamed`` says that a step reads all of it."""
    out: Dict[int, tuple] = {}
    for b in model.bindings():
        t = b.part.params.get(b.spec.key) if getattr(b.part, "params", None) else None
        if t is None:
            continue
        streamed = b.spec.kind in (P.MATRIX, P.VECTOR) or isinstance(b.part, P.Head)
        old = out.get(t.data_ptr())
        out[t.data_ptr()] = (t, streamed or (old is not None and old[1]))
    return out


def parameter_count(model) -> int:
    """All parameters, a tied tensor counted once (crates/core/src/config.rs:29-39)."""
    return sum(t.numel() for t, _ in _unique_tensors(model).values())


def parameter_count_of_spec(model) -> int:
    """The same from the parts' declared shapes, for a model whose weights are not loaded: tensors
    are told apart by their checkpoint names."""
    seen: Dict[str, int] = {}
    for b in model.bindings():
        n = 1
        for s in b.spec.shape:
            n *= int(s)
        seen[b.ref.name] = n
    return sum(seen.values())


def weight_bytes_per_step(model) -> int:
    """Bytes of the weights a decode step streams, each tensor once."""
    return sum(t.numel() * t.element_size() for t, streamed in _unique_tensors(model).values() if streamed)


def kv_bytes_per_position(cache) -> List[tuple]:
    """(bytes per cached position over all layers of the group, window) for every cache group."""
    itemsize = torch.empty(0, dtype=cache.dtype).element_size()
    return [(g.bytes_per_page(itemsize) // cache.page_size, g.spec.window) for g in cache.groups]


def kv_bytes(cache, contexts: Iterable[float]) -> float:
    """Bytes of cached keys and values that rows seeing ``contexts`` positions have to read."""
    total = 0.0
    groups = kv_bytes_per_position(cache)
    for n in contexts:
        for per_pos, window in groups:
            total += per_pos * (min(n, window) if window else n)
    return total


def matrix_flops_per_row(model) -> float:
    """FLOPs of the layers' matrix products for one row, every run of the schedule counted."""
    total = 0.0
    for e in model.schedule:
        for part in model.layers[e.layer].parts().values():
            total += part.matrix_flops_per_row()
    return total


def step_flops(model, row_contexts: Sequence[int], n_logit_rows: int) -> float:
    """FLOPs of one step whose rows see ``row_contexts`` keys each and that wants ``n_logit_rows``
    rows of logits."""
    flops = matrix_flops_per_row(model) * len(row_contexts)
    flops += model.head.matrix_flops_per_row() * n_logit_rows
    keys = float(sum(row_contexts))
    for e in model.schedule:
        mixer = model.layers[e.layer].mixer
        if mixer is not None:
            w = mixer.kv_spec().window if mixer.kv_spec() is not None else 0
            k = float(sum(min(c, w) for c in row_contexts)) if w else keys
            flops += mixer.flops_per_key() * k
    return flops

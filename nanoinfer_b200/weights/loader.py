"""Loads a model's parameters from ``model.safetensors`` by tensor name.

The reference asks for each tensor by name with its expected shape and stops at the first
problem (``MissingTensor``, "expected shape ..., got ...": crates/core/src/safetensors.rs:72-93,
crates/core/src/weights.rs:77-108).  Here the whole file is checked against the model first,
and ONE error lists every missing tensor, every unexpected tensor and every wrong shape.

How tensors are held on the device:
  * matrices and lookup tables: the engine's dtype (bfloat16 or float32);
  * vectors (biases, norm scales and shifts): 32-bit floats, whatever the file stores;
  * integer tables: int32.
A tensor the file stores [in, out] (Conv1D) is transposed to [out, in] once, here
(crates/core/src/weights.rs:48-57).

On a CUDA device the bytes take the short way (the reference maps the file and reads it in
place: crates/cli/src/main.rs:91-106): from the memory map into one of two pinned staging
buffers, from there to the device with an asynchronous copy, and a kernel converts and
transposes them into the tensor the engine computes with, while the host fills the other
buffer.  No tensor is converted, transposed or even held whole on the host.
"""
from __future__ import annotations

import math
import os
import re
from typing import Dict, List, Tuple

import torch

from ..models.model import Binding, Model
from ..parts.base import INT_TABLE, MATRIX, TABLE, VECTOR
from .safetensors_io import SafetensorsFile

_FLOAT = {"F32", "F16", "BF16", "F64"}
_INT = {"I64", "I32", "I16", "I8", "U8"}


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every problem found."""

    def __init__(self, path: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"{path} does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def stored_shape(b: Binding) -> Tuple[int, ...]:
    shape = tuple(b.spec.shape)
    if b.ref.transposed:
        if len(shape) != 2:
            raise ValueError(f"{b.where}.{b.spec.key}: only matrices can be stored transposed")
        return (shape[1], shape[0])
    return shape


def _pick_prefix(model: Model, names) -> str:
    names = set(names)
    wanted = {b.ref.name for b in model.bindings()}
    best, best_hits = "", -1
    for prefix in model.spec.name_prefixes:
        hits = sum(1 for n in wanted if prefix + n in names)
        if hits > best_hits:
            best, best_hits = prefix, hits
    return best


def check_weights(model: Model, st: SafetensorsFile) -> str:
    """Compare the file's header with the model; raise WeightError or return the name prefix in use."""
    prefix = _pick_prefix(model, st.names())
    missing, wrong = [], []
    used = set()
    seen = set()
    for b in model.bindings():
        name = prefix + b.ref.name
        used.add(name)
        key = (name, b.ref.transposed, b.spec.kind, tuple(b.spec.shape))
        if key in seen:
            continue
        seen.add(key)
        if name not in st.tensors:
            if name not in missing:
                missing.append(name)
            continue
        info = st.info(name)
        want = stored_shape(b)
        if tuple(info.shape) != want:
            wrong.append(f"{name}: expected shape {list(want)}, got {list(info.shape)}")
        elif b.spec.kind == INT_TABLE and info.dtype not in _INT:
            wrong.append(f"{name}: expected an integer tensor, got {info.dtype}")
        elif b.spec.kind != INT_TABLE and info.dtype not in _FLOAT:
            wrong.append(f"{name}: expected a floating-point tensor, got {info.dtype}")
    ignorable = [re.compile(p) for p in model.spec.ignorable]
    unexpected = []
    for name in sorted(st.names()):
        if name in used:
            continue
        bare = name[len(prefix):] if prefix and name.startswith(prefix) else name
        if any(p.fullmatch(bare) for p in ignorable):
            continue
        unexpected.append(name)
    if missing or unexpected or wrong:
        raise WeightError(st.path, sorted(missing), unexpected, wrong)
    return prefix


#: bytes of each of the two pinned staging buffers of the streamed load
STAGING_BYTES = 64 << 20
_STREAMED = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16}


class _Stager:
    """Two pinned host buffers and their device twins, used by turns: while the device copies and
    converts one, the host fills the other from the memory map."""

    def __init__(self, device: torch.device, nbytes: int = 0):
        nbytes = self.nbytes = nbytes or STAGING_BYTES
        self.host = [torch.empty(nbytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.dev = [torch.empty(nbytes, dtype=torch.uint8, device=device) for _ in range(2)]
        self.done = [torch.cuda.Event() for _ in range(2)]
        self.turn = 0
        self.bytes_moved = 0

    def load(self, st: SafetensorsFile, name: str, dst: torch.Tensor, transposed: bool) -> None:
        """The file's tensor ``name`` ([rows, cols] as stored, or a vector) into ``dst``."""
        from ..kernels import ops

        info = st.info(name)
        src_dtype = _STREAMED[info.dtype]
        rows, cols = info.shape if len(info.shape) == 2 else (1, math.prod(info.shape))
        raw = st.raw(name)
        item = raw.size // max(1, rows * cols)
        out = dst if dst.dim() == 2 else dst.view(1, -1)
        per = max(1, self.nbytes // (cols * item))           # rows of the file per piece
        for r0 in range(0, rows, per):
            n = min(per, rows - r0)
            k = self.turn
            self.turn ^= 1
            self.done[k].synchronize()                          # the device is through with this buffer
            nb = n * cols * item
            self.host[k].numpy()[:nb] = raw[r0 * cols * item:r0 * cols * item + nb]
            self.dev[k][:nb].copy_(self.host[k][:nb], non_blocking=True)
            ops.convert_rows(self.dev[k], src_dtype, n, cols, out, r0, transposed)
            self.done[k].record()
            self.bytes_moved += nb


def load_weights(model: Model, model_dir: str, dtype: torch.dtype, device: torch.device) -> None:
    """Check ``model_dir/model.safetensors`` against ``model``, then bind every parameter."""
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"engine dtype must be float32 or bfloat16, got {dtype}")
    path = os.path.join(model_dir, "model.safetensors")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path}: no such file")
    st = SafetensorsFile(path)
    try:
        prefix = check_weights(model, st)
        loaded: Dict[Tuple, torch.Tensor] = {}
        per_part: Dict[int, Dict[str, torch.Tensor]] = {}
        parts = {}
        stager = _Stager(device) if device.type == "cuda" else None
        for b in model.bindings():
            key = (b.ref.name, b.ref.transposed, b.spec.kind)
            if key not in loaded and stager is not None and b.spec.kind != INT_TABLE \
                    and st.info(prefix + b.ref.name).dtype in _STREAMED and len(b.spec.shape) <= 2:
                # the short way: bytes as stored to the device, converted and transposed there
                want = dtype if b.spec.kind in (MATRIX, TABLE) else torch.float32
                dst = torch.empty(tuple(b.spec.shape), dtype=want, device=device)
                stager.load(st, prefix + b.ref.name, dst, b.ref.transposed)
                loaded[key] = dst
            if key not in loaded:
                t = st.tensor(prefix + b.ref.name)
                if b.ref.transposed:
                    t = t.t()
                if b.spec.kind in (MATRIX, TABLE):
                    t = t.to(dtype)
                elif b.spec.kind == VECTOR:
                    t = t.to(torch.float32)
                else:
                    t = t.to(torch.int32)
                loaded[key] = t.contiguous().to(device)
            per_part.setdefault(id(b.part), {})[b.spec.key] = loaded[key]
            parts[id(b.part)] = b.part
        for pid, params in per_part.items():
            parts[pid].bind(params)
        for part in model.all_parts():
            if not hasattr(part, "params"):
                part.bind({})
        if stager is not None:
            torch.cuda.synchronize(device)     # the map is closed below: every copy out of it has been made
    finally:
        st.close()
    model.prepare(dtype, device)

"""The random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Every tensor the architecture's model asks for is filled from its parameter's declared rule:
N(0, std) for matrices, tables and biases, 1 + N(0, std) for norm scales.  The values of a
tensor depend on the seed and on the tensor's name only, so adding a layer does not change
the others.  Tensors are written in the checkpoint's own layout ([in, out] where the
architecture says the file stores them transposed).  The reference has only a unit-test
helper of this kind (an LCG filling a tiny model, crates/core/src/stages/mod.rs:705-734).
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict

import torch

from ..config.base import ModelConfig
from ..models.model import Model
from ..parts.base import INIT_NORMAL, INIT_ONE_PLUS_NORMAL, INIT_ZEROS, INT_TABLE
from .loader import stored_shape
from .safetensors_io import write_safetensors


def random_tensors(model: Model, seed: int, std: float = 0.02, dtype: torch.dtype = torch.float32
                   ) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for b in model.bindings():
        name = b.ref.name
        if name in out:
            continue
        gen = torch.Generator(device="cpu")
        gen.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
        shape = stored_shape(b)
        if b.spec.kind == INT_TABLE:
            out[name] = torch.zeros(shape, dtype=torch.int32)
            continue
        if b.spec.init == INIT_ZEROS:
            t = torch.zeros(shape, dtype=torch.float32)
        else:
            t = torch.randn(shape, generator=gen, dtype=torch.float32) * std
            if b.spec.init == INIT_ONE_PLUS_NORMAL:
                t = t + 1.0
            elif b.spec.init != INIT_NORMAL:
                raise ValueError(f"unknown init rule {b.spec.init!r} for {name}")
        out[name] = t.to(dtype)
    return out


def write_random_model(config: ModelConfig, out_dir: str, seed: int, dtype: torch.dtype = torch.float32,
                       std: float = 0.02) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns ``out_dir``."""
    from ..registry import get_architecture

    arch = get_architecture(config.architecture)
    model = Model(arch.build_spec(config), config)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config.to_dict(), fh, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(model, seed, std, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir

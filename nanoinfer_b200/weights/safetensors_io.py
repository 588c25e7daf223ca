"""Reading and writing the safetensors container.

The format is the one the reference parses (crates/core/src/safetensors.rs:1-63):
a little-endian u64 header length, a JSON header mapping each tensor name to
``{dtype, shape, data_offsets}`` (offsets relative to the end of the header,
``__metadata__`` skipped), then the raw bytes.  The reference accepts F32 only
(safetensors.rs:78-81); this reader also takes BF16, F16 and the integer types,
and returns torch tensors that view a memory map of the file.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


# name -> (numpy storage dtype, torch dtype)
_DTYPES = {
    "F32": (np.dtype("<f4"), torch.float32),
    "F64": (np.dtype("<f8"), torch.float64),
    "F16": (np.dtype("<f2"), torch.float16),
    "BF16": (np.dtype("<u2"), torch.bfloat16),  # stored as raw 16-bit words
    "I64": (np.dtype("<i8"), torch.int64),
    "I32": (np.dtype("<i4"), torch.int32),
    "I16": (np.dtype("<i2"), torch.int16),
    "I8": (np.dtype("i1"), torch.int8),
    "U8": (np.dtype("u1"), torch.uint8),
    "BOOL": (np.dtype("u1"), torch.bool),
}
_TORCH_TO_NAME = {v[1]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorInfo:
    dtype: str
    shape: Tuple[int, ...]
    start: int
    end: int

    @property
    def is_32bit_float(self) -> bool:
        return self.dtype == "F32"


class SafetensorsFile:
    """A parsed, memory-mapped safetensors file.  Nothing is copied until asked for."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as fh:
            try:
                self._map = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
            except ValueError:
                raise SafetensorsError(f"{path}: file too small") from None
        buf = self._map
        if len(buf) < 8:
            raise SafetensorsError(f"{path}: file too small")
        (n,) = struct.unpack("<Q", buf[:8])
        if 8 + n > len(buf):
            raise SafetensorsError(f"{path}: truncated header")
        try:
            header = json.loads(bytes(buf[8:8 + n]).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not an object")
        self._data_start = 8 + n
        data_len = len(buf) - self._data_start
        self.tensors: Dict[str, TensorInfo] = {}
        for name, v in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(v, dict):
                raise SafetensorsError(f"{path}: entry {name!r} is not an object")
            dtype, shape, offs = v.get("dtype"), v.get("shape"), v.get("data_offsets")
            if not isinstance(dtype, str):
                raise SafetensorsError(f"{path}: {name}: missing dtype")
            if not isinstance(shape, list) or not all(isinstance(d, int) and d >= 0 for d in shape):
                raise SafetensorsError(f"{path}: {name}: missing or bad shape")
            if (not isinstance(offs, list) or len(offs) != 2
                    or not all(isinstance(o, int) and o >= 0 for o in offs)):
                raise SafetensorsError(f"{path}: {name}: missing or bad data_offsets")
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: {name}: dtype {dtype} is not supported")
            start, end = offs
            if start > end or end > data_len:
                raise SafetensorsError(f"{path}: {name}: data out of bounds")
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if end - start != count * _DTYPES[dtype][0].itemsize:
                raise SafetensorsError(f"{path}: {name}: byte length does not match shape {shape}")
            self.tensors[name] = TensorInfo(dtype, tuple(shape), start, end)

    def names(self) -> Iterable[str]:
        return self.tensors.keys()

    def info(self, name: str) -> TensorInfo:
        return self.tensors[name]

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor as stored (a copy, so that the map may be closed)."""
        info = self.tensors[name]
        np_dtype, torch_dtype = _DTYPES[info.dtype]
        count = int(np.prod(info.shape, dtype=np.int64)) if info.shape else 1
        arr = np.frombuffer(self._map, dtype=np_dtype, count=count, offset=self._data_start + info.start)
        t = torch.from_numpy(arr.copy())
        if info.dtype == "BF16":
            t = t.view(torch.bfloat16)
        elif info.dtype == "BOOL":
            t = t.to(torch.bool)
        return t.reshape(info.shape)

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as they lie in the memory map (no copy; valid until ``close``)."""
        info = self.tensors[name]
        return np.frombuffer(self._map, dtype=np.uint8, count=info.end - info.start,
                             offset=self._data_start + info.start)

    def close(self) -> None:
        self._map.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) in name order, header padded to 8 bytes."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    blobs = []
    offset = 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"{name}: dtype {t.dtype} cannot be stored")
        if t.dtype == torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        elif t.dtype == torch.bool:
            raw = t.to(torch.uint8).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {
            "dtype": _TORCH_TO_NAME[t.dtype],
            "shape": list(t.shape),
            "data_offsets": [offset, offset + len(raw)],
        }
        offset += len(raw)
        blobs.append(raw)
    hdr = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hdr += b" " * ((8 - len(hdr) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(hdr)))
        fh.write(hdr)
        for raw in blobs:
            fh.write(raw)

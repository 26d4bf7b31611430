"""Reading and writing the safetensors container, by tensor name.

The format: 8 bytes little-endian header length, a JSON object
{name: {"dtype", "shape", "data_offsets": [begin, end]}} (plus an optional
"__metadata__"), then the raw little-endian data.  The reference reads every
tensor of every shard into a dict by name (engine/model.py:67-75); here the
file is mapped and a tensor is materialised only when it is asked for.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


class SafetensorsFile:
    """A mapped safetensors file.  ``entries`` maps name -> (dtype, shape)."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise FileNotFoundError(f"{self.path} not found: a model folder holds config.json and model.safetensors")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: {size} bytes is too short for a safetensors header")
        self._file = open(self.path, "rb")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len > size - 8:
            raise SafetensorsError(f"{self.path}: header length {header_len} exceeds the file ({size} bytes); truncated?")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({exc})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header must be a JSON object")
        self._data_start = 8 + header_len
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = {}
        self._spans: Dict[str, Tuple[int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, width = _DTYPES[info["dtype"]]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(v) for v in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: bad header entry for {name!r}: {info!r}") from None
            count = 1
            for s in shape:
                count *= s
            if begin < 0 or end < begin or end - begin != count * width:
                raise SafetensorsError(f"{self.path}: {name!r} spans {end - begin} bytes but shape {shape} "
                                       f"of {info['dtype']} needs {count * width}")
            if end > data_len:
                raise SafetensorsError(f"{self.path}: {name!r} ends at byte {end} of {data_len} data bytes; truncated?")
            self.entries[name] = (dtype, shape)
            self._spans[name] = (begin, end)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def get(self, name: str) -> torch.Tensor:
        """The tensor as stored (a view of the mapping; copy it before the file is closed)."""
        dtype, shape = self.entries[name]
        begin, end = self._spans[name]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._data_start + begin)
        return flat.view(shape)

    def close(self) -> None:
        self.entries = {}
        try:
            if self._map is not None:
                self._map.close()
        except BufferError:
            pass  # a tensor still views the mapping; the OS unmaps it when that goes
        self._file.close()


def write_safetensors(path, tensors: Iterable[Tuple[str, Tuple[torch.dtype, Tuple[int, ...]]]], produce) -> None:
    """Write a safetensors file without holding every tensor at once.

    ``tensors``: (name, (dtype, shape)) in file order; ``produce(name)`` returns
    the tensor (any device) when its turn comes.
    """
    header = {}
    offset = 0
    order = []
    for name, (dtype, shape) in tensors:
        if dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {dtype} for {name!r}")
        count = 1
        for s in shape:
            count *= s
        nbytes = count * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        order.append((name, dtype, tuple(shape)))
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, dtype, shape in order:
            t = produce(name)
            if t.dtype != dtype or tuple(t.shape) != shape:
                raise SafetensorsError(f"{name!r}: produced {t.dtype} {tuple(t.shape)}, declared {dtype} {shape}")
            t = t.detach().to("cpu").contiguous()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")

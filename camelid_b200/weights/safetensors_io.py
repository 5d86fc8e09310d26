"""Reader and writer of the safetensors container (no third-party package).

Layout: 8 bytes little-endian header length, a JSON header mapping tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}``, then the payload; offsets are
relative to the payload. The checks are those the reference makes on headers
(src/model_source.rs:818-896): offsets inside the payload, byte count equal to
prod(shape) * element size, no overlap, no duplicate names across shards
(src/model_source.rs:737-763, :786-800).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Iterable

import torch

from ..errors import SafetensorsError

DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class SafetensorsFile:
    """One file, memory-mapped; ``tensor(name)`` is a zero-copy CPU view of the map."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a safetensors header")
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be an object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + hlen
        payload = size - self._base
        self.entries: dict[str, dict] = {}
        spans = []
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], [int(s) for s in info["shape"]], info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}") from None
            if dt not in DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            if not (0 <= b <= e <= payload):
                raise SafetensorsError(f"{path}: tensor {name!r} offsets [{b}, {e}) lie outside the payload ({payload} bytes)")
            if e - b != _numel(shape) * DTYPES[dt][1]:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} holds {e - b} bytes but shape {shape} of {dt} needs {_numel(shape) * DTYPES[dt][1]}")
            self.entries[name] = {"dtype": dt, "shape": shape, "begin": b, "end": e}
            spans.append((b, e, name))
        spans.sort()
        for (b0, e0, n0), (b1, _e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: tensors {n0!r} and {n1!r} overlap")

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> list[int]:
        return self.entries[name]["shape"]

    def dtype(self, name: str) -> torch.dtype:
        return DTYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        dt = DTYPES[e["dtype"]][0]
        n = _numel(e["shape"])
        if n == 0:
            return torch.empty(e["shape"], dtype=dt)
        # A read-only map: torch warns about non-writable buffers, the view is never written.
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(self._map, dtype=dt, count=n, offset=self._base + e["begin"])
        return t.reshape(e["shape"])

    def close(self):
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass            # views of the map are still alive; the map goes with them
        self._f.close()


class ModelFiles:
    """All tensors of a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` lists."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        if os.path.isfile(index):
            with open(index) as f:
                weight_map = json.load(f).get("weight_map", {})
            paths = sorted({os.path.join(folder, p) for p in weight_map.values()})
        elif os.path.isfile(single):
            paths = [single]
        else:
            raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json exists")
        self.files = [SafetensorsFile(p) for p in paths]
        self._where: dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.names():
                if name in self._where:
                    raise SafetensorsError(f"tensor {name!r} occurs in both {self._where[name].path} and {f.path}")
                self._where[name] = f

    def names(self) -> list[str]:
        return list(self._where)

    def shape(self, name: str) -> list[int]:
        return self._where[name].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._where[name].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

    def close(self):
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write CPU tensors in name order, each starting on an 8-byte boundary of the payload."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)

"""Reading and writing safetensors files, without any library for the format.

A file is: an 8-byte little-endian length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the tensors' bytes.  AIR's own models are GGUF files mapped read-only
(src/model/storage.cpp:22-66); this reader maps the file the same way and hands out
views, and refuses headers whose ranges leave the file or overlap.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A read-only mapping of one file: ``names()``, ``info(name)``, ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e.strerror}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than a header length")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} is beyond the file's {size} bytes")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be an object")
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + n
        self._data_size = size - self._base
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        ranges = []
        for name, e in header.items():
            try:
                dt, shape, (lo, hi) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for '{name}'") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has dtype {dt}, which is not supported")
            count = 1
            for s in shape:
                count *= s
            if not (0 <= lo <= hi <= self._data_size):
                raise SafetensorsError(f"{path}: tensor '{name}' lies outside the file")
            if hi - lo != count * _DTYPES[dt][1]:
                raise SafetensorsError(f"{path}: tensor '{name}' has {hi - lo} bytes, its shape needs "
                                       f"{count * _DTYPES[dt][1]}")
            self._entries[name] = (dt, shape, lo, hi)
            if hi > lo:
                ranges.append((lo, hi, name))
        ranges.sort()
        for (_, hi0, n0), (lo1, _, n1) in zip(ranges, ranges[1:]):
            if lo1 < hi0:
                raise SafetensorsError(f"{path}: tensors '{n0}' and '{n1}' overlap")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def info(self, name: str):
        """(torch dtype, shape) of a tensor."""
        dt, shape, _, _ = self._entries[name]
        return _DTYPES[dt][0], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapping (do not write to it)."""
        dt, shape, lo, hi = self._entries[name]
        if hi == lo:
            return torch.empty(shape, dtype=_DTYPES[dt][0])
        view = memoryview(self._map)[self._base + lo:self._base + hi]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the buffer is read-only; the tensor is only read
            return torch.frombuffer(view, dtype=_DTYPES[dt][0]).reshape(shape)

    def close(self):
        # Tensors may still view the mapping; it is released with the last of them.
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = list(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot write dtype {t.dtype} of '{name}'")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().to("cpu").contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)

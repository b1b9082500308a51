"""Reading and writing safetensors files (8-byte little-endian header length, a JSON header
of name -> {dtype, shape, data_offsets}, then the raw little-endian data).

catena-models has the same reader for its safetensors models (src/weights.rs:33-120): header
parse, duplicate and range checks, lookup by tensor name.  Files are memory-mapped; a tensor
is materialised only when it is asked for.
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np
import torch

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def _numel(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except FileNotFoundError as exc:
            raise SafetensorsError(f"{path}: no such file") from exc
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} runs past the end of the file")
        try:
            pairs = json.loads(self._fh.read(hlen).decode("utf-8"), object_pairs_hook=list)
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not valid JSON ({exc})") from exc
        self.data_start = 8 + hlen
        self.metadata = {}
        self.entries = {}
        spans = []
        for name, info in pairs:
            if name == "__metadata__":
                self.metadata = dict(info)
                continue
            if name in self.entries:
                raise SafetensorsError(f"{path}: tensor '{name}' appears twice")
            info = dict(info)
            dtype, shape = info.get("dtype"), info.get("shape")
            begin, end = info.get("data_offsets", (None, None))
            if dtype not in DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype!r}")
            width = torch.empty((), dtype=DTYPES[dtype]).element_size()
            if begin is None or end is None or begin > end or self.data_start + end > size:
                raise SafetensorsError(f"{path}: tensor '{name}' lies outside the file")
            if end - begin != _numel(shape) * width:
                raise SafetensorsError(f"{path}: tensor '{name}' has {end - begin} bytes for shape {shape} {dtype}")
            self.entries[name] = (dtype, tuple(int(s) for s in shape), begin, end)
            spans.append((begin, end, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: tensors '{n0}' and '{n1}' overlap")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return list(self.entries)

    def info(self, name):
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name):
        """A CPU tensor with the stored dtype (a copy; the map can be closed afterwards)."""
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=DTYPES[dtype])
        raw = np.frombuffer(self._map, dtype=np.uint8, count=end - begin, offset=self.data_start + begin)
        return torch.from_numpy(raw.copy()).view(DTYPES[dtype]).reshape(shape)

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None
        self._fh.close()


def write_safetensors(path, tensors, metadata=None):
    """Write {name: CPU tensor} in name order, data 64-byte aligned within the file."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((-(8 + len(blob))) % 64)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                fh.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)

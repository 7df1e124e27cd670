"""Reader and writer of the safetensors container, written for this package.

Layout: 8 bytes little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": ...}``,
then the raw little-endian tensor bytes.  The reader maps the file and hands out
tensors that view the mapping (no copy until the caller moves them).
"""
from __future__ import annotations

import json
import mmap
import struct
from typing import Dict, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A mapped safetensors file: ``names()``, ``info(name)`` and ``tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{path}: truncated (no header length)")
            (n,) = struct.unpack("<Q", head)
            f.seek(0, 2)
            size = f.tell()
            if n <= 0 or 8 + n > size:
                raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
            f.seek(8)
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        self._base = 8 + n
        self.metadata = header.pop("__metadata__", None)
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        spans = []
        for name, e in header.items():
            if e.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unknown dtype {e.get('dtype')!r}")
            dt, width = _DTYPES[e["dtype"]]
            shape = tuple(int(x) for x in e["shape"])
            b, en = (int(x) for x in e["data_offsets"])
            count = int(np.prod(shape)) if shape else 1
            if en - b != count * width:
                raise SafetensorsError(f"{path}: tensor '{name}' of shape {list(shape)} {e['dtype']} needs "
                                       f"{count * width} bytes, its offsets give {en - b}")
            if b < 0 or self._base + en > size:
                raise SafetensorsError(f"{path}: tensor '{name}' ends at byte {self._base + en}, file has {size} (truncated?)")
            spans.append((b, en, name))
            self._entries[name] = (dt, shape, b, en)
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{path}: tensors '{n0}' and '{n1}' overlap")

    def names(self):
        return list(self._entries)

    def info(self, name: str):
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, e = self._entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._map)[self._base + b:self._base + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the mapping is read-only; tensors from it are never written
            t = torch.frombuffer(buf, dtype=dt)
        return t.view(shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: dict = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = list(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ('{name}')")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")

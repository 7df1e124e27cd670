"""Binds checkpoint tensors to the model's declared weights, by name.

Files: ``model.safetensors`` alone, else the shards of
``model.safetensors.index.json`` (its ``weight_map`` gives name -> file), as in
cklxx/arle's loader (infer/src/weight_loader.rs:27-61, :102-120).  Unlike that
loader, which assumes bfloat16 bytes and checks lengths only
(crates/cuda-kernels/src/tensor.rs:1146-1152), the stored dtype and shape of each
tensor are read and checked, and all problems are reported in ONE error: the
missing names, the unexpected names and the wrong shapes together.

Precision kept in memory: floating tensors stored in 16 bits become bfloat16,
tensors stored in 32 bits stay float32, integer tables become int32.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Sequence

import torch

from ..parts.base import WeightDecl
from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """Raised once per load with everything that is wrong with the checkpoint."""

    def __init__(self, where, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.other = list(wrong_shape), list(other)
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name}: expected {list(want)}, got {list(got)}")
        lines.extend(f"  {o}" for o in self.other)
        super().__init__("\n".join(lines))


def _open_files(model_dir: str):
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return {None: SafetensorsFile(single)}, None
    if os.path.isfile(index):
        with open(index) as f:
            idx = json.load(f)
        wm = idx.get("weight_map")
        if not isinstance(wm, dict):
            raise SafetensorsError(f"{index}: missing 'weight_map'")
        files = {fn: SafetensorsFile(os.path.join(model_dir, fn)) for fn in sorted(set(wm.values()))}
        return files, wm
    raise FileNotFoundError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")


def kept_dtype(stored: torch.dtype, integer: bool) -> torch.dtype:
    if integer or not stored.is_floating_point:
        return torch.int32
    return torch.float32 if stored in (torch.float32, torch.float64) else torch.bfloat16


def load_weights(model_dir: str, decls: Sequence[WeightDecl], ignored: Iterable[str] = (),
                 device="cpu") -> Dict[str, torch.Tensor]:
    files, weight_map = _open_files(model_dir)
    where = {}
    twice = []
    for fn, f in files.items():
        for n in f.names():
            if n in where:
                twice.append(f"tensor {n} is stored in two files: {os.path.basename(where[n].path)} and {os.path.basename(f.path)}")
            where[n] = f
    wanted = {d.name: d for d in decls}
    ignored = set(ignored)
    missing = [n for n in wanted if n not in where]
    unexpected = sorted(n for n in where if n not in wanted and n not in ignored)
    wrong = []
    for n, d in wanted.items():
        if n in where:
            _, shape = where[n].info(n)
            if tuple(shape) != tuple(d.shape):
                wrong.append((n, d.shape, shape))
    if missing or unexpected or wrong or twice:
        raise WeightError(model_dir, missing, unexpected, wrong, twice)
    out = {}
    for n, d in wanted.items():
        t = where[n].tensor(n)
        out[n] = t.to(device=device, dtype=kept_dtype(t.dtype, d.integer))
    return out

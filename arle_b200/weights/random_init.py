"""Random-weights mode: a model folder (config.json + model.safetensors) from a
configuration and a seed, or the same tensors made directly on a device.

Every tensor gets a generator of its own, seeded from (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or on their order.
Projection and embedding matrices are N(0, sigma); norm gains are 1 + U(-a, a).
cklxx/arle has no random-weights mode on its inference path; its training side
initialises by name-seeded N(0, 0.02) with all-ones norms
(crates/train/src/qwen3.rs:877-935), which is where sigma's default comes from.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Sequence

import torch

from ..parts.base import WeightDecl
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(decls: Sequence[WeightDecl], seed: int, sigma: float = 0.02, gain_jitter: float = 0.1,
                   dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    out = {}
    for d in decls:
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, d.name))
        if d.integer:
            t = torch.zeros(d.shape, dtype=torch.int32, device=device)
        elif d.init == "normal":
            t = torch.empty(d.shape, dtype=torch.float32, device=device).normal_(0.0, sigma, generator=g).to(dtype)
        elif d.init == "gain":
            t = (1.0 + (torch.rand(d.shape, dtype=torch.float32, device=device, generator=g) * 2 - 1) * gain_jitter).to(dtype)
        elif d.init == "zeros":
            t = torch.zeros(d.shape, dtype=dtype, device=device)
        else:
            raise ValueError(f"unknown init '{d.init}' for {d.name}")
        out[d.name] = t
    return out


def write_random_model(model_dir: str, config: dict, seed: int, sigma: float = 0.02, gain_jitter: float = 0.1,
                       dtype=torch.bfloat16) -> str:
    """Writes ``config.json`` (the given dict, which must name its architecture) and
    ``model.safetensors`` with seeded random weights.  Returns the folder."""
    from ..config import config_from_dict
    from ..parts.model import declared_weights

    spec = config_from_dict(config).to_model_spec()
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    tensors = random_tensors(declared_weights(spec), seed, sigma, gain_jitter, dtype)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed, "sigma": sigma, "gain_jitter": gain_jitter})
    return model_dir

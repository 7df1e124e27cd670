"""Random-weights mode: a model folder (config.json + model.safetensors) from a
configuration and a seed, or the same tensors made directly on a device.

Every tensor gets a key of its own, hashed from (seed, tensor name), and every
element a counter, so a tensor's values depend neither on which other tensors
exist, nor on their order, nor on the device they are made on.  Projection and
embedding matrices are N(0, sigma) (a sum of twelve uniforms); norm gains are
1 + U(-a, a).
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


# Counter-based random bits in integer arithmetic only, so that the same (seed, tensor
# name, element index) gives the same value on every device: element i of a tensor gets
# the 64-bit mix (the finaliser of SplitMix64) of key + i * odd constant.  Integer
# products wrap the same way on the CPU and on the GPU; no transcendental function,
# whose last bit may differ between libraries, is involved.
_GOLDEN = -7046029254386353131           # 0x9E3779B97F4A7C15 as a signed 64-bit integer
_MIX1 = -4658895280553007687             # 0xBF58476D1CE4E5B9
_MIX2 = -7723592293110705685             # 0x94D049BB133111EB
_CHUNK = 1 << 24


def _srl(x: torch.Tensor, k: int) -> torch.Tensor:
    """Logical shift right of int64 (torch's >> keeps the sign)."""
    return (x >> k) & ((1 << (64 - k)) - 1)


def _mix64(x: torch.Tensor) -> torch.Tensor:
    x = (x ^ _srl(x, 30)) * _MIX1
    x = (x ^ _srl(x, 27)) * _MIX2
    return x ^ _srl(x, 31)


def _bits(key: int, stream: int, start: int, n: int, device) -> torch.Tensor:
    """64 random bits for elements start .. start+n-1 of the tensor with this key; ``stream``
    numbers independent draws for the same element."""
    idx = torch.arange(start, start + n, dtype=torch.int64, device=device)
    offset = (key + (stream + 1) * 0x632BE59BD9B4E019) & 0x7FFFFFFFFFFFFFFF
    return _mix64(idx * _GOLDEN + offset)


def _normal_chunk(key: int, start: int, n: int, sigma: float, device) -> torch.Tensor:
    """Twelve 16-bit uniform integers per element, summed (Irwin-Hall): mean 12 * 32767.5,
    standard deviation 65536 to five digits, tails out to six sigma.  The sum is an exact
    integer; one float32 multiplication scales it."""
    total = torch.zeros(n, dtype=torch.int64, device=device)
    for stream in range(3):
        b = _bits(key, stream, start, n, device)
        total += (b & 0xFFFF) + (_srl(b, 16) & 0xFFFF) + (_srl(b, 32) & 0xFFFF) + _srl(b, 48)
    centred = (total * 2 - 12 * 65535).to(torch.float32)           # exact: |value| < 2^21
    return centred * (float(sigma) / 131072.0)


def _uniform_chunk(key: int, start: int, n: int, device) -> torch.Tensor:
    """U[0, 1) with 24 bits, exactly representable in float32."""
    return _srl(_bits(key, 0, start, n, device), 40).to(torch.float32) * (1.0 / 16777216.0)


def random_tensors(decls: Sequence[WeightDecl], seed: int, sigma: float = 0.02, gain_jitter: float = 0.1,
                   dtype=torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    """The tensors of ``decls`` with seeded random values, made on ``device``.  The values
    are the same bit for bit whatever the device, so a model made directly on the GPU is
    the model the same configuration and seed write to a folder."""
    out = {}
    for d in decls:
        key = _tensor_seed(seed, d.name)
        n = 1
        for s_ in d.shape:
            n *= int(s_)
        if d.integer:
            t = torch.zeros(d.shape, dtype=torch.int32, device=device)
        elif d.init == "zeros":
            t = torch.zeros(d.shape, dtype=dtype, device=device)
        elif d.init in ("normal", "gain"):
            flat = torch.empty(n, dtype=dtype, device=device)
            for at in range(0, n, _CHUNK):
                m = min(_CHUNK, n - at)
                if d.init == "normal":
                    v = _normal_chunk(key, at, m, sigma, device)
                else:
                    v = (_uniform_chunk(key, at, m, device) * 2.0 - 1.0) * float(gain_jitter) + 1.0
                flat[at:at + m] = v.to(dtype)
            t = flat.view(d.shape)
        else:
            raise ValueError(f"unknown init '{d.init}' for {d.name}")
        out[d.name] = t
    return out


def write_random_model(model_dir: str, config: dict, seed: int, sigma: float = 0.02, gain_jitter: float = 0.1,
                       dtype=torch.bfloat16, device="cpu") -> str:
    """Writes ``config.json`` (the given dict, which must name its architecture) and
    ``model.safetensors`` with seeded random weights.  Returns the folder.  ``device`` is
    where the values are made (they are the same everywhere; a GPU is quicker for a
    large model)."""
    from ..config import config_from_dict
    from ..parts.model import declared_weights

    spec = config_from_dict(config).to_model_spec()
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    tensors = {k: v.cpu() for k, v in random_tensors(declared_weights(spec), seed, sigma, gain_jitter, dtype, device).items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed, "sigma": sigma, "gain_jitter": gain_jitter})
    return model_dir

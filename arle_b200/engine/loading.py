"""From a model folder (or a configuration and a seed) to a loaded model."""
from __future__ import annotations

import torch

from ..config import config_from_dict, load_config
from ..parts.model import DecoderModel
from ..parts.registry import build_model
from ..weights import load_weights, random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
    elif str(dtype).lower() in _DTYPES:
        return _DTYPES[str(dtype).lower()]
    raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")


def load_model(model_dir: str, dtype="bfloat16", device="cuda") -> DecoderModel:
    """The model class is chosen by ``architectures`` in config.json; weights are
    bound by tensor name from model.safetensors (or its sharded index)."""
    dtype = parse_dtype(dtype)
    config = load_config(model_dir)
    spec = config.to_model_spec()
    model = build_model(spec)
    tensors = load_weights(model_dir, model.weight_decls(), spec.ignored_tensors)
    model.load(tensors, dtype, device)
    model.config = config
    return model


def random_model(config: dict, seed: int, dtype="bfloat16", device="cuda", sigma: float = 0.02,
                 gain_jitter: float = 0.1, num_layers: int = None) -> DecoderModel:
    """A model with seeded random weights made directly on the device (no files).
    ``num_layers`` keeps only the first blocks of the configuration (the
    benchmark's way of fitting time or memory; layer sizes stay)."""
    dtype = parse_dtype(dtype)
    if num_layers is not None:
        config = dict(config, num_hidden_layers=num_layers)
        if "layer_types" in config:
            config["layer_types"] = config["layer_types"][:num_layers]
    cfg = config_from_dict(config)
    spec = cfg.to_model_spec()
    model = build_model(spec)
    tensors = random_tensors(model.weight_decls(), seed, sigma, gain_jitter, torch.bfloat16, device)
    model.load(tensors, dtype, device)
    model.config = cfg
    return model

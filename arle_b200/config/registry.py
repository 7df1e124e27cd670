"""One registry from an architecture's name (``architectures`` in config.json) to
the class that reads its configuration and describes its model.

cklxx/arle maps the same strings to an enum and refuses unknown ones with the
list of names it knows (infer/src/model_registry.rs:139-177, :195-252).  Its map
also sends "Qwen2ForCausalLM" to the Qwen3 model; that model has biases and no
q/k norm, so the alias is not taken over here.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

from .model_spec import ModelSpec

_ARCHITECTURES: Dict[str, type] = {}


class UnknownArchitecture(ValueError):
    pass


def register_architecture(name: str, config_cls: type) -> None:
    """``config_cls`` needs ``from_dir(model_dir)`` / ``from_dict(d)`` returning an
    object with ``to_model_spec() -> ModelSpec``."""
    _ARCHITECTURES[name] = config_cls


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(config_dict: dict) -> type:
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, list):
        raise UnknownArchitecture("config.json has no 'architectures' list; known: " + ", ".join(registered_architectures()))
    for a in archs:
        if a in _ARCHITECTURES:
            return _ARCHITECTURES[a]
    raise UnknownArchitecture(f"architecture(s) {archs} not supported; known: " + ", ".join(registered_architectures()))


def load_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and model.safetensors")
    with open(path) as f:
        d = json.load(f)
    return config_class_for(d).from_dir(model_dir)


def config_from_dict(d: dict):
    return config_class_for(d).from_dict(d)

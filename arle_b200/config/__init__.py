from .model_spec import ModelSpec, ScheduleEntry
from .qwen3 import ConfigError, Qwen3Config
from .registry import (UnknownArchitecture, config_class_for, config_from_dict, load_config,
                       register_architecture, registered_architectures)

register_architecture(Qwen3Config.architecture, Qwen3Config)

__all__ = ["ModelSpec", "ScheduleEntry", "ConfigError", "Qwen3Config", "UnknownArchitecture", "config_class_for",
           "config_from_dict", "load_config", "register_architecture", "registered_architectures"]

"""arle_b200: a small, whole inference engine for one B200, for the Qwen3 dense
architecture, built from what cklxx/arle's ``infer`` crate does for that model.

    from arle_b200 import Engine, SamplingParams
    outs = Engine("/path/to/model").generate([[1, 2, 3]], SamplingParams(max_new_tokens=16))
"""
__version__ = "0.1.0"

_LAZY = {"Engine": ("engine.engine", "Engine"), "EngineOptions": ("engine.engine", "EngineOptions"),
         "GenerationOutput": ("engine.engine", "GenerationOutput"), "SamplingParams": ("sampling", "SamplingParams"),
         "ModelRunner": ("engine.runner", "ModelRunner"), "StepEntry": ("engine.batch", "StepEntry"),
         "load_model": ("engine.loading", "load_model"), "random_model": ("engine.loading", "random_model"),
         "write_random_model": ("weights", "write_random_model")}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    raise AttributeError(name)

from .batch import StepContext, StepEntry, Workspace
from .loading import load_model, parse_dtype, random_model
from .runner import ModelRunner

__all__ = ["StepContext", "StepEntry", "Workspace", "load_model", "parse_dtype", "random_model", "ModelRunner"]

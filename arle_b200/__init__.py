"""arle_b200: a small, whole inference engine for one B200, for the Qwen3 dense
architecture, built from what cklxx/arle's ``infer`` crate does for that model."""
__version__ = "0.1.0"

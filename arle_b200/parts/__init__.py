from .attention import Attention, AttentionSpec
from .base import Block, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, StateNeed, WeightDecl
from .block import PreNormBlock, PreNormBlockSpec
from .mlp import GatedMlp, GatedMlpSpec
from .model import DecoderModel, ResidualStream, declared_weights
from .norm import RmsNorm, RmsNormSpec
from .registry import build_model, build_part, register_model, register_part, registered_models, registered_parts
from .rotary import Rotary, RotarySpec

__all__ = ["Attention", "AttentionSpec", "Block", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part",
           "PositionEncoding", "StateNeed", "WeightDecl", "PreNormBlock", "PreNormBlockSpec", "GatedMlp",
           "GatedMlpSpec", "DecoderModel", "ResidualStream", "declared_weights", "RmsNorm", "RmsNormSpec",
           "build_model", "build_part", "register_model", "register_part", "registered_models", "registered_parts", "Rotary", "RotarySpec"]

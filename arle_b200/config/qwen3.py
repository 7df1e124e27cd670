"""Typed configuration of the Qwen3 dense architecture, read from ``config.json``.

Keys and validation follow cklxx/arle's ``Qwen3Config``
(crates/qwen3-spec/src/lib.rs:95-108 fields, :135-160 validation; the wrapper in
infer/src/model/qwen3/config.rs:61-101 adds ``context_length`` as an alias of
``max_position_embeddings``, bos/eos ids and the stop ids of
``generation_config.json``).  Every size and constant of the model comes from
these keys; none stands in code.

Beyond the reference, which ignores them: keys that would change the arithmetic
(``attention_bias``, ``rope_scaling``, a ``hidden_act`` other than silu) are
refused by name instead of silently dropped, and the sliding-window keys
(``use_sliding_window``, ``sliding_window``, ``max_window_layers``,
``layer_types``) choose a windowed attention mixer for the layers they name.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Optional, Tuple

from .model_spec import ModelSpec, ScheduleEntry


class ConfigError(ValueError):
    pass


_REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
             "rms_norm_eps", "rope_theta", "tie_word_embeddings")


def _positive_int(d: dict, key: str) -> int:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: '{key}' must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    layer_windows: Tuple[Optional[int], ...]   # per layer: key window, None = all keys
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()

    architecture = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: dict, generation_config: Optional[dict] = None) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in d]
        if "num_key_value_heads" not in d and "num_kv_heads" not in d:
            missing.append("num_key_value_heads")
        if "max_position_embeddings" not in d and "context_length" not in d:
            missing.append("max_position_embeddings")
        if missing:
            raise ConfigError("config.json: missing required key(s): " + ", ".join(missing))
        if d.get("attention_bias"):
            raise ConfigError("config.json: 'attention_bias' = true is not supported (Qwen3 projections carry no bias)")
        if d.get("rope_scaling") is not None:
            raise ConfigError("config.json: 'rope_scaling' is not supported; it must be null or absent")
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"config.json: 'hidden_act' = {d['hidden_act']!r} is not supported (silu only)")
        for k in ("rms_norm_eps", "rope_theta"):
            if isinstance(d[k], bool) or not isinstance(d[k], (int, float)) or not d[k] > 0:
                raise ConfigError(f"config.json: '{k}' must be a positive number, got {d[k]!r}")
        if not isinstance(d["tie_word_embeddings"], bool):
            raise ConfigError("config.json: 'tie_word_embeddings' must be true or false")
        n_layers = _positive_int(d, "num_hidden_layers")
        nq = _positive_int(d, "num_attention_heads")
        kv_key = "num_key_value_heads" if "num_key_value_heads" in d else "num_kv_heads"
        nkv = _positive_int(d, kv_key)
        hidden = _positive_int(d, "hidden_size")
        if "head_dim" in d and d["head_dim"] is not None:
            hd = _positive_int(d, "head_dim")
        else:
            if hidden % nq:
                raise ConfigError("config.json: no 'head_dim' and hidden_size is not a multiple of num_attention_heads")
            hd = hidden // nq
        if nq % nkv:
            raise ConfigError(f"config.json: num_attention_heads ({nq}) must be a multiple of {kv_key} ({nkv})")
        if hd % 2:
            raise ConfigError(f"config.json: head_dim ({hd}) must be even for rotary position encoding")
        pos_key = "max_position_embeddings" if "max_position_embeddings" in d else "context_length"
        max_pos = _positive_int(d, pos_key)

        window = d.get("sliding_window")
        types = d.get("layer_types")
        if types is None:
            use = bool(d.get("use_sliding_window", False)) and window is not None
            first = d.get("max_window_layers", n_layers)
            types = ["sliding_attention" if (use and i >= first) else "full_attention" for i in range(n_layers)]
        if len(types) != n_layers:
            raise ConfigError(f"config.json: 'layer_types' has {len(types)} entries for {n_layers} layers")
        wins = []
        for i, t in enumerate(types):
            if t == "full_attention":
                wins.append(None)
            elif t == "sliding_attention":
                if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                    raise ConfigError(f"config.json: layer {i} is 'sliding_attention' but 'sliding_window' is {window!r}")
                wins.append(window)
            else:
                raise ConfigError(f"config.json: layer_types[{i}] = {t!r} (expected full_attention or sliding_attention)")

        eos = d.get("eos_token_id")
        stops: Tuple[int, ...] = ()
        gen_eos = (generation_config or {}).get("eos_token_id")
        if isinstance(gen_eos, int):
            stops = (gen_eos,)
        elif isinstance(gen_eos, list):
            stops = tuple(int(x) for x in gen_eos)
        elif isinstance(eos, int):
            stops = (eos,)
        elif isinstance(eos, list):
            stops = tuple(int(x) for x in eos)
        return cls(hidden_size=hidden, intermediate_size=_positive_int(d, "intermediate_size"),
                   num_hidden_layers=n_layers, num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd,
                   vocab_size=_positive_int(d, "vocab_size"), rms_norm_eps=float(d["rms_norm_eps"]),
                   rope_theta=float(d["rope_theta"]), tie_word_embeddings=d["tie_word_embeddings"],
                   max_position_embeddings=max_pos, layer_windows=tuple(wins),
                   bos_token_id=d.get("bos_token_id") if isinstance(d.get("bos_token_id"), int) else None,
                   eos_token_id=eos if isinstance(eos, int) else None, stop_token_ids=stops)

    @classmethod
    def from_dir(cls, model_dir: str) -> "Qwen3Config":
        with open(os.path.join(model_dir, "config.json")) as f:
            d = json.load(f)
        gen = None
        gpath = os.path.join(model_dir, "generation_config.json")
        if os.path.isfile(gpath):
            with open(gpath) as f:
                gen = json.load(f)
        return cls.from_dict(d, gen)

    # ------------------------------------------------------------------- spec
    def to_model_spec(self) -> ModelSpec:
        """Blocks of a Qwen3 model: pre-norm, attention with per-head q/k norm and
        whole-head rotary encoding, SwiGLU feed-forward
        (infer/src/model/qwen3/prefill.rs:618-776; tensor names
        crates/qwen3-spec/src/lib.rs:185-206)."""
        from ..parts.attention import AttentionSpec
        from ..parts.block import PreNormBlockSpec
        from ..parts.mlp import GatedMlpSpec
        from ..parts.norm import RmsNormSpec
        from ..parts.rotary import RotarySpec

        blocks = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            blocks.append(PreNormBlockSpec(
                mixer_norm=RmsNormSpec(p + "input_layernorm.weight", self.hidden_size, self.rms_norm_eps),
                mixer=AttentionSpec(
                    prefix=p + "self_attn.", hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                    num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                    scale=1.0 / math.sqrt(self.head_dim), qk_norm_eps=self.rms_norm_eps,
                    position=RotarySpec(rotary_dim=self.head_dim, theta=self.rope_theta),
                    window=self.layer_windows[i]),
                ffn_norm=RmsNormSpec(p + "post_attention_layernorm.weight", self.hidden_size, self.rms_norm_eps),
                ffn=GatedMlpSpec(prefix=p + "mlp.", hidden_size=self.hidden_size,
                                 intermediate_size=self.intermediate_size, activation="silu")))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            blocks=tuple(blocks), schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=RmsNormSpec("model.norm.weight", self.hidden_size, self.rms_norm_eps),
            embed_name="model.embed_tokens.weight",
            head_name=None if self.tie_word_embeddings else "lm_head.weight",
            max_position=self.max_position_embeddings, stop_token_ids=self.stop_token_ids,
            bos_token_id=self.bos_token_id,
            ignored_tensors=("lm_head.weight",) if self.tie_word_embeddings else ())

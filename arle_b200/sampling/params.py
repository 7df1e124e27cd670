"""Sampling parameters, with cklxx/arle's names, defaults and meanings
(infer/src/sampler.rs:16-76).  Of these the reference's CUDA sampler applies
temperature, top_k, top_p and ignore_eos (infer/src/ops/sampling.rs:194-224);
this engine applies those and min_p, stop_token_ids, seed and max_new_tokens.
The three penalties are declared for interface parity and refused when set,
rather than silently ignored."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0            # 0 = greedy (argmax, ties to the lowest index)
    top_k: int = -1                     # keep the K most probable; -1 = off
    top_p: float = 1.0                  # nucleus; 1.0 = off
    min_p: float = 0.0                  # drop tokens below min_p * p_max; 0 = off
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    ignore_eos: bool = False            # generate past the model's stop tokens
    stop_token_ids: Tuple[int, ...] = ()
    seed: Optional[int] = None          # None: derived from the engine's seed and the request
    max_new_tokens: Optional[int] = None

    def __post_init__(self):
        if self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0:
            raise ValueError("repetition/frequency/presence penalties are not implemented by this sampler")
        if self.temperature < 0 or not (0 < self.top_p <= 1.0) or not (0 <= self.min_p <= 1.0):
            raise ValueError("temperature must be >= 0, top_p in (0, 1], min_p in [0, 1]")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))

    def is_greedy(self) -> bool:
        """infer/src/sampler.rs:82-84."""
        return (self.temperature <= 0.0 or self.top_k == 1) and self.top_p >= 1.0 and self.min_p <= 0.0

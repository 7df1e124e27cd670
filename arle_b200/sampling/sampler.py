"""Picks next tokens from a step's logits with the sampling kernel.

The uniform number of every non-greedy draw comes from a generator that belongs
to the request (seeded from its ``seed``, or from the engine's seed and the
request's number), one draw per sampled token, so a request's tokens do not
depend on what else is in the batch.  cklxx/arle draws from one engine-wide
generator in batch order (infer/src/model/qwen3/forward.rs:458-508)."""
from __future__ import annotations

import random
from typing import List, Optional, Sequence

import torch

from .. import ops
from .params import SamplingParams


def request_rng(engine_seed: int, request_number: int, params: SamplingParams) -> random.Random:
    if params.seed is not None:
        return random.Random(int(params.seed))
    return random.Random(engine_seed * 1_000_003 + request_number)


class Sampler:
    def __init__(self, vocab_size: int, device):
        self.vocab = vocab_size
        self.device = torch.device(device)
        self._scratch: Optional[torch.Tensor] = None
        self._out: Optional[torch.Tensor] = None
        self._argmax_scratch: Optional[torch.Tensor] = None

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[random.Random]) -> List[int]:
        """logits float32 [R, vocab] on the device; returns R token ids on the host."""
        R = logits.shape[0]
        if self._out is None or self._out.numel() < R:
            self._out = torch.empty(max(R, 64), dtype=torch.int32, device=self.device)
        out = self._out[:R]
        if all(p.is_greedy() for p in params):
            if self._argmax_scratch is None or self._argmax_scratch.numel() < R * 64:
                self._argmax_scratch = torch.empty(max(R, 64) * 64, dtype=torch.float32, device=self.device)
            ops.argmax(logits, self._argmax_scratch, out)
            return out.tolist()
        if self._scratch is None or self._scratch.numel() < R * self.vocab:
            self._scratch = torch.empty(R * self.vocab, dtype=torch.float32, device=self.device)
        host = torch.empty(5, R, dtype=torch.float32)
        for i, (p, g) in enumerate(zip(params, rngs)):
            greedy = p.is_greedy()
            host[0, i] = 0.0 if greedy else p.temperature
            host[1, i] = p.top_p
            host[2, i] = p.min_p
            host[3, i] = 0.0 if greedy else g.random()
            host[4, i] = float(p.top_k)
        dev = host.to(self.device)
        top_k = dev[4].to(torch.int32)
        ops.sample(logits, dev[0], top_k, dev[1], dev[2], dev[3], self._scratch, out)
        return out.tolist()

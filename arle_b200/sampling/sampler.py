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


class SampleHandle:
    """Token ids of one sampling launch on their way to the host; ``result()`` waits for
    the copy and returns them."""

    def __init__(self, host: torch.Tensor, n: int, event):
        self._host, self._n, self._event = host, n, event

    def result(self) -> List[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host[: self._n].tolist()


class Sampler:
    def __init__(self, vocab_size: int, device):
        self.vocab = vocab_size
        self.device = torch.device(device)
        self._scratch: Optional[torch.Tensor] = None
        self._out: Optional[torch.Tensor] = None
        self._argmax_scratch: Optional[torch.Tensor] = None
        self._host = [None, None]           # two pinned buffers in turn: one launch may be in flight while the next is issued
        self._turn = 0

    def _launch(self, logits, params, rngs, want_slots, last_token) -> torch.Tensor:
        R = logits.shape[0]
        if self._out is None or self._out.numel() < R:
            self._out = torch.empty(max(R, 64), dtype=torch.int32, device=self.device)
        out = self._out[:R]
        if all(p.is_greedy() for p in params):
            if self._argmax_scratch is None or self._argmax_scratch.numel() < R * 64:
                self._argmax_scratch = torch.empty(max(R, 64) * 64, dtype=torch.float32, device=self.device)
            ops.argmax(logits, self._argmax_scratch, out, want_slots, last_token if want_slots is not None else None)
            return out
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
        if want_slots is not None:
            ops.scatter_tokens(out, want_slots, last_token)
        return out

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[random.Random],
               want_slots: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None) -> List[int]:
        """logits float32 [R, vocab] on the device; returns R token ids on the host.  With
        ``want_slots`` (int32 [R], the request slot of each row) and ``last_token`` the
        tokens are also left on the device, in last_token[slot], for the next step."""
        return self._launch(logits, params, rngs, want_slots, last_token).tolist()

    def sample_async(self, logits, params, rngs, want_slots=None, last_token=None) -> SampleHandle:
        """Like ``sample``, but returns at once with a handle; the copy to the host runs
        behind the kernels already queued."""
        out = self._launch(logits, params, rngs, want_slots, last_token)
        R = out.numel()
        if self.device.type != "cuda":
            return SampleHandle(out.clone(), R, None)
        self._turn ^= 1
        host = self._host[self._turn]
        if host is None or host.numel() < R:
            host = self._host[self._turn] = torch.empty(max(R, 256), dtype=torch.int32, pin_memory=True)
        host[:R].copy_(out, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return SampleHandle(host, R, ev)

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
    the copy and returns them.  The handle owns its pinned buffers until then, so a
    later launch can never write over tokens that have not been read."""

    def __init__(self, sampler: "Sampler", host: torch.Tensor, n: int, event, params_host=None):
        self._sampler, self._host, self._n, self._event, self._params_host = sampler, host, n, event, params_host
        self._tokens: Optional[List[int]] = None

    def result(self) -> List[int]:
        if self._tokens is None:
            if self._event is not None:
                self._event.synchronize()
            self._tokens = self._host[: self._n].tolist()
            self._sampler._give_back(self._host, self._params_host)
            self._host = self._params_host = None
        return self._tokens


class Sampler:
    def __init__(self, vocab_size: int, device):
        self.vocab = vocab_size
        self.device = torch.device(device)
        self._scratch: Optional[torch.Tensor] = None
        self._out: Optional[torch.Tensor] = None
        self._argmax_scratch: Optional[torch.Tensor] = None
        self._params_dev: Optional[torch.Tensor] = None
        # pinned host buffers not held by a handle: token ids (int32) and per-row parameters (float32 [5, R])
        self._free_token_hosts: List[torch.Tensor] = []
        self._free_param_hosts: List[torch.Tensor] = []

    # ------------------------------------------------------- pinned buffers
    def _pinned(self) -> bool:
        return self.device.type == "cuda"

    def _take(self, pool: List[torch.Tensor], n: int, dtype) -> torch.Tensor:
        for i, b in enumerate(pool):
            if b.numel() >= n:
                return pool.pop(i)
        return torch.empty(max(n, 256), dtype=dtype, pin_memory=self._pinned())

    def _give_back(self, tokens_host, params_host) -> None:
        if tokens_host is not None:
            self._free_token_hosts.append(tokens_host)
        if params_host is not None:
            self._free_param_hosts.append(params_host)

    # --------------------------------------------------------------- launch
    def _launch(self, logits, params, rngs, want_slots, last_token):
        """Returns (device tokens int32 [R], the pinned parameter buffer in use or None)."""
        R = logits.shape[0]
        if self._out is None or self._out.numel() < R:
            self._out = torch.empty(max(R, 64), dtype=torch.int32, device=self.device)
        out = self._out[:R]
        if all(p.is_greedy() for p in params):
            if self._argmax_scratch is None or self._argmax_scratch.numel() < R * 64:
                self._argmax_scratch = torch.empty(max(R, 64) * 64, dtype=torch.float32, device=self.device)
            ops.argmax(logits, self._argmax_scratch, out, want_slots, last_token if want_slots is not None else None)
            return out, None
        if self._scratch is None or self._scratch.numel() < R * self.vocab:
            self._scratch = torch.empty(R * self.vocab, dtype=torch.float32, device=self.device)
        # temperature, top_p, min_p, uniform as float32 rows and top_k as the int32 bits of a fifth row,
        # in pinned memory, so that one copy that does not block the host brings them over
        flat = self._take(self._free_param_hosts, 5 * R, torch.float32)
        host = flat[: 5 * R].view(5, R)
        top_k_bits = host[4].view(torch.int32)
        for i, (p, g) in enumerate(zip(params, rngs)):
            greedy = p.is_greedy()
            host[0, i] = 0.0 if greedy else p.temperature
            host[1, i] = p.top_p
            host[2, i] = p.min_p
            host[3, i] = 0.0 if greedy else g.random()
            top_k_bits[i] = int(p.top_k)
        if self._params_dev is None or self._params_dev.numel() < 5 * R:
            self._params_dev = torch.empty(max(5 * R, 320), dtype=torch.float32, device=self.device)
        dev = self._params_dev[: 5 * R].view(5, R)
        dev.copy_(host, non_blocking=True)
        ops.sample(logits, dev[0], dev[4].view(torch.int32), dev[1], dev[2], dev[3], self._scratch, out)
        if want_slots is not None:
            ops.scatter_tokens(out, want_slots, last_token)
        return out, flat

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[random.Random],
               want_slots: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None) -> List[int]:
        """logits float32 [R, vocab] on the device; returns R token ids on the host.  With
        ``want_slots`` (int32 [R], the request slot of each row) and ``last_token`` the
        tokens are also left on the device, in last_token[slot], for the next step."""
        return self.sample_async(logits, params, rngs, want_slots, last_token).result()

    def sample_async(self, logits, params, rngs, want_slots=None, last_token=None) -> SampleHandle:
        """Like ``sample``, but returns at once with a handle; the copy to the host runs
        behind the kernels already queued.  Any number of handles may be outstanding:
        each has pinned buffers of its own until its tokens have been read."""
        out, params_host = self._launch(logits, params, rngs, want_slots, last_token)
        R = out.numel()
        host = self._take(self._free_token_hosts, R, torch.int32)
        if self.device.type != "cuda":
            host[:R].copy_(out)
            return SampleHandle(self, host, R, None, params_host)
        host[:R].copy_(out, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return SampleHandle(self, host, R, ev, params_host)

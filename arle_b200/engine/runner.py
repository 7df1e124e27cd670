"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step(entries)`` reserves cache room for every entry (all or
nothing), builds the step's tables, runs the model on exactly the tokens given,
from the cache that earlier steps left, and returns float32 logits at the wanted
places, in the order of the entries and of their ``want`` lists.  Prompts may be
cut anywhere, portions of prompts may stand beside single decoded tokens, and a
request may sit out any number of steps.

cklxx/arle has three entry points for this (decode, prefill, mixed:
infer/src/model.rs:502-510, :664-701) with constraints between them
(infer/src/model/qwen3/batch_decode.rs:1038-1088); here there is one.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..cache import CacheManager, OutOfPages
from ..parts.model import DecoderModel
from .batch import StepContext, StepEntry, Workspace


class ModelRunner:
    def __init__(self, model: DecoderModel, page_size: int, num_pages: int, max_slots: int,
                 max_tokens_per_request: Optional[int] = None, device="cuda"):
        self.model = model
        self.device = torch.device(device)
        self.cache = CacheManager(model.cache_needs, model.state_needs, page_size, num_pages, max_slots,
                                  max_tokens_per_request or model.spec.max_position, model.dtype, self.device)
        self.ws = Workspace(self.device)
        self.ctx = StepContext(self.cache, self.ws)
        self.steps_run = 0
        self.tokens_run = 0

    # --------------------------------------------------------------- requests
    def add_request(self, rid) -> None:
        self.cache.add_request(rid)

    def end_request(self, rid) -> None:
        self.cache.free_request(rid)

    # ------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Returns logits float32 [wanted, vocab] (None when nothing is wanted).  The
        tensor is a view of a workspace buffer: copy it before the next step.
        Raises OutOfPages, with nothing changed, when the cache cannot take the
        step's tokens."""
        if not entries:
            return None
        vocab = self.model.spec.vocab_size
        for e in entries:
            if not self.cache.has_request(e.request):
                self.cache.add_request(e.request)
            for t in e.tokens:
                if not 0 <= int(t) < vocab:
                    raise ValueError(f"request {e.request!r}: token id {t} is outside the vocabulary [0, {vocab})")
        starts = [self.cache.num_tokens(e.request) for e in entries]
        self.cache.append([(e.request, len(e.tokens)) for e in entries])
        try:
            ctx = self.ctx.build(entries, starts)
            logits = self.model.forward(ctx)
        except Exception:
            for e, s in zip(entries, starts):
                self.cache.truncate(e.request, s)
            raise
        for e in entries:
            self.cache.release_passed(e.request)
        self.steps_run += 1
        self.tokens_run += ctx.num_tokens
        return logits

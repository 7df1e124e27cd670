"""The Python entry point: ``Engine(model_path).generate(prompts, SamplingParams)``.

It plays the role of cklxx/arle's ``LoadedInferenceEngine`` / ``complete()``
(infer/src/server_engine/loaded.rs:48-99; request_handle_engine.rs:54-96) for
token ids: load a model folder, size the cache, run the scheduler loop until the
given requests are finished, return their tokens and finish reasons ("stop" or
"length", infer/src/server_engine/types.rs:31-43).  Option names follow the
reference's ``infer`` command line (infer/src/main.rs:27-237).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..sampling import Sampler, SamplingParams, request_rng
from .batch import StepEntry
from .loading import load_model, parse_dtype
from .runner import ModelRunner
from .scheduler import Scheduler, SchedulerConfig


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    page_size: int = 16
    num_pages: Optional[int] = None            # None: from free memory and mem_fraction_static
    mem_fraction_static: float = 0.85
    num_slots: int = 64                        # most requests running at a time
    max_seq_len: Optional[int] = None          # most tokens a request may hold; None: max_position_embeddings
    max_num_batched_tokens: int = 16384
    chunked_prefill_size: int = 16384
    max_prefill_tokens: Optional[int] = None
    prefill_max_requests: Optional[int] = None
    scheduler_mixed_policy: str = "mixed"
    max_tokens: int = 256                      # default max_new_tokens of a request
    seed: int = 42
    cuda_graph: bool = True
    kernel_set: str = "fast"                   # "plain": the general kernels only, whatever the shapes


@dataclass
class GenerationOutput:
    request_id: object
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: str
    preemptions: int = 0


class Engine:
    def __init__(self, model_path: Optional[str] = None, *, model=None, options: Optional[EngineOptions] = None, **kw):
        self.options = options or EngineOptions(**kw)
        o = self.options
        dtype = parse_dtype(o.dtype)
        if model is None:
            if model_path is None:
                raise ValueError("Engine needs a model folder (model_path) or a loaded model")
            model = load_model(model_path, dtype, o.device)
        elif model.dtype != dtype:
            raise ValueError(f"the given model was loaded as {model.dtype}, the options ask for {dtype}")
        self.model = model
        max_seq = o.max_seq_len or model.spec.max_position
        per_page = self._bytes_per_page(model, o.page_size, dtype)
        pages = o.num_pages if o.num_pages is not None else self._pages_from_memory(
            per_page, o, max_seq, self._bytes_beside_the_cache(model, o))
        self.runner = ModelRunner(model, o.page_size, pages, o.num_slots, max_seq, o.device, kernel_set=o.kernel_set)
        if o.cuda_graph and torch.device(o.device).type == "cuda":
            self.runner.enable_graphs()
        self.scheduler = Scheduler(self.runner.cache, SchedulerConfig(
            o.max_num_batched_tokens, o.chunked_prefill_size, o.max_prefill_tokens, o.prefill_max_requests,
            o.scheduler_mixed_policy), model.spec.stop_token_ids, o.max_tokens)
        self.sampler = Sampler(model.spec.vocab_size, o.device)
        self._rngs: Dict[object, object] = {}
        self._inflight: list = []           # (plan, sample handle) of the steps launched in the last tick
        self._next_id = 0

    @staticmethod
    def _bytes_per_page(model, page_size: int, dtype) -> int:
        width = 2 if dtype == torch.bfloat16 else 4
        return sum(n.elements_per_token() * page_size * width for n in model.cache_needs)

    @staticmethod
    def _bytes_beside_the_cache(model, o: EngineOptions) -> int:
        """What the engine will hold besides weights and pages: the per-request state arrays of
        mixers that ask for them (one row per slot), the step buffers of the largest step the
        scheduler may plan, and those of the widest captured decode step."""
        state = 0
        for n in model.state_needs:
            elems = 1
            for s_ in n.shape:
                elems *= int(s_)
            state += o.num_slots * elems * torch.empty((), dtype=n.dtype).element_size()
        scratch = getattr(model, "scratch_bytes", None)
        if scratch is None:
            return state
        steps = scratch(o.max_num_batched_tokens, min(o.num_slots, o.max_num_batched_tokens))
        graphs = scratch(min(o.num_slots, 256), min(o.num_slots, 256)) if o.cuda_graph else 0
        return state + steps + graphs

    @staticmethod
    def _pages_from_memory(per_page: int, o: EngineOptions, max_seq: int, beside: int = 0) -> int:
        if per_page == 0:
            return 1
        cap = o.num_slots * -(-max_seq // o.page_size)
        if torch.device(o.device).type != "cuda":
            return min(cap, 4096)
        free, total = torch.cuda.mem_get_info(torch.device(o.device))
        budget = free - int((1.0 - o.mem_fraction_static) * total) - beside
        if budget < per_page * o.num_slots:
            raise RuntimeError(f"not enough free device memory for the cache: {free >> 20} MiB free, "
                               f"mem_fraction_static={o.mem_fraction_static}")
        return max(1, min(cap, budget // per_page))

    # ----------------------------------------------------------------- public
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, request_id=None):
        rid = request_id if request_id is not None else f"req-{self._next_id}"
        self._next_id += 1
        vocab = self.model.spec.vocab_size
        ids = np.asarray(prompt, dtype=np.int64)
        if ids.size and (ids.min() < 0 or ids.max() >= vocab):
            t = int(ids[(ids < 0) | (ids >= vocab)][0])
            raise ValueError(f"token id {t} is outside the vocabulary [0, {vocab})")
        req = self.scheduler.add_request(rid, prompt, params)
        self._rngs[rid] = request_rng(self.options.seed, req.number, req.params)
        return req

    def step(self) -> list:
        """One scheduler tick (one or two model steps).  The tick's steps are launched
        first, with the tokens of the previous tick still on their way (the device hands
        each request's last token to its next step itself); then the previous tick's
        tokens are read and booked.  Returns the requests that finished by them."""
        plans = self.scheduler.schedule()
        if any(e.count > 1 and -1 in e.tokens for p in plans for e in p.entries):
            finished = self._drain()            # a prompt portion must know all its tokens
        else:
            finished = None
        launched = []
        for plan in plans:
            entries = [StepEntry(e.request.rid, e.tokens, (e.count - 1,) if e.samples else ()) for e in plan.entries]
            sampling = [e.request for e in plan.entries if e.samples]
            logits = self.runner.step(entries)
            handle = None
            if sampling:
                handle = self.sampler.sample_async(logits, [r.params for r in sampling],
                                                   [self._rngs[r.rid] for r in sampling],
                                                   self.runner.last_ctx.want_slots, self.runner.last_token)
            self.scheduler.on_launch(plan)
            launched.append((plan, handle))
        if finished is None:
            finished = self._drain()
        self._inflight = launched
        return finished

    def _drain(self) -> list:
        """Reads the tokens of the steps in flight and books them."""
        finished = []
        for plan, handle in self._inflight:
            done = self.scheduler.on_step_done(plan, handle.result() if handle is not None else [])
            for r in done:
                self._rngs.pop(r.rid, None)
            finished.extend(done)
        self._inflight = []
        return finished

    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token: Optional[Callable] = None) -> List[GenerationOutput]:
        """Runs the given prompts (lists of token ids) to completion and returns one
        ``GenerationOutput`` per prompt, in order."""
        if isinstance(sampling_params, SamplingParams) or sampling_params is None:
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        seen = {r.rid: 0 for r in reqs}
        while any(r.finish_reason is None for r in reqs):
            if self.scheduler.has_work():
                self.step()
            elif self._inflight:
                self._drain()
            else:
                raise RuntimeError("scheduler has no work but requests are unfinished")
            if on_token is not None:
                for r in reqs:
                    while seen[r.rid] < len(r.output) and r.output[seen[r.rid]] >= 0:
                        on_token(r.rid, r.output[seen[r.rid]])
                        seen[r.rid] += 1
        self._drain()
        self.scheduler.finished.clear()
        if torch.device(self.options.device).type == "cuda":
            from .. import ops
            ops.check_errors(self.options.device)
        return [GenerationOutput(r.rid, r.prompt, list(r.output), r.finish_reason, r.preemptions) for r in reqs]

    def stats(self) -> dict:
        s = dict(self.scheduler.stats)
        s.update(model_steps=self.runner.steps_run, tokens_run=self.runner.tokens_run,
                 free_pages=self.runner.cache.free_pages(), total_pages=self.runner.cache.total_pages())
        return s

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

import gc
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache import CacheManager, OutOfPages
from ..parts.model import DecoderModel
from .batch import StepContext, StepEntry, Workspace


class ModelRunner:
    def __init__(self, model: DecoderModel, page_size: int, num_pages: int, max_slots: int,
                 max_tokens_per_request: Optional[int] = None, device="cuda", kernel_set: str = "fast"):
        if kernel_set not in ("fast", "plain"):
            raise ValueError(f"kernel_set must be 'fast' or 'plain', got {kernel_set!r}")
        self.model = model
        self.kernel_set = kernel_set
        self.device = torch.device(device)
        self.cache = CacheManager(model.cache_needs, model.state_needs, page_size, num_pages, max_slots,
                                  max_tokens_per_request or model.spec.max_position, model.dtype, self.device)
        self.ws = Workspace(self.device)
        self.ctx = StepContext(self.cache, self.ws)
        # the token each request sampled last, written by the sampling kernels; a step entry
        # whose single token id is negative reads its token from here
        self.last_token = torch.zeros(max_slots, dtype=torch.int32, device=self.device)
        self.ctx.last_token = self.last_token
        self.last_ctx = self.ctx
        self.steps_run = 0
        self.tokens_run = 0
        self.graph_steps = 0
        self._graphs = None            # None: graphs off; else {(rows, table width): _DecodeGraph}
        self._graph_ws = None
        self._max_graph_rows = 0

    # ----------------------------------------------------------------- graphs
    def enable_graphs(self, max_rows: int = 256) -> None:
        """Decode-only steps (every entry one token whose logits are wanted) of up to
        ``max_rows`` rows run as CUDA graphs, one per (row count, block-table width
        rounded up to a power of two), captured at first use.  cklxx/arle captures
        one graph per batch size the same way
        (infer/src/model/qwen3/batch_decode.rs:1695-1730)."""
        if self.device.type != "cuda":
            raise RuntimeError("CUDA graphs need a CUDA device")
        self._graphs = {}
        self._graph_ws = Workspace(self.device)
        self._max_graph_rows = max_rows

    def disable_graphs(self) -> None:
        self._graphs = None

    def _graph_key(self, entries, starts):
        if self._graphs is None or len(entries) > self._max_graph_rows:
            return None
        if any(len(e.tokens) != 1 or tuple(e.want) != (0,) for e in entries):
            return None
        pages = max(-(-(s + 1) // self.cache.page_size) for s in starts)
        # a power of two, but never wider than the host tables are
        width = min(1 << max(3, (pages - 1).bit_length()), self.cache.max_pages_per_request)
        return (len(entries), width)

    def _run_graph(self, key, entries, starts):
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = _DecodeGraph(self, key[1])
        return g.run(entries, starts)

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
            if len(e.tokens) == 1 and int(e.tokens[0]) < 0:
                continue                            # the token this request sampled last, still on the device
            ids = np.asarray(e.tokens, dtype=np.int64)
            if ids.size and (ids.min() < 0 or ids.max() >= vocab):
                t = int(ids[(ids < 0) | (ids >= vocab)][0])
                raise ValueError(f"request {e.request!r}: token id {t} is outside the vocabulary [0, {vocab})")
        starts = [self.cache.num_tokens(e.request) for e in entries]
        self.cache.append([(e.request, len(e.tokens)) for e in entries])
        try:
            key = self._graph_key(entries, starts)
            if key is not None:
                ctx, logits = self._run_graph(key, entries, starts)
                self.graph_steps += 1
            else:
                ctx = self.ctx.build(entries, starts)
                with ops.use_kernel_set(self.kernel_set):
                    logits = _forward(self.model, ctx)
        except Exception:
            for e, s in zip(entries, starts):
                self.cache.truncate(e.request, s)
            raise
        for e in entries:
            self.cache.release_passed(e.request)
        self.steps_run += 1
        self.tokens_run += ctx.num_tokens
        self.last_ctx = ctx
        return logits


def _forward(model, ctx):
    """One pass of the model over a step.  What parts keep in ``ctx.memo`` is derived by the pass that uses it:
    a step that runs twice (eagerly, then under capture) derives it twice, so that the capture holds those launches."""
    ctx.memo.clear()
    return model.forward(ctx)


class _DecodeGraph:
    """A captured decode step for one (row count, block-table width).  It owns its
    step tables, so their addresses never change; the scratch buffers are shared by
    all graphs of a runner (they are as large as the widest captured step needs).
    A replay copies the step's tables into place and launches the graph.  When a
    shared buffer had to grow since the capture, the graph is captured again."""

    def __init__(self, runner: ModelRunner, table_width: int):
        self.runner = runner
        self.table_width = table_width
        self.ws = runner._graph_ws
        self.ctx = StepContext(runner.cache, self.ws)
        self.ctx.last_token = runner.last_token
        self.graph = None
        self.generation = -1
        self.logits = None
        self.launches = 0

    def run(self, entries, starts):
        from .. import ops

        ctx = self.ctx.build(entries, starts, self.table_width)
        if self.graph is None or self.generation != self.ws.generation:
            # This step runs eagerly (which also brings every buffer to its size); the
            # capture that follows records the same launches and executes nothing, so
            # the step has run exactly once and its logits stand.
            model = self.runner.model
            with ops.use_kernel_set(self.runner.kernel_set):
                _forward(model, ctx)
                torch.cuda.synchronize(self.runner.device)
                # No graph may be destroyed while a stream captures (it invalidates the capture):
                # collect what is garbage now, an earlier engine's graphs for one, and keep the
                # collector from running until the capture has ended.
                gc.collect()
                gc_was_on = gc.isenabled()
                gc.disable()
                self.ws.frozen = True
                try:
                    before = ops.launch_count()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        self.logits = _forward(model, ctx)
                    self.launches = ops.launch_count() - before
                finally:
                    self.ws.frozen = False
                    if gc_was_on:
                        gc.enable()
            self.graph = graph
            self.generation = self.ws.generation
            return ctx, self.logits
        self.graph.replay()
        ops.add_launches(self.launches)
        return ctx, self.logits

"""A decoder model put together from a ``ModelSpec``: embedding table, blocks,
the schedule that orders them, final norm and output projection.

``DecoderModel.forward(ctx)`` runs exactly the tokens of one step (``ctx`` is a
``StepContext``) and returns float32 logits at the wanted rows.  It is the only
forward pass of the package: generation, the trace replayer and the benchmark
all go through it.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..config.model_spec import ModelSpec
from .base import WeightDecl
from .registry import build_part, register_model


class ResidualStream:
    """The 32-bit residual of a step and the branch output not yet summed into it.

    ``add(delta)`` only remembers the branch output; the next ``normed(...)`` sums
    it into the residual and normalises in one kernel.  Two ``add`` calls in a row
    (a block with parallel branches) are summed right away.

    For steps of few rows the norm kernel can disappear altogether: ``sink_for(norm, ...)``
    hands out an ``ops.ResidualSink`` that a branch's last product fills (residual sum, the norm's
    gain, sums of squares), and the ``normed(...)`` of that norm then returns ``ops.ScaledRows``, whose
    per-row factor the next product applies.  ``next_entry`` is what runs after the current block
    (its first norm and that norm's reader), set by the model."""

    def __init__(self, resid: torch.Tensor, ws, act_dtype: torch.dtype):
        self.resid = resid
        self.ws = ws
        self.act_dtype = act_dtype
        self.pending: Optional[torch.Tensor] = None
        self.next_entry = None
        self._sink = None
        self._sinks_made = 0

    def add(self, delta: Optional[torch.Tensor]) -> None:
        """``delta`` None: the branch has already put its output into the residual (through a sink)."""
        if delta is None:
            return
        if self.pending is not None:
            ops.residual_add(self.resid, self.pending)
        self.pending = delta

    def sink_for(self, norm, reader, buffer_name: str):
        """A sink for the branch that runs now, if the norm that follows it can be deferred and its
        reader takes rows without their factor; else None."""
        T = self.resid.shape[0]
        if (norm is None or reader is None or self.pending is not None or self.act_dtype != torch.bfloat16
                or not self.resid.is_cuda or ops.kernel_set() != "fast" or not reader.takes_scaled_rows(T)):
            return None
        d = norm.deferred()
        if d is None:
            return None
        gain, eps = d
        xs = self.ws.get(buffer_name, tuple(self.resid.shape), self.act_dtype)
        # two tables in turn: the one being filled is never the one the running product reads
        ss = self.ws.get(f"row_ss_{self._sinks_made & 1}", ops.SS_TABLE_SHAPE, torch.float32)
        self._sinks_made += 1
        self._sink = (norm, ops.ResidualSink(self.resid, gain, eps, xs, ss))
        return self._sink[1]

    def normed(self, norm, buffer_name: str):
        if self._sink is not None:
            for_norm, sink = self._sink
            self._sink = None
            if sink.filled:
                if for_norm is not norm or self.pending is not None:
                    raise RuntimeError("a residual sink was filled for another norm than the one that runs next")
                return ops.ScaledRows(sink.xs, sink.ss, sink.eps)
        out = self.ws.get(buffer_name, tuple(self.resid.shape), self.act_dtype)
        norm.apply(self.resid, self.pending, None, out, write_resid=self.pending is not None)
        self.pending = None
        return out

    def normed_rows(self, norm, rows: torch.Tensor, buffer_name: str) -> torch.Tensor:
        """Norm of the rows listed only (the residual itself is left as it is)."""
        out = self.ws.get(buffer_name, (rows.numel(), self.resid.shape[1]), self.act_dtype)
        norm.apply(self.resid, self.pending, rows, out, write_resid=False)
        return out


def declared_weights(spec: ModelSpec) -> List[WeightDecl]:
    """Every tensor a checkpoint of this model must hold."""
    decls = [WeightDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size))]
    for b in spec.blocks:
        decls.extend(build_part(b).weight_decls())
    decls.extend(build_part(spec.final_norm).weight_decls())
    if spec.head_name is not None:
        decls.append(WeightDecl(spec.head_name, (spec.vocab_size, spec.hidden_size)))
    names = [d.name for d in decls]
    if len(set(names)) != len(names):
        dup = sorted({n for n in names if names.count(n) > 1})
        raise ValueError("tensor names declared twice: " + ", ".join(dup))
    return decls


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks = [build_part(b) for b in spec.blocks]
        self.final_norm = build_part(spec.final_norm)
        self.embed = self.head = None
        self.dtype = None
        # cache layers: one per schedule entry that keeps keys of its own
        self.cache_needs = []
        self.entry_cache_layer: List[Optional[int]] = []
        self.state_needs = []
        self.entry_state: List[Optional[int]] = []
        for i, e in enumerate(spec.schedule):
            mixer = self.blocks[e.block].mixer
            need = mixer.cache_need()
            if e.keys_of is not None:
                src = spec.schedule[e.keys_of]
                src_need = self.blocks[src.block].mixer.cache_need()
                if need is None or src_need is None or need.arrays() != src_need.arrays():
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {e.keys_of}: their per-token arrays differ")
                self.entry_cache_layer.append(self.entry_cache_layer[e.keys_of])
            elif need is not None:
                self.entry_cache_layer.append(len(self.cache_needs))
                self.cache_needs.append(need)
            else:
                self.entry_cache_layer.append(None)
            sneed = mixer.state_need()
            if sneed is not None:
                self.entry_state.append(len(self.state_needs))
                self.state_needs.append(sneed)
            else:
                self.entry_state.append(None)

    # ---------------------------------------------------------------- weights
    def weight_decls(self):
        return declared_weights(self.spec)

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> "DecoderModel":
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"engine dtype must be bfloat16 or float32, got {dtype}")
        device = torch.device(device)
        self.dtype = dtype

        def matrix(t):
            return t.to(device=device, dtype=dtype if dtype == torch.bfloat16 else t.dtype).contiguous()

        self.embed = matrix(tensors[self.spec.embed_name])
        self.head = self.embed if self.spec.head_name is None else matrix(tensors[self.spec.head_name])
        for b in self.blocks:
            b.load(tensors, dtype, device)
        self.final_norm.load(tensors, dtype, device)
        return self

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a step reads: every scheduled block once and the output
        projection (the embedding gather reads a few rows only)."""
        n = self.head.numel() * self.head.element_size() + self.final_norm.weight_bytes()
        for e in self.spec.schedule:
            n += self.blocks[e.block].weight_bytes()
        return n

    # ---------------------------------------------------------------- forward
    # The forward pass in three steps that a model class of another arrangement may replace
    # one by one: the residual the blocks start from, the scheduled blocks, the logits.
    def embed_tokens(self, ctx) -> torch.Tensor:
        """The float32 residual [T, hidden] of this step's tokens."""
        resid = ctx.ws.get("residual", (ctx.num_tokens, self.spec.hidden_size), torch.float32)
        ops.embedding(ctx.token_ids, self.embed, resid, None, getattr(ctx, "last_token", None),
                      getattr(ctx, "slot_of_token", None))
        return resid

    def run_blocks(self, stream: ResidualStream, ctx) -> None:
        order = self.spec.schedule
        for i, e in enumerate(order):
            stream.next_entry = self.blocks[order[i + 1].block].entry() if i + 1 < len(order) else None
            cl = self.entry_cache_layer[i]
            cache = ctx.cache_view(cl, writable=e.keys_of is None) if cl is not None else None
            st = ctx.state_view(self.entry_state[i]) if self.entry_state[i] is not None else None
            self.blocks[e.block].forward(stream, ctx, cache, st)

    def logits_at_wanted(self, stream: ResidualStream, ctx) -> torch.Tensor:
        final = stream.normed_rows(self.final_norm, ctx.want_rows, "final_normed")
        logits = ctx.ws.get("logits", (ctx.num_wanted, self.spec.vocab_size), torch.float32)
        ops.gemm(final, self.head, logits)
        return logits

    def forward(self, ctx) -> Optional[torch.Tensor]:
        stream = ResidualStream(self.embed_tokens(ctx), ctx.ws, self.dtype)
        self.run_blocks(stream, ctx)
        if ctx.num_wanted == 0:
            return None
        return self.logits_at_wanted(stream, ctx)

    def scratch_bytes(self, tokens: int, wanted: int) -> int:
        """Bytes of step buffers a step of this many tokens and wanted rows holds (an upper
        estimate from the widest block), so that the engine can leave room for them."""
        act = 2 if self.dtype == torch.bfloat16 else 4
        widest = max((b.scratch_elements_per_token() for b in self.blocks), default=0)
        H = self.spec.hidden_size
        return tokens * (4 * H + widest * act) + wanted * (self.spec.vocab_size * 4 + H * act)


register_model("decoder", DecoderModel)

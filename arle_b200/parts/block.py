"""Pre-norm block: x <- x + mixer(norm(x)); x <- x + ffn(norm(x))
(infer/src/model/qwen3/prefill.rs:618-776).  The block never touches the residual
itself: it hands branch outputs to the ``ResidualStream``, which folds each into
the 32-bit residual inside the kernel of the next norm, the fusion cklxx/arle's
decode path uses (infer/src/model/qwen3/batch_decode.rs:2422-2452)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

from .base import Block
from .registry import build_part, register_part


@dataclass(frozen=True)
class PreNormBlockSpec:
    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object
    kind: ClassVar[str] = "prenorm_block"


class PreNormBlock(Block):
    def __init__(self, spec: PreNormBlockSpec):
        self.spec = spec
        self.mixer_norm = build_part(spec.mixer_norm)
        self.mixer = build_part(spec.mixer)
        self.ffn_norm = build_part(spec.ffn_norm)
        self.ffn = build_part(spec.ffn)
        self._parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def weight_decls(self):
        return tuple(d for p in self._parts for d in p.weight_decls())

    def load(self, tensors, dtype, device):
        for p in self._parts:
            p.load(tensors, dtype, device)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self._parts)

    def scratch_elements_per_token(self):
        # the two normalised inputs and the larger of the two branches' buffers
        return (self.mixer_norm.scratch_elements_per_token() + self.ffn_norm.scratch_elements_per_token()
                + max(self.mixer.scratch_elements_per_token(), self.ffn.scratch_elements_per_token()))

    def entry(self):
        return self.mixer_norm, self.mixer

    def forward(self, stream, ctx, cache, state):
        T = ctx.num_tokens
        h = stream.normed(self.mixer_norm, "normed_a")
        # where a branch's last product can add into the residual and leave the next norm's input behind,
        # and that norm's reader can apply the norm's factor itself, the norm between them is no kernel
        sink = stream.sink_for(self.ffn_norm, self.ffn, "normed_b") if self.mixer.can_sink(T) else None
        if sink is not None:
            stream.add(self.mixer.forward(h, ctx, cache, state, sink=sink))
        else:
            stream.add(self.mixer.forward(h, ctx, cache, state))
        h = stream.normed(self.ffn_norm, "normed_b")
        nxt = stream.next_entry
        sink = stream.sink_for(nxt[0], nxt[1], "normed_a") if nxt is not None and self.ffn.can_sink(T) else None
        if sink is not None:
            stream.add(self.ffn.forward(h, ctx, sink=sink))
        else:
            stream.add(self.ffn.forward(h, ctx))


register_part(PreNormBlockSpec.kind, PreNormBlock)

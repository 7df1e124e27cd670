"""Gated feed-forward (SwiGLU): down(act(gate(x)) * up(x)), no biases
(infer/src/model/qwen3/prefill.rs:291-337).  Gate and up are packed into one [2I, H]
matrix at load (cklxx/arle offers a packed layout as an option,
infer/src/model/qwen3/weights.rs:98-122); here row 2i is gate_i and row 2i + 1 is up_i, so
that the kernel that forms both sums of a pair can apply the gate itself."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

from .. import ops
from .base import FeedForward, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class GatedMlpSpec:
    prefix: str
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    kind: ClassVar[str] = "gated_mlp"


class GatedMlp(FeedForward):
    def __init__(self, spec: GatedMlpSpec):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} not supported by the gated feed-forward (silu)")
        self.spec = spec
        self.w_gate_up = self.w_down = None

    def weight_decls(self):
        s, p = self.spec, self.spec.prefix
        return (WeightDecl(p + "gate_proj.weight", (s.intermediate_size, s.hidden_size)),
                WeightDecl(p + "up_proj.weight", (s.intermediate_size, s.hidden_size)),
                WeightDecl(p + "down_proj.weight", (s.hidden_size, s.intermediate_size)))

    def load(self, tensors, dtype, device):
        p = self.spec.prefix
        g, u, d = (tensors[p + n + "_proj.weight"] for n in ("gate", "up", "down"))
        wt = dtype if dtype == torch.bfloat16 else (torch.float32 if torch.float32 in (g.dtype, u.dtype) else torch.bfloat16)
        g, u = g.to(device=device, dtype=wt), u.to(device=device, dtype=wt)
        self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1]).contiguous()
        self.w_down = d.to(device=device, dtype=dtype if dtype == torch.bfloat16 else d.dtype).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def scratch_elements_per_token(self):
        return 3 * self.spec.intermediate_size + self.spec.hidden_size

    def takes_scaled_rows(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_gate_up, gated=True)

    def can_sink(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_down)

    def forward(self, x, ctx, sink=None):
        s = self.spec
        T = x.shape[0]
        gu = ctx.ws.get("gate_up", (T, 2 * s.intermediate_size), x.dtype)
        act = ctx.ws.get("ffn_act", (T, s.intermediate_size), x.dtype)
        ops.gemm_silu_mul(x, self.w_gate_up, gu, act)
        out = ctx.ws.get("ffn_out", (T, s.hidden_size), x.dtype)
        if ops.gemm(act, self.w_down, out, sink=sink):
            return None                       # summed into the residual by the product itself
        return out


register_part(GatedMlpSpec.kind, GatedMlp)

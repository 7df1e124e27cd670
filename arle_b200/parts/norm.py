"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * weight, statistics in float32
(crates/cuda-kernels/csrc/misc/norm.cu:221-300).  The gain is held in float32."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

import torch

from .. import ops
from .base import Norm, WeightDecl
from .registry import register_part


@dataclass(frozen=True)
class RmsNormSpec:
    weight_name: str
    size: int
    eps: float
    kind: ClassVar[str] = "rmsnorm"


class RmsNorm(Norm):
    def __init__(self, spec: RmsNormSpec):
        self.spec = spec
        self.eps = spec.eps
        self.weight = None

    def weight_decls(self):
        return (WeightDecl(self.spec.weight_name, (self.spec.size,), init="gain"),)

    def load(self, tensors, dtype, device):
        self.weight = tensors[self.spec.weight_name].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * 4

    def scratch_elements_per_token(self):
        return self.spec.size

    def deferred(self):
        return self.weight, self.eps

    def apply(self, resid, delta, rows, out, write_resid: bool):
        """out = norm(resid (+ delta)) on all rows or on ``rows``; see ops.rmsnorm."""
        ops.rmsnorm(resid, delta, rows, self.weight, self.eps, out, write_resid)
        return out


register_part(RmsNormSpec.kind, RmsNorm)

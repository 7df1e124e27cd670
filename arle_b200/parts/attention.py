"""Grouped-query attention over the paged cache, with optional per-head RMSNorm
of q and k, an optional rotary position encoding and an optional key window.

Order of operations (infer/src/model/qwen3/prefill.rs:652-722): q/k/v projections
without bias -> per-head norm of q and k -> rotation -> k, v into the cache ->
causal attention, query head h reading kv head h // (num_heads / num_kv_heads)
-> output projection.  The three input projections are packed into one matrix at
load, so a step runs one product for them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional

import torch

from .. import ops
from .base import CacheNeed, Mixer, WeightDecl
from .registry import build_part, register_part


@dataclass(frozen=True)
class AttentionSpec:
    prefix: str                     # e.g. "model.layers.3.self_attn."
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    qk_norm_eps: Optional[float]    # None: no per-head norm
    position: Optional[object]      # a position-encoding spec or None
    window: Optional[int] = None    # None: all keys; W: keys p-W+1 .. p
    kind: ClassVar[str] = "attention"


class Attention(Mixer):
    def __init__(self, spec: AttentionSpec):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim % 2 or spec.head_dim > 256:
            raise ValueError(f"head_dim {spec.head_dim} not supported (even, at most 256)")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("window must be positive")
        self.spec = spec
        self.position = build_part(spec.position) if spec.position is not None else None
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # ---------------------------------------------------------------- weights
    def weight_decls(self):
        s, p = self.spec, self.spec.prefix
        dq, dkv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        decls = [WeightDecl(p + "q_proj.weight", (dq, s.hidden_size)),
                 WeightDecl(p + "k_proj.weight", (dkv, s.hidden_size)),
                 WeightDecl(p + "v_proj.weight", (dkv, s.hidden_size)),
                 WeightDecl(p + "o_proj.weight", (s.hidden_size, dq))]
        if s.qk_norm_eps is not None:
            decls += [WeightDecl(p + "q_norm.weight", (s.head_dim,), init="gain"),
                      WeightDecl(p + "k_norm.weight", (s.head_dim,), init="gain")]
        return tuple(decls)

    def load(self, tensors, dtype, device):
        s, p = self.spec, self.spec.prefix
        mats = [tensors[p + n + "_proj.weight"] for n in ("q", "k", "v")]
        wt = dtype if dtype == torch.bfloat16 else (torch.float32 if any(m.dtype == torch.float32 for m in mats) else torch.bfloat16)
        self.w_qkv = torch.cat([m.to(device=device, dtype=wt) for m in mats], dim=0).contiguous()
        o = tensors[p + "o_proj.weight"]
        self.w_o = o.to(device=device, dtype=dtype if dtype == torch.bfloat16 else o.dtype).contiguous()
        if s.qk_norm_eps is not None:
            self.q_norm = tensors[p + "q_norm.weight"].to(device=device, dtype=torch.float32).contiguous()
            self.k_norm = tensors[p + "k_norm.weight"].to(device=device, dtype=torch.float32).contiguous()
        if self.position is not None:
            self.position.load(tensors, dtype, device)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def scratch_elements_per_token(self):
        s = self.spec
        return (2 * s.num_heads + 2 * s.num_kv_heads) * s.head_dim + s.hidden_size

    # ------------------------------------------------------------------ cache
    def cache_need(self):
        return CacheNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def takes_scaled_rows(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_qkv)

    def can_sink(self, num_rows):
        return ops.fused_gemm_shape_ok(num_rows, self.w_o)

    def _angles(self, qkv, ctx, inv_freq, rdim):
        """Cosines and sines of the step's positions, evaluated once for all layers that rotate by the same
        frequencies (kept in the step's memo under the encoding's description)."""
        if not rdim or not ops.attention_prep_takes_angles(qkv, self.spec.head_dim, rdim):
            return None
        key = ("rotary_angles", getattr(self.position, "spec", None) or id(self.position))
        angles = ctx.memo.get(key)
        if angles is None:
            angles = ctx.ws.get(f"rotary_angles_{len(ctx.memo)}", (qkv.shape[0], rdim // 2, 2), torch.float32)
            ops.rotary_angles(ctx.positions, inv_freq, angles)
            ctx.memo[key] = angles
        return angles

    # ---------------------------------------------------------------- forward
    def forward(self, x, ctx, cache, state, sink=None):
        s = self.spec
        T = x.shape[0]
        nq, nkv, hd = s.num_heads, s.num_kv_heads, s.head_dim
        rot = self.position.rotary() if self.position is not None else None
        inv_freq, rdim = rot if rot is not None else (None, 0)
        eps = s.qk_norm_eps if s.qk_norm_eps is not None else 0.0
        attn = ctx.ws.get("attn_out", (T, nq * hd), x.dtype)
        if cache.writable:
            qkv = ctx.ws.get("qkv", (T, (nq + 2 * nkv) * hd), x.dtype)
            ops.gemm(x, self.w_qkv, qkv)
            if ops.fused_decode_supported(qkv, ctx, cache.k.dtype, nq, nkv, hd, cache.page_size, rdim):
                # a step of decoded tokens only: norm, rotation, cache store and attention in one launch
                ops.decode_attention_with_prep(qkv, attn, cache.k, cache.v, cache.slot_mapping, self.q_norm, self.k_norm, eps,
                                               inv_freq if rdim else None, cache.block_table, nq, nkv, hd, cache.page_size,
                                               s.scale, s.window, ctx)
                out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
                return None if ops.gemm(attn, self.w_o, out, sink=sink) else out
            ops.attention_prep(qkv, ctx.positions, cache.slot_mapping, self.q_norm, self.k_norm, eps, inv_freq, rdim,
                               cache.k, cache.v, nq, nkv, hd, cache.page_size, angles=self._angles(qkv, ctx, inv_freq, rdim))
        else:
            qkv = ctx.ws.get("q_only", (T, nq * hd), x.dtype)
            ops.gemm(x, self.w_qkv[: nq * hd], qkv)
            ops.attention_prep(qkv, ctx.positions, None, self.q_norm, None, eps, inv_freq, rdim, None, None, nq, 0, hd,
                               cache.page_size, angles=self._angles(qkv, ctx, inv_freq, rdim))
        ops.paged_attention(qkv[:, : nq * hd], attn, cache.k, cache.v, ctx.positions, ctx.row_of_token,
                            cache.block_table, nq, nkv, hd, cache.page_size, s.scale, s.window, batch=ctx)
        out = ctx.ws.get("mixer_out", (T, s.hidden_size), x.dtype)
        if ops.gemm(attn, self.w_o, out, sink=sink):
            return None                       # summed into the residual by the product itself
        return out


register_part(AttentionSpec.kind, Attention)

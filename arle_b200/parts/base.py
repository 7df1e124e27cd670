"""Interfaces of the parts a model is put together from.

A model is a list of blocks and a schedule that says in which order they run.
A block arranges a *mixer* (the part that lets tokens see each other, attention
here), a *feed-forward*, and *norms*; a mixer may use a *position encoding*.
Every part is described by a frozen dataclass (its *spec*) that carries all of
its sizes and constants, and is built from that spec by the class registered
under the spec's ``kind`` (see ``arle_b200.parts.registry``).  No part knows
which model it is in, and no part reads a model configuration.

What a part must provide:

``weight_decls()``
    the tensors it wants from the checkpoint, by full name, with shape and the
    way a random model initialises them;
``load(tensors, dtype, device)``
    take those tensors (and pack or convert them as its kernels like);
``forward(...)``
    run on the tokens of one step.  Mixers get the step's ``StepContext``, a
    view of their cache layer (or None) and of their per-request state (or
    None); everything else gets tensors.

Mixers additionally say what they need from the cache manager:
``cache_need()`` (paged keys and values: all of them, or a window) and
``state_need()`` (a fixed-size array per request).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class WeightDecl:
    """One checkpoint tensor a part binds by name.

    ``init`` tells the random-weights writer how to fill it: ``"normal"`` (zero
    mean, the writer's sigma), ``"gain"`` (1 + U(-a, a)), ``"zeros"``."""

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    integer: bool = False


@dataclass(frozen=True)
class CacheNeed:
    """Paged per-token arrays a mixer wants for each token it has seen.

    Attention keeps two, keys and values, each ``[num_kv_heads, head_dim]`` per token:
    ``CacheNeed(num_kv_heads, head_dim)``.  A mixer whose per-token record has another
    form names its arrays itself in ``streams``, one ``(heads, width)`` per array: one
    compressed vector per token is ``streams=((1, width),)``; keys and values of
    different widths are two different entries.  The cache manager gives every stream a
    paged array ``[pages, heads, page_size, width]`` per layer, all under one block table.

    ``window`` None keeps every token; an integer keeps only what the last
    ``window`` positions can still see, so older pages go back to the pool."""

    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    streams: Optional[Tuple[Tuple[int, int], ...]] = None

    def arrays(self) -> Tuple[Tuple[int, int], ...]:
        if self.streams is not None:
            return tuple((int(h), int(w)) for h, w in self.streams)
        return ((self.num_kv_heads, self.head_dim), (self.num_kv_heads, self.head_dim))

    def elements_per_token(self) -> int:
        return sum(h * w for h, w in self.arrays())

    def group_key(self):
        return (self.arrays(), self.window)


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size array per live request (recurrent state and the like).  The
    slot is zeroed when a request gets it."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of all parts: weights in, tensors through."""

    def weight_decls(self) -> Sequence[WeightDecl]:
        return ()

    def load(self, tensors: dict, dtype: torch.dtype, device: torch.device) -> None:
        """Bind this part's tensors.  ``tensors`` maps each declared name to a
        tensor in its stored precision; ``dtype`` is the engine's compute type
        (bfloat16 or float32)."""

    def weight_bytes(self) -> int:
        """Bytes of weights one forward pass reads (for roofline accounting)."""
        return 0

    def scratch_elements_per_token(self) -> int:
        """Activation elements per token this part keeps in step buffers (an estimate the
        engine uses to leave memory for them beside the cache)."""
        return 0

    # Optional fusion of the norms into the products around them (decode steps of few rows; see
    # ``ops.ResidualSink`` and ``ops.ScaledRows``).  A part that says yes to ``takes_scaled_rows`` may
    # get ``ops.ScaledRows`` as its input instead of a tensor; a part that says yes to ``can_sink`` may
    # be called with ``sink=`` and, if it gave the sink to its last product, returns None instead of
    # its output.  Parts that know nothing of this are never asked to.
    def takes_scaled_rows(self, num_rows: int) -> bool:
        return False

    def can_sink(self, num_rows: int) -> bool:
        return False


class Norm(Part):
    """y = norm(x) over the last axis.  ``forward(stream, ...)`` is driven by the
    ``ResidualStream`` so that the sum of the pending branch output into the
    32-bit residual and the norm happen in one kernel."""

    eps: float
    weight: torch.Tensor

    def deferred(self):
        """(gain float32 [width], eps) when the norm is x * rsqrt(mean(x^2) + eps) * gain, so that its
        per-row factor can be applied after a product instead of before it; None otherwise."""
        return None


class PositionEncoding(Part):
    """How a mixer learns where a token stands.  The attention mixer understands
    the rotary family: ``rotary()`` returns (inv_freq[rotary_dim/2] float32 on the
    device, rotary_dim) and the angle of pair i at position p is p * inv_freq[i],
    computed in 32-bit inside the kernel; it returns None for "no rotation"."""

    def rotary(self):
        return None


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, ctx, cache, state) -> torch.Tensor:
        """x: [T, hidden] normalised input of this step's tokens.  ``cache`` is a
        ``LayerCacheView`` (or None; ``cache.writable`` is False when this run reads
        another run's cache and must not store), ``state`` the state arena of this mixer
        ([slots, *shape]; rows ``ctx.state_slots`` belong to this step's
        requests) or None.  Returns the branch output [T, hidden]."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of norms, mixer and feed-forward around the residual stream."""

    mixer: Mixer

    def forward(self, stream, ctx, cache, state) -> None:
        raise NotImplementedError

    def entry(self):
        """(the norm this block applies first, the part that reads its output), or None: lets the
        block that runs before this one fold its last residual sum and this norm into its last
        product."""
        return None

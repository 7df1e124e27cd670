"""What a model is, as data: its blocks, the order they run in, and the tensors
around them.  An architecture's configuration class turns its ``config.json``
into one ``ModelSpec``; ``arle_b200.parts.model.DecoderModel`` is built from the
spec alone.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a block.

    ``block`` indexes ``ModelSpec.blocks`` (the same block, hence the same
    weights, may be named by several entries).  ``keys_of`` is None when the run
    keeps a cache of its own, or the index of an earlier schedule entry whose
    cache this run reads instead of writing one."""

    block: int
    keys_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: Tuple[object, ...]               # block specs, see arle_b200.parts
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object                        # norm spec
    embed_name: str
    head_name: Optional[str]                  # None: the output projection is the embedding table
    max_position: int
    stop_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    ignored_tensors: Tuple[str, ...] = ()     # names a checkpoint may carry that the model does not read
    kind: str = "decoder"                     # the registered model class that is built from this spec

    def validate(self) -> None:
        if not self.blocks or not self.schedule:
            raise ValueError("a model needs at least one block and one schedule entry")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.block < len(self.blocks):
                raise ValueError(f"schedule entry {i} names block {e.block}, but there are {len(self.blocks)} blocks")
            if e.keys_of is not None:
                if not 0 <= e.keys_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.keys_of}, which does not run before it")
                if self.schedule[e.keys_of].keys_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.keys_of}, which has none of its own")

"""One step's batch as the kernels see it.

A step is a list of entries ``(request, its next tokens, wanted places)``.  The
entries are laid end to end into T token rows; a decoded token is simply an entry
with one token.  All integer tables of the step are packed into ONE pinned host
array and copied to the device in one transfer, the way cklxx/arle uploads
positions / indptr / page indices per step (crates/cuda-kernels/src/tilelang.rs:424-612,
:703-818), but without separate code paths for decode, prefill and mixed batches.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepEntry:
    request: object                 # request id (any hashable)
    tokens: Sequence[int]           # its next tokens, in order
    want: Sequence[int] = ()        # indices into ``tokens`` whose logits are wanted


class Workspace:
    """Named scratch buffers that live across steps.  ``get`` returns a view of the
    wanted shape on a buffer that only ever grows, so steady-state steps allocate
    nothing."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.frozen = False
        self.generation = 0            # counts (re)allocations: addresses handed out earlier may be stale after one

    def get(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer '{name}' would have to grow inside a captured graph")
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.generation += 1
        return buf[:n].view(shape)

    def get_zeroed(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """Like ``get``, but the buffer is zero when it is first handed out (and after it
        had to grow).  For flags and counters that kernels leave at zero."""
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer '{name}' would have to grow inside a captured graph")
            buf = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
            self.generation += 1
        return buf[:n].view(shape)

    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclass
class GroupTables:
    block_table: torch.Tensor       # int32 [R, width]
    slot_mapping: torch.Tensor      # int32 [T]


class StepContext:
    """Device-side description of one step, handed to every part.

    token_ids, positions, row_of_token, slot_of_token: int32 [T] (a negative token id
    stands for the token its request sampled last, kept on the device in ``last_token``).
    q_indptr: int32 [R+1] (row r owns token rows q_indptr[r] .. q_indptr[r+1]-1).
    kv_lens: int32 [R], tokens the request holds after this step.  state_slots: int32 [R].
    want_rows, want_slots: int32 [W] (token row and request slot of each wanted place).
    Host-side copies of what launch shapes depend on: q_lens, kv_lens_host,
    max_q_len, max_kv_len, decode_only."""

    def __init__(self, cache_manager, ws: Workspace):
        self.cache = cache_manager
        self.ws = ws
        self.device = ws.device
        self.num_tokens = 0
        self.num_rows = 0
        self.num_wanted = 0
        self.requests: List[object] = []
        self.q_lens: List[int] = []
        self.kv_lens_host: List[int] = []
        self.max_q_len = 0
        self.max_kv_len = 0
        self.decode_only = False
        self.num_single = 0
        self.table_width = 0
        self.token_ids = self.positions = self.row_of_token = None
        self.q_indptr = self.kv_lens = self.state_slots = self.want_rows = None
        self.slot_of_token = self.want_slots = None
        self.last_token: Optional[torch.Tensor] = None       # int32 [slots]: each request's last sampled token
        self.h2d_bytes = 0
        self.groups: List[GroupTables] = []
        self.memo: dict = {}                                 # what parts derive from a step once for all layers (cleared per step)
        self._pinned: Optional[torch.Tensor] = None
        self._dev: Optional[torch.Tensor] = None
        self._copied = torch.cuda.Event() if self.device.type == "cuda" else None

    # ------------------------------------------------------------------ build
    def build(self, entries: Sequence[StepEntry], starts: Sequence[int], table_width: Optional[int] = None) -> "StepContext":
        """``starts[i]`` is the number of tokens request i held before this step; the
        cache manager has already made room for the new ones.  ``table_width`` fixes
        the width of every block table (a captured graph needs the same layout at
        every replay); by default each is as wide as the longest request needs."""
        cm = self.cache
        self.memo.clear()
        R = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        W = sum(len(e.want) for e in entries)
        self.num_tokens, self.num_rows, self.num_wanted = T, R, W
        self.requests = [e.request for e in entries]
        self.q_lens = q_lens
        self.kv_lens_host = [s + n for s, n in zip(starts, q_lens)]
        self.max_q_len = max(q_lens)
        self.max_kv_len = max(self.kv_lens_host)
        self.decode_only = self.max_q_len == 1
        self.num_single = sum(1 for n in q_lens if n == 1)
        n_groups = len(cm.groups)
        widths = []
        for gi, g in enumerate(cm.groups):
            need = max(1, max(-(-kv // g.page_size) for kv in self.kv_lens_host))
            if table_width is not None and need > table_width:
                raise ValueError(f"a request needs {need} pages, the fixed table width is {table_width}")
            widths.append(table_width if table_width is not None else need)
        self.table_width = max(widths) if widths else 0
        # layout of the packed int32 array
        sizes = [T, T, T, R + 1, R, R, max(W, 1), T, max(W, 1)]
        for gi in range(n_groups):
            sizes += [R * widths[gi], T]
        offs = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])])
        total = int(offs[-1])
        host = self._host_buffer(total)
        h = host.numpy()
        tok = h[offs[0]:offs[0] + T]
        pos = h[offs[1]:offs[1] + T]
        row = h[offs[2]:offs[2] + T]
        qi = h[offs[3]:offs[3] + R + 1]
        kvl = h[offs[4]:offs[4] + R]
        sts = h[offs[5]:offs[5] + R]
        want = h[offs[6]:offs[6] + W]
        slot_tok = h[offs[7]:offs[7] + T]
        want_slot = h[offs[8]:offs[8] + W]
        slots = np.fromiter((cm.slot(e.request) for e in entries), dtype=np.int64, count=R)
        starts_np = np.asarray(starts, dtype=np.int64)
        sts[:] = slots
        if self.max_q_len == 1 and W == R and all(tuple(e.want) == (0,) for e in entries):
            # every entry is one decoded token whose logits are wanted: no loops over requests
            tok[:] = [e.tokens[0] for e in entries]
            pos[:] = starts_np
            row[:] = np.arange(R)
            qi[:] = np.arange(R + 1)
            kvl[:] = starts_np + 1
            want[:] = np.arange(R)
            slot_tok[:] = slots
            want_slot[:] = slots
            for gi, g in enumerate(cm.groups):
                bt = h[offs[9 + 2 * gi]:offs[9 + 2 * gi] + R * widths[gi]].reshape(R, widths[gi])
                bt[:] = g.table[slots, :widths[gi]]
                pages = g.table[slots, starts_np // g.page_size].astype(np.int64)
                if (pages < 0).any():
                    raise RuntimeError(f"a token of this step has no page in cache group {gi}")
                h[offs[10 + 2 * gi]:offs[10 + 2 * gi] + T] = pages * g.page_size + starts_np % g.page_size
        else:
            at = 0
            wi = 0
            qi[0] = 0
            for r, (e, st, n) in enumerate(zip(entries, starts, q_lens)):
                tok[at:at + n] = np.asarray(e.tokens, dtype=np.int32)
                pos[at:at + n] = np.arange(st, st + n, dtype=np.int32)
                row[at:at + n] = r
                slot_tok[at:at + n] = slots[r]
                for w in e.want:
                    if not 0 <= w < n:
                        raise ValueError(f"request {e.request!r}: wanted place {w} is not among its {n} tokens")
                    want[wi] = at + w
                    want_slot[wi] = slots[r]
                    wi += 1
                at += n
                qi[r + 1] = at
                kvl[r] = st + n
            for gi in range(n_groups):
                bt = h[offs[9 + 2 * gi]:offs[9 + 2 * gi] + R * widths[gi]].reshape(R, widths[gi])
                bt[:] = cm.block_rows(gi, self.requests, widths[gi])
                sm = h[offs[10 + 2 * gi]:offs[10 + 2 * gi] + T]
                at = 0
                for e, st, n in zip(entries, starts, q_lens):
                    sm[at:at + n] = cm.slot_mapping(gi, e.request, st, n)
                    at += n
        dev = self._device_buffer(total)
        dev[:total].copy_(host[:total], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
        self.h2d_bytes = total * 4
        d = dev
        self.token_ids = d[offs[0]:offs[0] + T]
        self.positions = d[offs[1]:offs[1] + T]
        self.row_of_token = d[offs[2]:offs[2] + T]
        self.q_indptr = d[offs[3]:offs[3] + R + 1]
        self.kv_lens = d[offs[4]:offs[4] + R]
        self.state_slots = d[offs[5]:offs[5] + R]
        self.want_rows = d[offs[6]:offs[6] + W]
        self.slot_of_token = d[offs[7]:offs[7] + T]
        self.want_slots = d[offs[8]:offs[8] + W]
        self.groups = []
        for gi in range(n_groups):
            bt = d[offs[9 + 2 * gi]:offs[9 + 2 * gi] + R * widths[gi]].view(R, widths[gi])
            sm = d[offs[10 + 2 * gi]:offs[10 + 2 * gi] + T]
            self.groups.append(GroupTables(bt, sm))
        return self

    def _host_buffer(self, n: int) -> torch.Tensor:
        if self._copied is not None:
            self._copied.synchronize()      # the last step's copy has read the pinned array
        if self._pinned is None or self._pinned.numel() < n:
            cap = max(n, 4096)
            self._pinned = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        return self._pinned

    def _device_buffer(self, n: int) -> torch.Tensor:
        if self._dev is None or self._dev.numel() < n:
            self._dev = torch.empty(max(n, 4096), dtype=torch.int32, device=self.device)
        return self._dev

    # ------------------------------------------------------------------ views
    def cache_view(self, cache_layer: int, writable: bool = True):
        gi = self.cache.group_of_layer(cache_layer)
        t = self.groups[gi]
        return self.cache.layer_view(cache_layer, t.block_table, t.slot_mapping, writable)

    def state_view(self, state_index: int) -> torch.Tensor:
        return self.cache.states[state_index]

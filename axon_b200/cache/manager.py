"""The cache on the device, managed by the host library's ``CacheManager``.

Every run of a layer (schedule entry) that keeps keys and values belongs to a
*group*: the entries whose mixers need the same geometry (kv heads, head size) and
the same retention (all positions, or a window).  A group owns one pool
``[pages + 1, entries, 2, kv_heads, page_size, head_dim]`` (the extra page is the sink
that unheld table entries point at) and one block table ``[slots, pages per request]``.
One page id covers all entries of its group.  Entries with fixed-size state get a slab
``[slots, *shape]`` indexed by the request's slot, zeroed when a slot is opened.

Pages are taken before a step writes positions (``reserve``), given back when a
request ends (``close``) or a window has passed them (``commit``), and used again after
the next ``flush`` (two-phase free, src/cuda/qwen2/pages.rs:141-153,308-311).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..kernels import lib
from ..kernels.ops import KvView
from ..parts.spec import KvNeed, StateNeed

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class _Group:
    need: KvNeed
    entries: List[int]           # schedule entries that own a plane of this group's pool
    pool: Optional[torch.Tensor] = None
    table: Optional[torch.Tensor] = None    # device [slots, stride] int32
    staging: Optional[torch.Tensor] = None  # pinned host copy
    uploaded_version: int = 0


class PagedCache:
    """Pools, block tables and state slabs of one model on one device."""

    def __init__(self, needs: Sequence[Union[KvNeed, StateNeed, None]], dtype: torch.dtype,
                 device: Union[str, torch.device], *, page_size: int = 16, max_tokens: int = 4096,
                 max_slots: int = 16, max_positions: int = 4096, shuffle_seed: int = 0,
                 allocate: bool = True):
        """``needs[i]`` is what schedule entry ``i`` keeps (None for an entry that keeps
        nothing or reads another entry's cache).  ``max_tokens`` sizes every pool: it
        holds that many positions over all live requests, counted in whole pages."""
        host = lib.host()
        self.dtype, self.device = dtype, torch.device(device)
        self.page_size, self.max_slots, self.max_positions = page_size, max_slots, max_positions
        self.groups: List[_Group] = []
        self._entry_group: Dict[int, Tuple[int, int]] = {}
        self.states: Dict[int, torch.Tensor] = {}
        by_key: Dict[Tuple[int, int, Optional[int]], int] = {}
        for i, need in enumerate(needs):
            if isinstance(need, KvNeed):
                key = (need.kv_heads, need.head_dim, need.window)
                if key not in by_key:
                    by_key[key] = len(self.groups)
                    self.groups.append(_Group(need, []))
                g = by_key[key]
                self._entry_group[i] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(i)
            elif isinstance(need, StateNeed):
                if allocate:
                    self.states[i] = torch.zeros((max_slots, *need.shape), dtype=_STATE_DTYPES[need.dtype],
                                                 device=self.device)
            elif need is not None:
                raise TypeError(f"schedule entry {i}: unknown cache need {need!r}")
        n_pages = (max_tokens + page_size - 1) // page_size
        self.n_pages = n_pages
        cfgs = [host.GroupConfig(page_size, n_pages, g.need.window or 0) for g in self.groups]
        if not cfgs:
            # a model without keys and values still gets slots (for its state)
            cfgs = [host.GroupConfig(page_size, n_pages, 0)]
        self.manager = host.CacheManager(cfgs, max_slots, max_positions, shuffle_seed)
        if allocate:
            for gi, g in enumerate(self.groups):
                n = g.need
                g.pool = torch.zeros((n_pages + 1, len(g.entries), 2, n.kv_heads, page_size, n.head_dim),
                                     dtype=dtype, device=self.device)
                stride = self.manager.table_stride(gi)
                g.table = torch.full((max_slots, stride), n_pages, dtype=torch.int32, device=self.device)
                g.staging = torch.empty((max_slots, stride), dtype=torch.int32).pin_memory()
        self._views: Dict[int, KvView] = {}

    # -- slots ------------------------------------------------------------
    def open(self) -> int:
        """A slot for a new request (its state zeroed), or -1 when all are taken."""
        slot = self.manager.open_slot()
        if slot >= 0:
            for s in self.states.values():
                s[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        self.manager.close_slot(slot)

    def reserve(self, slot: int, new_len: int) -> bool:
        return self.manager.reserve(slot, new_len)

    def commit(self, slot: int, new_len: int) -> None:
        self.manager.commit(slot, new_len)

    def flush(self) -> None:
        self.manager.flush()

    def length(self, slot: int) -> int:
        return self.manager.length(slot)

    # -- device side ------------------------------------------------------
    def sync_tables(self) -> None:
        """Copy block tables that changed since the last step to the device."""
        for gi, g in enumerate(self.groups):
            v = self.manager.version(gi)
            if v != g.uploaded_version and g.table is not None:
                g.staging.numpy()[...] = self.manager.table(gi)
                g.table.copy_(g.staging, non_blocking=True)
                g.uploaded_version = v

    def view(self, entry: int) -> Any:
        """What schedule entry ``entry`` keeps: a :class:`KvView`, a state slab, or None."""
        if entry in self.states:
            return self.states[entry]
        if entry not in self._entry_group:
            return None
        v = self._views.get(entry)
        if v is None:
            gi, plane = self._entry_group[entry]
            g = self.groups[gi]
            v = KvView(g.pool, g.table, plane, self.page_size, g.need.kv_heads, g.need.head_dim,
                       g.need.window or 0)
            self._views[entry] = v
        return v

    def bytes_per_token(self) -> int:
        """Cache bytes one position takes over all groups."""
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.entries) * 2 * g.need.kv_heads * g.need.head_dim * item for g in self.groups)

"""The cache on the device, managed by the host library's ``CacheManager``.

Every part of a schedule entry (a run of a layer) that keeps keys and values belongs to a
*group*: the parts whose needs agree in geometry (kv heads, row widths, planes) and in
retention (all positions, or a window).  A group owns one pool of ``pages + 1`` pages (the
extra page is the sink that unheld table entries point at), each page holding every
member's planes for ``page_size`` positions, and one block table ``[slots, pages per
request]``.  One page id covers all members of its group.  Parts with fixed-size state get
a slab ``[slots, *shape]`` indexed by the request's slot, zeroed when a slot is opened.

Pages are taken before a step writes positions (``reserve``), given back when a
request ends (``close``) or a window has passed them (``commit``), and used again after
the next ``flush`` (two-phase free, src/cuda/qwen2/pages.rs:141-153,308-311).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..kernels import lib
from ..kernels.ops import KvView
from ..parts.spec import KvNeed, StateNeed

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}
#: pinned copies of a block table that take turns, so that a step queued behind others never
#: has its table overwritten on the host before its copy has run
_TABLE_STAGES = 4
#: what is left free beside the pool when it is sized from the device's free memory
POOL_RESERVE_BYTES = 256 << 20

Need = Union[KvNeed, StateNeed, None]


def plan_pool_tokens(free_bytes: int, bytes_per_token: int, page_size: int, parallel: int, max_ctx: int,
                     workspace_bytes: int = 0, reserve_bytes: int = POOL_RESERVE_BYTES) -> int:
    """Positions a cache pool gets when nobody says: what fits into the device's free memory
    beside the step's workspace and a reserve, in whole pages, and no more than every request
    slot at full context needs (the reference's rule, src/serve.rs:2411-2449)."""
    most = parallel * (-(-max_ctx // page_size)) * page_size
    if bytes_per_token <= 0:
        return most
    room = free_bytes - workspace_bytes - reserve_bytes
    pages = max(room, 0) // (bytes_per_token * page_size)
    # the sink page comes on top of the pages that are handed out
    tokens = max(pages - 1, 0) * page_size
    return int(min(tokens, most))


@dataclass
class _Group:
    need: KvNeed
    members: List[Tuple[int, str]]           # (schedule entry, part) that own planes of this group's pool
    pool: Optional[torch.Tensor] = None
    table: Optional[torch.Tensor] = None     # device [slots, stride] int32
    staging: List[torch.Tensor] = field(default_factory=list)    # pinned host copies, taking turns
    events: List[Optional[torch.cuda.Event]] = field(default_factory=list)
    turn: int = 0
    uploaded_version: int = 0


class PagedCache:
    """Pools, block tables and state slabs of one model on one device."""

    def __init__(self, needs: Sequence[Union[Need, Mapping[str, Need]]], dtype: torch.dtype,
                 device: Union[str, torch.device], *, page_size: int = 16, max_tokens: int = 4096,
                 max_slots: int = 16, max_positions: int = 4096, shuffle_seed: int = 0,
                 allocate: bool = True, check_tables: bool = False):
        """``needs[i]`` is what schedule entry ``i`` keeps: a mapping from the name of each of
        its cache-keeping parts to that part's need (a bare need stands for one part named
        ``"mixer"``; None or an empty mapping for an entry that keeps nothing or reads another
        entry's cache).  ``max_tokens`` sizes every pool: it holds that many positions over all
        live requests, counted in whole pages.  ``check_tables`` makes the kernels compare every
        block-table entry they read with the pool's size (see ``fault()``)."""
        host = lib.host()
        self.dtype, self.device = dtype, torch.device(device)
        self.page_size, self.max_slots, self.max_positions = page_size, max_slots, max_positions
        self.groups: List[_Group] = []
        self._member_group: Dict[Tuple[int, str], Tuple[int, int]] = {}
        self._entry_parts: Dict[int, List[str]] = {}
        self.states: Dict[Tuple[int, str], torch.Tensor] = {}
        by_key: Dict[Tuple, int] = {}
        for i, entry_needs in enumerate(needs):
            if entry_needs is None:
                entry_needs = {}
            elif not isinstance(entry_needs, Mapping):
                entry_needs = {"mixer": entry_needs}
            for name, need in entry_needs.items():
                if need is None:
                    continue
                self._entry_parts.setdefault(i, []).append(name)
                if isinstance(need, KvNeed):
                    key = (need.kv_heads, need.head_dim, need.window, need.value_dim, need.planes)
                    if key not in by_key:
                        by_key[key] = len(self.groups)
                        self.groups.append(_Group(need, []))
                    g = by_key[key]
                    self._member_group[(i, name)] = (g, len(self.groups[g].members))
                    self.groups[g].members.append((i, name))
                elif isinstance(need, StateNeed):
                    if allocate:
                        self.states[(i, name)] = torch.zeros((max_slots, *need.shape), dtype=_STATE_DTYPES[need.dtype],
                                                             device=self.device)
                else:
                    raise TypeError(f"schedule entry {i}, part '{name}': unknown cache need {need!r}")
        n_pages = (max_tokens + page_size - 1) // page_size
        self.n_pages = n_pages
        cfgs = [host.GroupConfig(page_size, n_pages, g.need.window or 0) for g in self.groups]
        if not cfgs:
            # a model without keys and values still gets slots (for its state)
            cfgs = [host.GroupConfig(page_size, n_pages, 0)]
        self.manager = host.CacheManager(cfgs, max_slots, max_positions, shuffle_seed)
        #: checked tables: two uint32 on the device, (set, the offending entry)
        self._fault = torch.zeros(2, dtype=torch.int32, device=self.device) if (check_tables and allocate) else None
        if allocate:
            for gi, g in enumerate(self.groups):
                n = g.need
                if n.planes == 2 and n.value_dim == n.head_dim:
                    shape = (n_pages + 1, len(g.members), 2, n.kv_heads, page_size, n.head_dim)
                else:
                    shape = (n_pages + 1, len(g.members), page_size * n.elements_per_token)
                g.pool = torch.zeros(shape, dtype=dtype, device=self.device)
                stride = self.manager.table_stride(gi)
                g.table = torch.full((max_slots, stride), n_pages, dtype=torch.int32, device=self.device)
                g.staging = [torch.empty((max_slots, stride), dtype=torch.int32).pin_memory() for _ in range(_TABLE_STAGES)]
                g.events = [None] * _TABLE_STAGES
        self._views: Dict[Tuple[int, str], KvView] = {}

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
        """Copy block tables that changed since the last step to the device.  The copy is queued
        on the stream behind the steps before it; its pinned source is one of several that take
        turns, and a source is written again only after the copy that read it has run, so a
        caller may queue steps without waiting for any of them."""
        for gi, g in enumerate(self.groups):
            v = self.manager.version(gi)
            if v != g.uploaded_version and g.table is not None:
                i = g.turn
                g.turn = (i + 1) % len(g.staging)
                if g.events[i] is not None:
                    g.events[i].synchronize()
                g.staging[i].numpy()[...] = self.manager.table(gi)
                g.table.copy_(g.staging[i], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                g.events[i] = ev
                g.uploaded_version = v

    def parts(self, entry: int) -> List[str]:
        """Names of the parts of schedule entry ``entry`` that keep something here."""
        return list(self._entry_parts.get(entry, ()))

    def view(self, entry: int, part: Optional[str] = None) -> Any:
        """What schedule entry ``entry`` keeps.  With ``part``: that part's :class:`KvView` or state
        slab.  Without: the same for an entry with one cache-keeping part, a dict by part name
        for an entry with several, None for an entry with none."""
        if part is None:
            names = self._entry_parts.get(entry, ())
            if not names:
                return None
            if len(names) == 1:
                return self.view(entry, names[0])
            return {n: self.view(entry, n) for n in names}
        key = (entry, part)
        if key in self.states:
            return self.states[key]
        if key not in self._member_group:
            return None
        v = self._views.get(key)
        if v is None:
            gi, plane = self._member_group[key]
            g = self.groups[gi]
            v = KvView(g.pool, g.table, plane, self.page_size, g.need.kv_heads, g.need.head_dim,
                       g.need.window or 0, v_dim=g.need.value_dim, planes=g.need.planes, fault=self._fault)
            self._views[key] = v
        return v

    @property
    def checks_tables(self) -> bool:
        return self._fault is not None

    def fault(self) -> Optional[int]:
        """With checked tables: None while every block-table entry the kernels read lay inside
        its pool, else the first offending entry seen (synchronises; clears the record)."""
        if self._fault is None:
            return None
        set_, entry = self._fault.tolist()
        if not set_:
            return None
        self._fault.zero_()
        return entry

    def bytes_per_token(self) -> int:
        """Cache bytes one position takes over all groups."""
        return bytes_per_token([g.need for g in self.groups for _ in g.members], self.dtype)


def bytes_per_token(needs: Sequence[Union[Need, Mapping[str, Need]]], dtype: torch.dtype) -> int:
    """Cache bytes one position takes for these needs (state slabs do not grow with positions)."""
    item = torch.empty((), dtype=dtype).element_size()
    total = 0
    for n in needs:
        for need in (n.values() if isinstance(n, Mapping) else (n,)):
            if isinstance(need, KvNeed):
                total += need.elements_per_token * item
    return total

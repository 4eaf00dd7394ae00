"""The cache manager: paged keys and values in groups, and fixed-size state slots.

Layers whose mixers need the same thing (``CacheNeed``: kv heads, head size, all keys or a
window of them) form a *group*.  A group owns a pool of pages, one device tensor
``[layers, pages + 1, 2, kv_heads, page_size, head_dim]`` (keys at index 0 of the third axis,
values at 1; page 0 is never handed out) and one block table per live request.  A page of one
head is a contiguous ``[page_size, head_dim]`` tile.

A request takes a slot when it is opened, grows page by page as its tokens arrive (all
groups together, or not at all: ``OutOfPages``), gives pages of windowed groups back as the
window passes them, and gives everything back when it is closed.  Beside the pages, each
mixer that declares a ``StateNeed`` gets a tensor ``[slots + 1, *shape]`` indexed by the
request's slot, zeroed when the request is opened (slot 0 stays zero).

Stands where lily/mem_cache/memory_pool.py:21-55 (request rows), :78-143 (per-layer K and V),
:146-165 (layers with different needs), :168-233 (per-request state) and
lily/mem_cache/allocator.py:34-57 (free list) stand in the reference; sizing follows
lily/model_executor/model_runner.py:160-196.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from lily_b200.cache.pages import GroupTables, OutOfPages, OutOfSlots, SlotPool, pages_for
from lily_b200.parts.base import CacheNeed, StateNeed


@dataclass
class CacheGroup:
    need: CacheNeed
    num_layers: int
    tables: GroupTables
    data: Optional[torch.Tensor]            # None when built without a device (host-only tests)

    def layer(self, index: int) -> torch.Tensor:
        return self.data[index]


def bytes_per_token(groups: Sequence[Tuple[CacheNeed, int]], dtype: torch.dtype) -> int:
    """Bytes of keys and values one token takes over all layers (model_runner.py:160-164)."""
    item = torch.empty((), dtype=dtype).element_size()
    return sum(2 * need.kv_heads * need.head_dim * layers * item for need, layers in groups)


class KVCacheManager:
    def __init__(self, groups: Sequence[Tuple[CacheNeed, int]], states: Sequence[StateNeed], *,
                 page_size: int, num_pages: int, max_requests: int, max_context: int,
                 dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None):
        if page_size < 1 or page_size & (page_size - 1):
            raise ValueError("page_size must be a power of two")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.max_context = max_context
        self.max_pages_per_request = pages_for(max_context, page_size)
        self.dtype = dtype
        self.device = device
        self.slots = SlotPool(max_requests)
        self.groups: List[CacheGroup] = []
        for need, layers in groups:
            data = None
            if device is not None:
                data = torch.zeros((layers, num_pages + 1, 2, need.kv_heads, page_size, need.head_dim),
                                   dtype=dtype, device=device)
            self.groups.append(CacheGroup(need, layers, GroupTables(num_pages, page_size, need.window), data))
        self.states: List[Optional[torch.Tensor]] = []
        self.state_needs = list(states)
        for need in states:
            self.states.append(None if device is None else
                               torch.zeros((max_requests + 1, *need.shape), dtype=need.dtype, device=device))
        self.lengths: Dict[int, int] = {}            # slot -> positions whose pages are held

    # ---- requests ------------------------------------------------------------

    def open_request(self) -> int:
        slot = self.slots.alloc()
        for g in self.groups:
            g.tables.open(slot)
        for s in self.states:
            if s is not None:
                s[slot].zero_()
        self.lengths[slot] = 0
        return slot

    def pages_needed(self, slot: int, new_len: int) -> int:
        """The largest number of pages any group must take for ``slot`` to hold ``new_len`` positions."""
        return max((g.tables.pages_needed(slot, new_len) for g in self.groups), default=0)

    def can_grow(self, wants: Sequence[Tuple[int, int]]) -> bool:
        """Whether all (slot, new_len) of a step fit at once."""
        for g in self.groups:
            if sum(g.tables.pages_needed(s, n) for s, n in wants) > g.tables.pool.available:
                return False
        return True

    def grow(self, slot: int, new_len: int) -> None:
        if new_len > self.max_context:
            raise ValueError(f"request would hold {new_len} positions, context length is {self.max_context}")
        for g in self.groups:
            if g.tables.pages_needed(slot, new_len) > g.tables.pool.available:
                raise OutOfPages(f"slot {slot}: {g.tables.pages_needed(slot, new_len)} pages needed, "
                                 f"{g.tables.pool.available} free")
        for g in self.groups:
            g.tables.grow(slot, new_len)
        self.lengths[slot] = max(self.lengths[slot], new_len)

    def advance(self, slot: int, seq_len: int) -> int:
        """Called after a step has cached ``seq_len`` positions: windowed groups let go of what
        no later query can see.  Returns the number of pages given back."""
        return sum(g.tables.pass_window(slot, seq_len) for g in self.groups)

    def close_request(self, slot: int) -> None:
        for g in self.groups:
            g.tables.close(slot)
        del self.lengths[slot]
        self.slots.free(slot)

    # ---- views ---------------------------------------------------------------

    def block_table(self, group: int, slot: int) -> List[int]:
        return self.groups[group].tables.tables[slot].pages

    def table_stamp(self, group: int, slot: int) -> int:
        """A number that changes whenever the request's block table in this group does (and that no other table has)."""
        return self.groups[group].tables.tables[slot].stamp

    def free_pages(self) -> int:
        return min((g.tables.pool.available for g in self.groups), default=self.num_pages)

    def free_tokens(self) -> int:
        return self.free_pages() * self.page_size

    def held_pages(self) -> List[int]:
        return [g.tables.pool.held() for g in self.groups]

    def live_requests(self) -> int:
        return len(self.lengths)


def pool_pages_from_memory(groups: Sequence[Tuple[CacheNeed, int]], dtype: torch.dtype, page_size: int,
                           free_bytes: int, total_bytes: int, mem_fraction_static: float) -> int:
    """Pages that fit in what is left of ``mem_fraction_static`` of the device after the weights
    (lily/model_executor/model_runner.py:173-181)."""
    rest = free_bytes - total_bytes * (1.0 - mem_fraction_static)
    cell = bytes_per_token(groups, dtype)
    if cell == 0:
        return 1
    return max(0, int(rest // (cell * page_size)))


__all__ = ["CacheGroup", "KVCacheManager", "OutOfPages", "OutOfSlots", "bytes_per_token", "pool_pages_from_memory"]

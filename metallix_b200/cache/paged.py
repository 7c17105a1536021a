"""The cache a model's layers share: pages of keys and values per group of
layers, block tables per request, and slots of fixed-size per-request state.

Accounting (which request holds which page, which pages are free) is the C++
``CacheManager``; this file owns the device memory and turns the manager's
tables into what the kernels read.

Device layout of a group of layers with the same needs:
``[entries, pages, 2 (K, V), kv_heads, page_tokens, head_dim]`` in the compute
dtype: one entry per layer of the group, so a page index means the same
positions in every layer of the group and one block table serves them all. The
reference keeps K and V per layer as ``[slots, kv_heads, head_dim]``
(crates/models/qwen/src/forward/paged.rs:135-146); here a head's rows of one
page are contiguous so that a kernel reads a page of one head as one block.
State entries are ``[request_slots, *state_shape]``, zeroed when a request is
admitted.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..config.spec import CacheNeed
from ..csrc import build
from ..parts.registry import CacheView


@dataclass
class Group:
    index: int
    need: CacheNeed
    entries: List[int]            # cache entries (layer indices) of this group
    page_tokens: int
    num_pages: int
    pool: Optional[torch.Tensor]  # [entries, pages, 2, kv_heads, page_tokens, head_dim]

    def bytes_per_page(self) -> int:
        if self.pool is None:
            return 0
        return self.pool[0, 0].numel() * self.pool.element_size() * len(self.entries)


class PagedCache:
    """Pools, state slots and the manager for one model."""

    @staticmethod
    def page_bytes(needs: Sequence[Optional[CacheNeed]], page_tokens: int, dtype: torch.dtype) -> int:
        """Bytes that one page index takes over all groups and all their
        entries: what a pool of n pages per group costs is n times this. The
        reference sizes its pool from a byte budget the same way
        (crates/core/engine/src/blocks.rs:162-180)."""
        size = torch.empty((), dtype=dtype).element_size()
        return sum(2 * need.kv_heads * need.head_dim * page_tokens * size
                   for need in needs if need is not None and need.kind == "kv_pages")

    def __init__(self, needs: Sequence[Optional[CacheNeed]], page_tokens: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype, device, allocate: bool = True):
        if page_tokens <= 0 or page_tokens & (page_tokens - 1):
            raise ValueError(f"page_tokens must be a power of two, got {page_tokens}")
        if num_pages <= 0:
            raise ValueError("the cache needs at least one page")
        self.page_tokens, self.max_requests = page_tokens, max_requests
        self.dtype, self.device = dtype, torch.device(device)
        self.groups: List[Group] = []
        self.entry_group: Dict[int, int] = {}
        self.entry_index: Dict[int, int] = {}
        self.states: Dict[int, torch.Tensor] = {}
        self.needs = list(needs)
        by_key: Dict[tuple, Group] = {}
        for entry, need in enumerate(self.needs):
            if need is None or need.kind == "none":
                continue
            if need.kind == "kv_pages":
                key = need.group_key()
                if key not in by_key:
                    by_key[key] = Group(len(self.groups), need, [], page_tokens, num_pages, None)
                    self.groups.append(by_key[key])
                group = by_key[key]
                self.entry_group[entry] = group.index
                self.entry_index[entry] = len(group.entries)
                group.entries.append(entry)
            elif need.kind == "state":
                if allocate:
                    self.states[entry] = torch.zeros(
                        (max_requests,) + tuple(need.state_shape),
                        dtype=getattr(torch, need.state_dtype), device=self.device)
            else:
                raise ValueError(f"unknown cache need {need.kind!r}")
        host = build.host()
        self.manager = host.CacheManager(
            [host.GroupConfig(page_tokens, g.need.window or 0, g.num_pages) for g in self.groups],
            max_requests)
        if allocate:
            for group in self.groups:
                group.pool = torch.zeros(
                    (len(group.entries), group.num_pages, 2, group.need.kv_heads, page_tokens,
                     group.need.head_dim), dtype=dtype, device=self.device)

    # ------------------------------------------------------------------ facts
    def bytes_per_token(self) -> int:
        """Bytes of keys and values one position takes over all groups."""
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * g.need.kv_heads * g.need.head_dim * size * len(g.entries) for g in self.groups)

    def pool_bytes(self) -> int:
        return sum(g.pool.numel() * g.pool.element_size() for g in self.groups if g.pool is not None)

    # ------------------------------------------------------------------- fork
    def fork(self, parent: int, child: int) -> None:
        """``child`` starts from everything ``parent`` has computed: the manager
        shares the full pages and names the partly filled ones and the state
        slot, which are copied here, on the device, in every layer of a group at
        once. Raises what the manager raises (no page, no slot) with nothing
        changed."""
        from .. import ops
        source_slot, target_slot, copies = self.manager.fork(parent, child)
        if self.device.type != "cuda":
            return
        for group in self.groups:
            pairs = [(source, target) for g, source, target in copies if g == group.index]
            if pairs and group.pool is not None:
                ops.copy_units(group.pool, torch.tensor(pairs, dtype=torch.int32, device=self.device))
        if self.states:
            slots = torch.tensor([[source_slot, target_slot]], dtype=torch.int32, device=self.device)
            for state in self.states.values():
                ops.copy_units(state.unsqueeze(0), slots)

    # ------------------------------------------------------------- step views
    def zero_state(self, slot: int) -> None:
        for state in self.states.values():
            state[slot].zero_()

    def view(self, entry: int, write: bool, tables: Dict[int, torch.Tensor],
             slots: Dict[int, torch.Tensor]) -> CacheView:
        need = self.needs[entry]
        if need is None or need.kind == "none":
            return CacheView(need=need or CacheNeed("none"), write=False)
        if need.kind == "state":
            return CacheView(need=need, state=self.states[entry], write=write)
        group = self.groups[self.entry_group[entry]]
        return CacheView(need=need, pool=group.pool[self.entry_index[entry]],
                         block_tables=tables[group.index],
                         slots=slots[group.index] if write else None, write=write)

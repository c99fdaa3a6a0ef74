"""The cache manager: device buffers, page groups, state slots, per-request holdings.

It is built from the cache needs of a model's run entries (``PagedKV`` /
``FixedState`` / none) and nothing else about the model.

Paged groups.  Entries that need all keys and entries that need a window of them are
different groups: each group has its own page pool and its own block table per request,
so a window group can give pages back as the window passes them while the other keeps
everything.  Within a group every entry has its own K and V buffer
``[num_pages, page_size, kv_heads, head_dim]`` (widths may differ between entries); a
page id names the same rows in all of them, as the reference's pages do
(crates/shiso-engine/src/kv.rs:18-31,97-109).

Fixed state.  One buffer ``[num_slots, bytes_per_slot]``; every fixed-state entry owns a
16-byte-aligned column range of it, seen in the entry's own element type (float32 unless
it asks otherwise), so one request's state of every such layer lies in one row and is
zeroed by one fill when the slot is assigned.

Requests.  ``append`` claims what ``n`` more tokens need in every group, all or
nothing, and raises ``OutOfPages`` otherwise (the reference fails the session there:
crates/shiso-engine/src/kv.rs:597-609); ``commit`` moves the length forward after the
step ran and returns window-passed pages; ``release`` gives everything back.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..parts.base import FixedState, PagedKV
from .pages import HOLE, BlockTable, OutOfPages, PagePool
from .slots import SlotPool


@dataclass
class PagedKVView:
    k: torch.Tensor
    v: torch.Tensor
    page_size: int
    group: int
    kv_heads: int
    head_dim: int
    owner: bool = True


@dataclass
class FixedStateView:
    state: torch.Tensor  # [num_slots, *shape], a strided view of the slot buffer
    owner: bool = True


class _Group:
    def __init__(self, index: int, window: Optional[int], num_pages: int):
        self.index = index
        self.window = window
        self.pool = PagePool(num_pages)


class _Held:
    """What one request holds."""

    def __init__(self, tables: list[BlockTable], slot: Optional[int]):
        self.tables = tables
        self.slot = slot
        self.length = 0  # positions written by finished steps
        self.reserved = 0  # positions claimed for the step in flight


class CacheManager:
    def __init__(
        self,
        needs: list,  # per run entry: PagedKV | FixedState | None
        page_size: int,
        num_pages: int,
        num_slots: int,
        dtype: torch.dtype,
        device,
        max_blocks_per_request: Optional[int] = None,
        scratch_tokens: int = 0,
    ):
        """``scratch_tokens`` > 0 adds, behind the pool, pages for that many positions and one
        state slot that no request ever holds (``scratch_pages``, ``scratch_slot``): the rows
        with which a step is padded to a captured shape write there."""
        if page_size <= 0:
            raise ValueError(f"page size must be positive, got {page_size}")
        self.page_size = page_size
        self.dtype = dtype
        self.device = torch.device(device)
        self.needs = list(needs)
        scratch_pages = -(-scratch_tokens // page_size) if scratch_tokens > 0 else 0
        self.scratch_pages = list(range(num_pages, num_pages + scratch_pages))
        self.scratch_slot = num_slots if scratch_tokens > 0 else None
        buffer_pages = num_pages + scratch_pages
        self.groups: list[_Group] = []
        self._views: list = [None] * len(needs)
        by_window: dict = {}
        for pos, need in enumerate(needs):
            if isinstance(need, PagedKV):
                if need.window is not None and need.window <= 0:
                    raise ValueError(f"run entry {pos}: window {need.window} must be positive")
                if need.window not in by_window:
                    group = _Group(len(self.groups), need.window, num_pages)
                    self.groups.append(group)
                    by_window[need.window] = group
                group = by_window[need.window]
                kv_dtype = need.dtype if need.dtype is not None else dtype
                self._views[pos] = PagedKVView(
                    k=torch.zeros((buffer_pages, page_size, need.num_kv_heads, need.head_dim), dtype=kv_dtype, device=self.device),
                    v=torch.zeros((buffer_pages, page_size, need.num_kv_heads, need.value_dim), dtype=kv_dtype, device=self.device),
                    page_size=page_size,
                    group=group.index,
                    kv_heads=need.num_kv_heads,
                    head_dim=need.head_dim,
                )
        self.num_pages = num_pages
        self.max_blocks = max_blocks_per_request or num_pages

        # Fixed-size state: one row of bytes per slot, one aligned column range per entry.
        offsets, total = {}, 0
        for pos, need in enumerate(needs):
            if isinstance(need, FixedState):
                offsets[pos] = total
                total += -(-need.nbytes // 16) * 16
        self.bytes_per_slot = total
        self.slots = SlotPool(num_slots)
        self.num_slots = num_slots
        self.state = torch.zeros((num_slots + (1 if scratch_tokens > 0 else 0), max(total, 16)), dtype=torch.uint8, device=self.device)
        for pos, off in offsets.items():
            need = needs[pos]
            view = self.state[:, off : off + need.nbytes].view(need.dtype).unflatten(1, need.shape)
            self._views[pos] = FixedStateView(state=view)

        self._held: dict = {}

    @staticmethod
    def costs(needs: list, page_size: int, dtype: torch.dtype) -> tuple:
        """``(bytes of one page across every paged entry, bytes of one state slot)``: what the
        pool's sizing needs to know about a model (the reference prices pages run by run the
        same way, crates/shiso-engine/src/kv.rs:26-31,84-109,176-198)."""
        page_bytes = state_bytes = 0
        for need in needs:
            if isinstance(need, PagedKV):
                itemsize = (need.dtype if need.dtype is not None else dtype).itemsize
                page_bytes += page_size * need.num_kv_heads * (need.head_dim + need.value_dim) * itemsize
            elif isinstance(need, FixedState):
                state_bytes += -(-need.nbytes // 16) * 16
        return page_bytes, state_bytes

    # ------------------------------------------------------------------ views for the model

    def view(self, entry: int, owner: bool = True):
        """The cache view of a run entry; ``owner=False`` for an entry that borrows it."""
        view = self._views[entry]
        if view is None or owner:
            return view
        if isinstance(view, PagedKVView):
            return PagedKVView(view.k, view.v, view.page_size, view.group, view.kv_heads, view.head_dim, owner=False)
        return FixedStateView(view.state, owner=False)

    # ------------------------------------------------------------------ requests

    def has(self, request) -> bool:
        return request in self._held

    def length(self, request) -> int:
        return self._held[request].length

    def live_requests(self) -> list:
        return list(self._held)

    def pages_needed(self, request, n_tokens: int) -> list[int]:
        """Pages per group that ``n_tokens`` more tokens of ``request`` (known or new) need."""
        held = self._held.get(request)
        out = []
        for group in self.groups:
            if held is None:
                out.append(-(-n_tokens // self.page_size))
            else:
                out.append(held.tables[group.index].missing_for(held.length + n_tokens))
        return out

    def can_append(self, request, n_tokens: int) -> bool:
        if request not in self._held and self.slots.free_slots == 0:
            return False
        needed = self.pages_needed(request, n_tokens)
        return all(n <= g.pool.free_pages for n, g in zip(needed, self.groups))

    def free_pages(self) -> list[int]:
        return [g.pool.free_pages for g in self.groups]

    def append(self, request, n_tokens: int) -> int:
        """Claims room for ``n_tokens`` more tokens; returns the position of the first.

        A request seen for the first time gets a zeroed state slot and empty block
        tables.  Everything is claimed or nothing is."""
        if n_tokens <= 0:
            raise ValueError(f"request {request!r}: a step brings at least one token")
        held = self._held.get(request)
        fresh = held is None
        if not fresh and held.reserved:
            raise RuntimeError(f"request {request!r} appears twice in one step")
        needed = self.pages_needed(request, n_tokens)
        for n, group in zip(needed, self.groups):
            if n > group.pool.free_pages:
                raise OutOfPages(n, group.pool.free_pages)
        new_length = (0 if fresh else held.length) + n_tokens
        if -(-new_length // self.page_size) > self.max_blocks:
            raise OutOfPages(-(-new_length // self.page_size), self.max_blocks, "blocks per request allowed")
        if fresh:
            slot = self.slots.take()  # raises OutOfPages before anything else is taken
            if self.bytes_per_slot:
                self.state[slot].zero_()
            held = _Held([BlockTable(self.page_size, g.window) for g in self.groups], slot)
            self._held[request] = held
        for group in self.groups:
            held.tables[group.index].grow(group.pool, held.length + n_tokens)
        held.reserved = n_tokens
        return held.length

    def commit(self, request) -> None:
        """The step that ``append`` prepared has run: the new positions now count."""
        held = self._held[request]
        held.length += held.reserved
        held.reserved = 0
        for group in self.groups:
            held.tables[group.index].release_passed(group.pool, held.length)

    def cancel(self, request) -> None:
        """The step that ``append`` prepared did not run: the pages it claimed go back."""
        held = self._held[request]
        held.reserved = 0
        for group in self.groups:
            held.tables[group.index].shrink(group.pool, held.length)

    def release(self, request) -> None:
        held = self._held.pop(request, None)
        if held is None:
            raise KeyError(f"request {request!r} holds nothing")
        for group in self.groups:
            held.tables[group.index].release_all(group.pool)
        self.slots.give_back(held.slot)

    def slot_of(self, request) -> int:
        return self._held[request].slot

    def block_table(self, request, group: int) -> list[int]:
        return self._held[request].tables[group].pages

    def fill_block_tables(self, requests: list, group: int, out: np.ndarray) -> None:
        """Writes the requests' tables of one group into ``out[len(requests), width]``;
        unused entries and holes are ``-1`` and are never read (the causal bound and
        the window stop first)."""
        out.fill(HOLE)
        for i, request in enumerate(requests):
            pages = self._held[request].tables[group].as_array()
            if len(pages) > out.shape[1]:
                raise RuntimeError(f"request {request!r} holds {len(pages)} blocks, the table has {out.shape[1]} columns")
            out[i, : len(pages)] = pages

    def max_blocks_held(self, requests: list) -> int:
        most = 1
        for request in requests:
            for table in self._held[request].tables:
                most = max(most, len(table.pages))
        return most

    def check(self) -> None:
        """Bookkeeping invariants: no page lost, held twice or free while held."""
        for group in self.groups:
            group.pool.check()
            seen = set()
            for request, held in self._held.items():
                for page in held.tables[group.index].live_pages():
                    if page in seen:
                        raise RuntimeError(f"page {page} of group {group.index} is held twice")
                    if group.pool.holders(page) != 1:
                        raise RuntimeError(f"page {page} is in a block table but the pool counts {group.pool.holders(page)} holders")
                    seen.add(page)
            if len(seen) != group.pool.used_pages:
                raise RuntimeError(
                    f"group {group.index}: {group.pool.used_pages} pages are out of the pool, block tables name {len(seen)}"
                )
        self.slots.check()
        slots = [h.slot for h in self._held.values()]
        if len(set(slots)) != len(slots):
            raise RuntimeError("two requests share a state slot")

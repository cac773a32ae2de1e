"""The cache manager: pages of keys and values, block tables, and state slots.

Storage
-------
Every schedule entry that owns a cache says, as a `KVSpec`, what it stores per
position: a list of rows `(heads, width)` (an attention mixer's keys and values are two
equal rows; a latent cache is one), a window, and how many positions share a stored row.
Entries whose specs are equal form a *group*; a group has its own pool of pages and, per
request, its own block table. One tensor per group holds its pages: page `p` of entry
`e` is `tensor[e, p]`, laid out row after row, each row `[heads, page_size, width]`; a
group of equal rows is shaped `[entries, pages, rows, heads, page_size, width]` (keys at
index 0 and values at index 1 of the rows' axis for attention), any other
`[entries, pages, elements per page]`. A request's logical page `i` holds stored rows
`i * page_size` to `(i + 1) * page_size - 1` and maps to the same physical page number
in every entry of the group. Groups may differ in how many pages a request needs of
them (`KVSpec.stride`), so every count below is per group.

A group with a window gives a page back as soon as every position in it is behind
the window of all tokens still to come; its block-table entry becomes -1. All pages
return when the request ends. Freed pages are handed out again, last freed first.

Beside the pages there are *state slots*: a request holds one slot number for its
whole life, and every entry that declares a `StateSpec` has a tensor
`[slots + 1, *shape]` indexed by it; the last row is a scratch slot that belongs to no
request (the padding rows of a captured step point at it). A slot is set to the mixer's
initial state when a request's first step runs. Muse-Glimmer declares no state; the
slots exist so a mixer with state of its own needs no change here.

The reference keeps one growing buffer per request and layer instead
(src/mlx_omnia/engine/core/cache/kv.py:18-128) and says which rows a window makes
unreadable through `Rows.keep` (src/mlx_omnia/engine/core/cache/layout.py:14-24);
paging, groups and slots are this engine's own design.

All bookkeeping is host-side Python and runs without a GPU (`device="meta"` or
`allocate=False` skips the tensors).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from mlx_omnia_b200.parts.base import KVSpec
from mlx_omnia_b200.parts.model import CacheNeed


class CacheError(RuntimeError):
    """Misuse of the cache manager: a page freed twice, an unknown request, ..."""


class PagePool:
    """Page numbers 0..count-1; a stack of free ones (last freed, first reused)."""

    def __init__(self, count: int) -> None:
        self.count = count
        self._free = list(range(count - 1, -1, -1))
        self._held = [False] * count

    @property
    def free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError("no free page")
        page = self._free.pop()
        self._held[page] = True
        return page

    def give(self, page: int) -> None:
        if not 0 <= page < self.count:
            raise CacheError(f"page {page} is not in a pool of {self.count}")
        if not self._held[page]:
            raise CacheError(f"page {page} is freed twice")
        self._held[page] = False
        self._free.append(page)

    def held(self) -> list[int]:
        return [p for p, h in enumerate(self._held) if h]


@dataclass
class Group:
    spec: KVSpec
    entries: list[int]  # schedule entries stored in this group, in tensor order
    pool: PagePool
    pages: torch.Tensor | None  # [entries, pages, rows, heads, page_size, width] or [entries, pages, elements]


@dataclass
class RequestCache:
    """What one live request holds."""

    request_id: str
    tokens: int = 0  # positions written so far
    tables: list[list[int]] = field(default_factory=list)  # per group: physical page per logical page (-1 freed)
    slot: int = -1
    fresh: bool = True  # no step has run for it yet
    # int32 copies of `tables` (capacity grown by doubling; entries beyond len(tables[g]) are -1),
    # so that a step lays its block tables out with array copies instead of Python loops
    arrays: list[np.ndarray] = field(default_factory=list)

    def table_array(self, group: int) -> np.ndarray:
        return self.arrays[group][: len(self.tables[group])]


class CacheManager:
    def __init__(self, needs: list[CacheNeed], *, page_size: int, pages_per_group: int | dict[KVSpec, int],
                 max_requests: int, dtype: torch.dtype = torch.bfloat16, device: torch.device | str = "cpu",
                 allocate: bool = True) -> None:
        if page_size < 1:
            raise ValueError("page_size must be at least 1")
        self.page_size = page_size
        self.needs = needs
        self.groups: list[Group] = []
        self.group_of_entry: dict[int, tuple[int, int]] = {}  # entry -> (group, index in group)
        by_spec: dict[KVSpec, int] = {}
        for entry, need in enumerate(needs):
            if need.kv is None:
                continue
            g = by_spec.get(need.kv)
            if g is None:
                g = by_spec[need.kv] = len(self.groups)
                count = pages_per_group[need.kv] if isinstance(pages_per_group, dict) else pages_per_group
                self.groups.append(Group(need.kv, [], PagePool(count), None))
            self.group_of_entry[entry] = (g, len(self.groups[g].entries))
            self.groups[g].entries.append(entry)
        for entry, need in enumerate(needs):
            if need.reads is not None:
                if need.reads not in self.group_of_entry:
                    raise ValueError(f"schedule entry {entry} reads entry {need.reads}, which keeps no pages")
                self.group_of_entry[entry] = self.group_of_entry[need.reads]
        if allocate:
            for group in self.groups:
                s = group.spec
                shape = (len(s.rows), *s.rows[0][:1], page_size, s.rows[0][1]) if s.uniform else \
                    (s.elements_per_position * page_size,)
                group.pages = torch.zeros(len(group.entries), group.pool.count, *shape, dtype=dtype, device=device)
        self.slots = PagePool(max_requests)
        self.scratch_slot = max_requests  # the state row that padding rows of a captured step point at
        self.state: dict[int, torch.Tensor] = {}
        self.initial_state: dict[int, torch.Tensor] = {}  # entries whose state does not start as zeros
        for entry, need in enumerate(needs):
            if need.state is not None and allocate:
                self.state[entry] = torch.zeros(max_requests + 1, *need.state.shape, dtype=need.state.dtype,
                                                device=device)
                if need.initial_state is not None:
                    self.initial_state[entry] = need.initial_state.to(need.state.dtype).to(device)
        self.requests: dict[str, RequestCache] = {}

    # -- sizes -----------------------------------------------------------------------
    @staticmethod
    def bytes_per_token(needs: list[CacheNeed], element_size: int) -> int:
        """Cache bytes one position costs over all entries that own pages (what a pool is
        sized by when the caller names no size)."""
        return sum(-(-need.kv.elements_per_position // need.kv.stride) * element_size
                   for need in needs if need.kv is not None)

    def bytes_per_page(self, group: int, element_size: int) -> int:
        g = self.groups[group]
        return len(g.entries) * g.spec.elements_per_position * self.page_size * element_size

    def pages_for(self, group: int, tokens: int) -> int:
        """Pages of `group` that a request of `tokens` positions occupies (none given back)."""
        return -(-self.groups[group].spec.stored(tokens) // self.page_size)

    def pages_needed(self, request: RequestCache, new_tokens: int) -> list[int]:
        """Pages each group must take for `request` to grow by `new_tokens`."""
        return [self.pages_for(g, request.tokens + new_tokens) - self.pages_for(g, request.tokens)
                for g in range(len(self.groups))]

    def capacity_tokens(self) -> int:
        """The longest request the pools can hold (the tightest group decides)."""
        return min((g.pool.count * self.page_size * g.spec.stride for g in self.groups), default=1 << 30)

    def can_grow(self, request: RequestCache, new_tokens: int, reserve: list[int] | None = None) -> bool:
        need = self.pages_needed(request, new_tokens)
        return all(n <= g.pool.free - (reserve[i] if reserve else 0)
                   for i, (n, g) in enumerate(zip(need, self.groups)))

    # -- life of a request -------------------------------------------------------------
    def open(self, request_id: str) -> RequestCache:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already open")
        if self.slots.free == 0:
            raise CacheError("no free request slot")
        request = RequestCache(request_id, tables=[[] for _ in self.groups], slot=self.slots.take(),
                               arrays=[np.full(16, -1, dtype=np.int32) for _ in self.groups])
        self.requests[request_id] = request
        return request

    def grow(self, request: RequestCache, new_tokens: int) -> None:
        """Take the pages for the next `new_tokens` positions in every group, or none
        at all (CacheError) when some group has too few free pages."""
        if new_tokens < 0:
            raise ValueError("new_tokens must not be negative")
        need = self.pages_needed(request, new_tokens)
        for n, group in zip(need, self.groups):
            if n > group.pool.free:
                raise CacheError(f"group {group.spec} needs {n} pages, {group.pool.free} free")
        for g, (n, group, table) in enumerate(zip(need, self.groups, request.tables)):
            if len(table) + n > len(request.arrays[g]):
                grown = np.full(max(2 * len(request.arrays[g]), len(table) + n), -1, dtype=np.int32)
                grown[: len(table)] = request.arrays[g][: len(table)]
                request.arrays[g] = grown
            for _ in range(n):
                request.arrays[g][len(table)] = page = group.pool.take()
                table.append(page)
        request.tokens += new_tokens

    def slot_of(self, request: RequestCache, group: int, position: int) -> int:
        row = position // self.groups[group].spec.stride
        page = request.tables[group][row // self.page_size]
        if page < 0:
            raise CacheError(f"position {position} of {request.request_id!r} lies in a page already given back")
        return page * self.page_size + row % self.page_size

    def release_behind_window(self, request: RequestCache) -> int:
        """Give back pages of windowed groups that no later token can read. With
        `tokens` positions written, the next query sits at position >= tokens and sees
        keys >= tokens - window + 1. Returns how many pages were freed."""
        freed = 0
        for g, (group, table) in enumerate(zip(self.groups, request.tables)):
            window = group.spec.window
            if window is None:
                continue
            dead_below = request.tokens - window + 1  # positions < this are never read again
            dead_rows = max(dead_below, 0) // group.spec.stride  # stored rows wholly below it
            for index in range(min(len(table), dead_rows // self.page_size) - 1, -1, -1):
                if table[index] < 0:
                    break  # everything below was given back earlier
                group.pool.give(table[index])
                table[index] = request.arrays[g][index] = -1
                freed += 1
        return freed

    def close(self, request_id: str) -> None:
        """The request ended: everything it holds is given back."""
        request = self.requests.pop(request_id, None)
        if request is None:
            raise CacheError(f"request {request_id!r} is not open")
        for group, table in zip(self.groups, request.tables):
            for page in table:
                if page >= 0:
                    group.pool.give(page)
            table.clear()
        self.slots.give(request.slot)
        request.slot = -1

    # -- views for a step --------------------------------------------------------------
    def entry_pages(self, entry: int) -> torch.Tensor:
        g, index = self.group_of_entry[entry]
        return self.groups[g].pages[index]

    def check(self) -> None:
        """Every page is either free or in exactly one table (used by tests)."""
        for g, group in enumerate(self.groups):
            seen: dict[int, str] = {}
            for request in self.requests.values():
                for page in request.tables[g]:
                    if page < 0:
                        continue
                    if page in seen:
                        raise CacheError(f"page {page} of group {g} is held by {seen[page]!r} and {request.request_id!r}")
                    seen[page] = request.request_id
            if sorted(seen) != group.pool.held():
                raise CacheError(f"group {g}: pages in tables {sorted(seen)} differ from pages taken {group.pool.held()}")
            if len(seen) + group.pool.free != group.pool.count:
                raise CacheError(f"group {g}: a page was lost")

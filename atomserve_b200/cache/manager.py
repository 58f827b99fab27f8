"""The cache manager: pages of keys and values in groups, a block table per request and
group, and per-request state slots.

Entries of the model's run order that own a cache are sorted into groups by what they need:
the tensors a page holds (for attention: keys and values of kv heads x head size) and the
window. Each group has, per tensor, its own pool `[entries, num_blocks, heads, block_size,
width]`, and its own allocator and, per request, its own block table. Position p of a request lives in page
`table[p // block_size]` at offset `p % block_size`; the slot written is
`page * block_size + offset` (atomserve/kv_cache.py:9-14). Pools start zeroed so that no read
can meet a NaN (atomserve/kv_cache.py:112-118).

Pages come back when a request ends or is preempted, and, in a windowed group, as soon as the
window has passed them: before a step that starts at position c, pages wholly below
c - window + 1 are released and their table entries set to -1.

The reference has one uniform pool (atomserve/kv_cache.py:89-135) and lets the scheduler talk to
the allocator directly (atomserve/scheduler.py:204-254); here the scheduler talks to this
manager, which keeps the groups in step: a reservation succeeds in every group or in none.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field

import torch

from atomserve_b200.cache.block_allocator import BlockAllocator, block_hash, blocks_for_tokens
from atomserve_b200.cache.state_slots import StateSlots
from atomserve_b200.parts.base import CacheView, PageSpec, StateSpec


@dataclass
class RequestCache:
    """What one request holds: a block table per group (-1: released) and a state slot."""

    block_tables: list[list[int]]
    state_slot: int = -1
    block_hashes: list[bytes] = field(default_factory=list)  # of full, computed pages (prefix cache)
    uid: int = field(default_factory=itertools.count().__next__)  # never reused, unlike id()
    generation: int = 0  # bumped whenever the tables are emptied: copies of them are then stale

    @property
    def block_table(self) -> list[int]:
        return self.block_tables[0]


@dataclass
class CacheGroup:
    spec: PageSpec
    entries: list[int]  # run-order indices whose pages live here, in pool order
    allocator: BlockAllocator
    # per tensor of the spec: [len(entries), num_blocks, heads, block_size, width]
    pools: dict[str, torch.Tensor] = field(default_factory=dict)

    @property
    def k(self) -> torch.Tensor | None:
        return self.pools.get("k")

    @property
    def v(self) -> torch.Tensor | None:
        return self.pools.get("v")

    @property
    def window(self) -> int | None:
        return self.spec.window


class CacheManager:
    def __init__(
        self,
        requirements: list[tuple[PageSpec | None, list[StateSpec]]],
        block_size: int,
        num_blocks: int,
        num_state_slots: int,
        dtype: torch.dtype = torch.float32,
        device: torch.device | str | None = None,
    ):
        """requirements: per run-order entry, what it owns (DecoderModel.cache_requirements).
        device None: bookkeeping only, no tensors (scheduler tests)."""
        self.block_size, self.num_blocks, self.dtype = block_size, num_blocks, dtype
        self.device = torch.device(device) if device is not None else None
        self.groups: list[CacheGroup] = []
        self.entry_group: dict[int, tuple[int, int]] = {}  # run-order index -> (group, index in group)
        self.entry_state: dict[int, dict[str, torch.Tensor]] = {}
        self.state = StateSlots(num_state_slots, self.device or "cpu")
        by_key: dict[PageSpec, int] = {}
        for i, (kv, states) in enumerate(requirements):
            if kv is not None:
                if kv not in by_key:
                    by_key[kv] = len(self.groups)
                    self.groups.append(CacheGroup(kv, [], BlockAllocator(num_blocks)))
                g = by_key[kv]
                self.entry_group[i] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(i)
            if states:
                self.entry_state[i] = {
                    s.name: self.state.register(f"{i}.{s.name}", tuple(s.shape), s.dtype) for s in states
                }
        self._windowed = any(g.window is not None for g in self.groups)  # only windows release pages early
        if self.device is not None:
            for g in self.groups:
                for t in g.spec.tensors:
                    shape = (len(g.entries), num_blocks, t.heads, block_size, t.width)
                    g.pools[t.name] = torch.zeros(shape, dtype=dtype, device=self.device)

    # ---- sizes --------------------------------------------------------------------------------

    @staticmethod
    def bytes_per_block(requirements: list[tuple[PageSpec | None, list[StateSpec]]], block_size: int, dtype: torch.dtype) -> int:
        """Memory that one page id costs across all entries and the tensors of their pages
        (atomserve/kv_cache.py:129-135)."""
        per_token = sum(spec.values_per_token for spec, _ in requirements if spec is not None)
        return per_token * block_size * dtype.itemsize

    @property
    def supports_prefix_caching(self) -> bool:
        """Sharing pages by content is sound only when all that a request keeps are pages of one
        unwindowed group (a window releases pages, state is not content-addressed)."""
        return len(self.groups) == 1 and self.groups[0].window is None and not self.entry_state

    @property
    def num_free_blocks(self) -> int:
        return min((g.allocator.num_free for g in self.groups), default=self.num_blocks)

    # ---- a request's life ---------------------------------------------------------------------

    def new_request(self) -> RequestCache:
        return RequestCache([[] for _ in self.groups])

    def admit(self, rc: RequestCache) -> bool:
        """Give the request its state slot; False if none is free."""
        if rc.state_slot >= 0:
            return True
        if self.state.num_free == 0:
            return False
        rc.state_slot = self.state.take()
        return True

    def first_needed_block(self, group: CacheGroup, start: int) -> int:
        """The lowest logical page a step starting at position `start` can still read."""
        if group.window is None:
            return 0
        return max(0, start - group.window + 1) // self.block_size

    def release_passed(self, rc: RequestCache, start: int) -> None:
        """Give back the pages that every window has passed before position `start` runs."""
        for g, table in zip(self.groups, rc.block_tables):
            if g.window is None:
                continue
            upto = min(self.first_needed_block(g, start), len(table))
            passed = [b for b in table[:upto] if b >= 0]
            if passed:
                g.allocator.free(passed)
                for i in range(upto):
                    table[i] = -1

    def reserve(self, rc: RequestCache, start: int, num_new: int) -> bool:
        """Make room for positions [start, start + num_new) in every group, or in none.
        Pages a window has passed are released first (that is never undone: no later step
        reads them)."""
        if self._windowed:
            self.release_passed(rc, start)
        needed = blocks_for_tokens(start + num_new, self.block_size)
        for t in rc.block_tables:
            if len(t) < needed:
                break
        else:
            return True  # the usual decode step: the last page still has room
        missing = [max(0, needed - len(t)) for t in rc.block_tables]
        if any(m > g.allocator.num_free for g, m in zip(self.groups, missing)):
            return False
        for g, table, m in zip(self.groups, rc.block_tables, missing):
            if m:
                table.extend(g.allocator.allocate(m))
        return True

    def free(self, rc: RequestCache) -> None:
        """Give back everything the request holds (end, abort, preemption)."""
        for g, table in zip(self.groups, rc.block_tables):
            held = [b for b in table if b >= 0]
            if held:
                g.allocator.free(held)
            table.clear()
        rc.generation += 1
        rc.block_hashes.clear()
        if rc.state_slot >= 0:
            self.state.give_back(rc.state_slot)
            rc.state_slot = -1

    # ---- prefix cache (single unwindowed group only) ------------------------------------------

    def use_cached_prefix(self, rc: RequestCache, token_ids: list[int]) -> int:
        """Point the request's table at pages that already hold its leading full pages; returns
        the number of tokens covered. At least one token is always left to compute
        (atomserve/scheduler.py:214-233)."""
        if not self.supports_prefix_caching:
            return 0
        alloc, table, bs = self.groups[0].allocator, rc.block_tables[0], self.block_size
        parent = b""
        for i in range((len(token_ids) - 1) // bs):
            h = block_hash(parent, token_ids[i * bs : (i + 1) * bs])
            block = alloc.lookup(h)
            if block is None:
                break
            alloc.acquire(block)
            table.append(block)
            rc.block_hashes.append(h)
            parent = h
        return len(table) * bs

    def register_full_blocks(self, rc: RequestCache, token_ids: list[int], num_computed: int) -> None:
        """Publish the pages that are now full and computed (atomserve/scheduler.py:235-250)."""
        if not self.supports_prefix_caching:
            return
        alloc, table, bs = self.groups[0].allocator, rc.block_tables[0], self.block_size
        while len(rc.block_hashes) < num_computed // bs:
            i = len(rc.block_hashes)
            parent = rc.block_hashes[-1] if i else b""
            h = block_hash(parent, token_ids[i * bs : (i + 1) * bs])
            alloc.register(table[i], h)
            rc.block_hashes.append(h)

    # ---- views for the step function ----------------------------------------------------------

    def entry_view(self, entry: int) -> CacheView | None:
        """The tensors of one run-order entry (slots and tables are filled in per step)."""
        view = CacheView(block_size=self.block_size)
        if entry in self.entry_group:
            g, j = self.entry_group[entry]
            view.pages = {name: pool[j] for name, pool in self.groups[g].pools.items()}
        if entry in self.entry_state:
            view.state = self.entry_state[entry]
        if entry not in self.entry_group and entry not in self.entry_state:
            return None
        return view

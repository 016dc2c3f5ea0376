"""Plain model of the paged cache bookkeeping, in Python: what the engine's C++ cache manager
is compared with.  Tests drive both with the same calls and compare every block table, length,
slot and free count.  It shares no code with the product.

The reference keeps keys and values in growing segments per session and uses
pages only as the unit of admission (crates/leone/src/kv.rs:14-31, 637-674;
crates/leone/src/scheduler.rs:652-667 rounds a reservation up to
``kv_page_tokens``).  Here the pages are real: a request's tokens live in
fixed-size pages scattered over a pool and found through its block table.
What is kept from the reference is the transaction: space for a step is
reserved before the step runs and a request's length advances only when the
step is committed (``prepare_append`` → ``write_span`` → ``commit_append``,
crates/leone/src/kv.rs:326-347, 791-927); a failed step rolls back.

Layers with different needs form different *groups*.  A group has its own
pool and its own block table per request.  Two kinds exist: ``full`` keeps
every page until the request ends; ``window`` gives a page back as soon as
every later query lies more than ``window`` tokens past its last token.
Fixed-size per-request state (a mixer with a recurrent state, sampling state)
lives in numbered slots, one per live request.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np


class OutOfPages(RuntimeError):
    """Not enough free pages (or state slots) for what was asked."""


class CacheError(RuntimeError):
    """A call that breaks the manager's rules (unknown request, double free...)."""


class PagePool:
    """Free list over page ids ``0..num_pages-1``; LIFO so freed pages are reused at once."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, count: int) -> List[int]:
        if count > len(self._free):
            raise OutOfPages(f"asked for {count} pages, {len(self._free)} free of {self.num_pages}")
        pages = [self._free.pop() for _ in range(count)]
        for p in pages:
            if self._held[p]:
                raise CacheError(f"page {p} handed out twice")
            self._held[p] = True
        self.high_water = max(self.high_water, self.num_held)
        return pages

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or not self._held[p]:
                raise CacheError(f"page {p} freed but not held")
            self._held[p] = False
            self._free.append(p)


@dataclass
class GroupSpec:
    """What a group of layers needs from the cache."""
    kind: str                   # "full" or "window"
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    layers: List[int] = field(default_factory=list)

    def key(self):
        return (self.kind, self.num_kv_heads, self.head_dim, self.window)


class CacheGroup:
    def __init__(self, gid: int, spec: GroupSpec, page_tokens: int, num_pages: int):
        if spec.kind not in ("full", "window"):
            raise ValueError(f"unknown cache group kind '{spec.kind}'")
        if spec.kind == "window" and (spec.window is None or spec.window <= 0):
            raise ValueError("a window group needs a positive window")
        self.gid = gid
        self.spec = spec
        self.page_tokens = page_tokens
        self.pool = PagePool(num_pages)
        # request -> list of page ids by logical block; -1 where a window has passed.
        self.tables: Dict[Hashable, List[int]] = {}

    def blocks_for(self, length: int) -> int:
        return -(-length // self.page_tokens)

    def first_live_block(self, committed_len: int) -> int:
        """First logical block that a query at position >= committed_len can still read."""
        if self.spec.kind != "window":
            return 0
        oldest_key = committed_len - self.spec.window + 1
        return max(0, oldest_key // self.page_tokens)

    def pages_needed(self, table: List[int], new_len: int) -> int:
        return max(0, self.blocks_for(new_len) - len(table))

    def pages_for_request(self, total_len: int) -> int:
        """Upper bound of pages a request of ``total_len`` tokens holds at one time."""
        if self.spec.kind == "full":
            return self.blocks_for(total_len)
        # A window request holds the window's blocks plus the blocks of one step's portion;
        # the caller adds the portion.  Without that knowledge the bound is the full length.
        return self.blocks_for(total_len)


class StateSlots:
    """Numbered fixed-size slots, one per live request."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages(f"all {self.num_slots} state slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise CacheError(f"state slot {slot} freed but not held")
        self._held[slot] = False
        self._free.append(slot)


@dataclass
class RequestCache:
    slot: int
    committed_len: int = 0
    reserved_len: int = 0
    fresh: bool = True          # no step has been committed yet: state slot must be cleared
    version: int = 0            # changes whenever a block table changes other than by growing at its end


class CacheManager:
    """Block tables and state slots of all live requests over all groups."""

    def __init__(self, group_specs: Sequence[GroupSpec], page_tokens: int, num_pages: int,
                 num_slots: int):
        self.page_tokens = page_tokens
        self.groups = [CacheGroup(i, s, page_tokens, num_pages) for i, s in enumerate(group_specs)]
        self.slots = StateSlots(num_slots)
        self.requests: Dict[Hashable, RequestCache] = {}
        self._versions = 0

    # -- lifetime -------------------------------------------------------------------
    def open(self, rid: Hashable) -> int:
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already open")
        slot = self.slots.take()
        self._versions += 1
        self.requests[rid] = RequestCache(slot=slot, version=self._versions)
        for g in self.groups:
            g.tables[rid] = []
        return slot

    def close(self, rid: Hashable) -> None:
        rc = self._get(rid)
        for g in self.groups:
            table = g.tables.pop(rid)
            g.pool.give_back([p for p in table if p >= 0])
        self.slots.give_back(rc.slot)
        del self.requests[rid]

    def is_open(self, rid: Hashable) -> bool:
        return rid in self.requests

    def _get(self, rid: Hashable) -> RequestCache:
        if rid not in self.requests:
            raise CacheError(f"request {rid!r} is not open")
        return self.requests[rid]

    def length(self, rid: Hashable) -> int:
        return self._get(rid).committed_len

    def slot(self, rid: Hashable) -> int:
        return self._get(rid).slot

    def table_version(self, rid: Hashable) -> int:
        """A number that changes whenever one of the request's block tables changes other than
        by growing at its end (a mirror of the tables may then append instead of rewriting)."""
        return self._get(rid).version

    # -- the step transaction -------------------------------------------------------
    def can_reserve(self, wants: Dict[Hashable, int]) -> bool:
        """Would ``reserve`` succeed for these (request → new length) pairs together?"""
        for g in self.groups:
            need = sum(g.pages_needed(g.tables[rid], new_len) for rid, new_len in wants.items())
            if need > g.pool.num_free:
                return False
        return True

    def reserve(self, wants: Dict[Hashable, int]) -> None:
        """Take pages so each request can hold ``new_len`` tokens.  All or nothing."""
        for rid, new_len in wants.items():
            rc = self._get(rid)
            if new_len < rc.committed_len:
                raise CacheError(f"request {rid!r}: cannot reserve {new_len} below its length")
        if not self.can_reserve(wants):
            raise OutOfPages("not enough free pages for this step")
        for rid, new_len in wants.items():
            rc = self.requests[rid]
            for g in self.groups:
                table = g.tables[rid]
                table.extend(g.pool.take(g.pages_needed(table, new_len)))
            rc.reserved_len = max(rc.reserved_len, new_len)

    def commit(self, rid: Hashable, new_len: int) -> None:
        """The step that wrote tokens up to ``new_len`` succeeded."""
        rc = self._get(rid)
        if new_len > rc.reserved_len or new_len < rc.committed_len:
            raise CacheError(f"request {rid!r}: commit to {new_len} outside what was reserved")
        rc.committed_len = new_len
        rc.fresh = False
        for g in self.groups:
            if g.spec.kind != "window":
                continue
            table = g.tables[rid]
            live_from = min(g.first_live_block(new_len), len(table))
            passed = [p for p in table[:live_from] if p >= 0]
            if passed:
                g.pool.give_back(passed)
                for b in range(live_from):
                    table[b] = -1
                self._versions += 1
                rc.version = self._versions

    def rollback(self, rid: Hashable) -> None:
        """The step failed: return pages beyond the committed length."""
        self.truncate(rid, self._get(rid).committed_len)

    def truncate(self, rid: Hashable, length: int) -> None:
        """Drop everything past ``length`` tokens (crates/leone/src/kv.rs:929-950)."""
        rc = self._get(rid)
        if length > rc.committed_len:
            raise CacheError(f"request {rid!r}: cannot truncate to {length} past its length")
        for g in self.groups:
            # a rewind into what a window group has already released cannot be served
            if g.spec.kind == "window":
                table = g.tables[rid]
                for b in range(g.first_live_block(length), min(g.blocks_for(length), len(table))):
                    if table[b] < 0:
                        raise CacheError(f"request {rid!r}: cannot truncate to {length}: block {b} was released")
        for g in self.groups:
            table = g.tables[rid]
            keep = g.blocks_for(length)
            extra = [p for p in table[keep:] if p >= 0]
            g.pool.give_back(extra)
            if len(table) > keep:
                self._versions += 1
                rc.version = self._versions
            del table[keep:]
        rc.committed_len = length
        rc.reserved_len = length

    # -- views for the step function --------------------------------------------------
    def block_table(self, gid: int, rids: Sequence[Hashable], width: Optional[int] = None) -> np.ndarray:
        g = self.groups[gid]
        tables = [g.tables[r] for r in rids]
        w = max([len(t) for t in tables] + [1])
        if width is not None:
            if width < w:
                raise CacheError(f"block table needs {w} columns, only {width} given")
            w = width
        out = np.full((len(rids), w), -1, dtype=np.int32)
        for i, t in enumerate(tables):
            out[i, :len(t)] = t
        return out

    # -- accounting -------------------------------------------------------------------
    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def pages_needed_for(self, total_len: int) -> List[int]:
        return [g.pages_for_request(total_len) for g in self.groups]

    def check_invariants(self) -> None:
        """Every page is either free or in exactly one table; counts add up."""
        for g in self.groups:
            seen = {}
            for rid, table in g.tables.items():
                for p in table:
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheError(f"group {g.gid}: page {p} held by {seen[p]!r} and {rid!r}")
                    seen[p] = rid
            free = set(g.pool._free)
            if len(free) != len(g.pool._free):
                raise CacheError(f"group {g.gid}: a page is on the free list twice")
            if free & set(seen):
                raise CacheError(f"group {g.gid}: a held page is on the free list")
            if len(free) + len(seen) != g.pool.num_pages:
                raise CacheError(
                    f"group {g.gid}: {g.pool.num_pages - len(free) - len(seen)} pages lost")
        held_slots = sorted(rc.slot for rc in self.requests.values())
        if len(set(held_slots)) != len(held_slots):
            raise CacheError("a state slot is held twice")
        if len(held_slots) + self.slots.num_free != self.slots.num_slots:
            raise CacheError("a state slot was lost")

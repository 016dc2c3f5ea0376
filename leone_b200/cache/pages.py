"""Paged cache bookkeeping: pools of pages, block tables, fixed-size state slots.

This module decides *which page holds which tokens of which request*; it owns
no device memory (the engine allocates the pools this module describes).  The
bookkeeping itself is C++ (``csrc/host_runtime.cpp``, built into
``libleone_host.so`` on first use); the classes here are its Python front:
they map request names to the 64-bit ids the library uses, turn its return
codes into exceptions and give read-only views of its state.

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

import ctypes
from collections.abc import Mapping
from ctypes import byref, c_int, c_longlong, c_void_p
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np


class OutOfPages(RuntimeError):
    """Not enough free pages (or state slots) for what was asked."""


class CacheError(RuntimeError):
    """A call that breaks the manager's rules (unknown request, double free...)."""


_LIB = None


def host_library():
    """The C++ host runtime, compiled on first use."""
    global _LIB
    if _LIB is None:
        from ..csrc.build import ensure_built
        lib = ctypes.CDLL(ensure_built("host"))
        lib.leone_host_last_error.restype = ctypes.c_char_p
        lib.leone_freelist_create.restype = c_void_p
        lib.leone_cache_create.restype = c_void_p
        lib.leone_cache_first_live_block.restype = c_longlong
        lib.leone_pack_step_size.restype = c_longlong
        _LIB = lib
    return _LIB


def _check(code: int) -> None:
    if code == 0:
        return
    message = host_library().leone_host_last_error().decode()
    if code == 1:
        raise OutOfPages(message)
    raise CacheError(message)


def _ll(values) -> ctypes.Array:
    values = list(values)
    return (c_longlong * max(len(values), 1))(*values)


class _FreeList:
    def __init__(self, count: int):
        self._lib = host_library()
        self._h = c_void_p(self._lib.leone_freelist_create(int(count)))
        self._n = int(count)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.leone_freelist_destroy(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return int(self._lib.leone_freelist_num_free(self._h))

    def _take(self, count: int) -> List[int]:
        out = (c_int * max(count, 1))()
        _check(self._lib.leone_freelist_take(self._h, int(count), out))
        return list(out[:count])

    def _give_back(self, ids: Sequence[int]) -> None:
        ids = [int(i) for i in ids]
        _check(self._lib.leone_freelist_give_back(self._h, (c_int * max(len(ids), 1))(*ids), len(ids)))


class PagePool(_FreeList):
    """Free list over page ids ``0..num_pages-1``; LIFO so freed pages are reused at once."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        super().__init__(num_pages)
        self.num_pages = num_pages

    @property
    def num_held(self) -> int:
        return self.num_pages - self.num_free

    @property
    def high_water(self) -> int:
        return int(self._lib.leone_freelist_high_water(self._h))

    def take(self, count: int) -> List[int]:
        return self._take(count)

    def give_back(self, pages: Sequence[int]) -> None:
        self._give_back(pages)


class StateSlots(_FreeList):
    """Numbered fixed-size slots, one per live request."""

    def __init__(self, num_slots: int):
        super().__init__(num_slots)
        self.num_slots = num_slots

    def take(self) -> int:
        return self._take(1)[0]

    def give_back(self, slot: int) -> None:
        self._give_back([slot])


@dataclass
class GroupSpec:
    """What a group of layers needs from the cache."""
    kind: str                   # "full" or "window": when pages go back to the pool
    num_kv_heads: int
    head_dim: int               # elements of a cached key row
    window: Optional[int] = None
    layers: List[int] = field(default_factory=list)
    value_head_dim: Optional[int] = None    # elements of a cached value row (None: head_dim; 0: no values)
    dtype: object = None        # storage dtype of the pages (None: the engine's run dtype)
    tag: str = ""               # groups with different tags are never merged

    def key(self):
        return (self.kind, self.num_kv_heads, self.head_dim, self.window, self.value_head_dim, self.dtype, self.tag)

    def page_elements(self, page_tokens: int):
        """Elements of one page of one layer: (key pool, value pool)."""
        vd = self.head_dim if self.value_head_dim is None else self.value_head_dim
        return (self.num_kv_heads * page_tokens * self.head_dim, self.num_kv_heads * page_tokens * vd)


@dataclass(frozen=True)
class RequestCache:
    """A request's bookkeeping, as it was when it was asked for."""
    slot: int
    committed_len: int
    reserved_len: int
    fresh: bool                 # no step has been committed yet: state slot must be cleared
    version: int                # changes whenever a block table changes other than by growing at its end


class _PoolView:
    """The pool of one group, read-only."""

    def __init__(self, manager, gid):
        self._m, self._gid = manager, gid

    def _get(self, what):
        return int(self._m._lib.leone_cache_pool(self._m._h, self._gid, what))

    num_pages = property(lambda self: self._get(0))
    num_free = property(lambda self: self._get(1))
    num_held = property(lambda self: self._get(2))
    high_water = property(lambda self: self._get(3))


class _TablesView:
    """``tables[rid]``: the request's page per logical block (a copy); -1 where a window has passed."""

    def __init__(self, manager, gid):
        self._m, self._gid = manager, gid

    def __contains__(self, rid) -> bool:
        return rid in self._m._ids

    def __getitem__(self, rid) -> List[int]:
        m = self._m
        n = int(m._lib.leone_cache_table_len(m._h, self._gid, c_longlong(m._id(rid))))
        out = (c_int * max(n, 1))()
        _check(m._lib.leone_cache_table_copy(m._h, self._gid, c_longlong(m._id(rid)), 0, n, out))
        return list(out[:n])

    def tail(self, rid, start: int) -> List[int]:
        """Entries from ``start`` on (what a mirror of the table appends)."""
        m = self._m
        n = int(m._lib.leone_cache_table_len(m._h, self._gid, c_longlong(m._id(rid))))
        if start >= n:
            return []
        out = (c_int * (n - start))()
        _check(m._lib.leone_cache_table_copy(m._h, self._gid, c_longlong(m._id(rid)), start, n - start, out))
        return list(out)

    def length(self, rid) -> int:
        m = self._m
        return int(m._lib.leone_cache_table_len(m._h, self._gid, c_longlong(m._id(rid))))


class CacheGroup:
    def __init__(self, manager, gid: int, spec: GroupSpec, page_tokens: int):
        self.gid = gid
        self.spec = spec
        self.page_tokens = page_tokens
        self.pool = _PoolView(manager, gid)
        self.tables = _TablesView(manager, gid)
        self._m = manager

    def blocks_for(self, length: int) -> int:
        return -(-length // self.page_tokens)

    def first_live_block(self, committed_len: int) -> int:
        """First logical block that a query at position >= committed_len can still read."""
        return int(self._m._lib.leone_cache_first_live_block(self._m._h, self.gid, c_longlong(committed_len)))

    def pages_needed(self, table: List[int], new_len: int) -> int:
        return max(0, self.blocks_for(new_len) - len(table))

    def pages_for_request(self, total_len: int) -> int:
        """Upper bound of pages a request of ``total_len`` tokens holds at one time (for a window
        group the window's blocks plus one step's portion would do; without knowing the portion
        the bound is the full length)."""
        return self.blocks_for(total_len)


class _SlotsView:
    def __init__(self, manager):
        self._m = manager

    num_slots = property(lambda self: int(self._m._lib.leone_cache_slots(self._m._h, 0)))
    num_free = property(lambda self: int(self._m._lib.leone_cache_slots(self._m._h, 1)))


class _RequestsView(Mapping):
    def __init__(self, manager):
        self._m = manager

    def __getitem__(self, rid) -> RequestCache:
        if rid not in self._m._ids:
            raise KeyError(rid)
        get = self._m._get_field
        return RequestCache(slot=get(rid, 2), committed_len=get(rid, 0), reserved_len=get(rid, 1),
                            fresh=bool(get(rid, 3)), version=get(rid, 4))

    def __iter__(self):
        return iter(list(self._m._ids))

    def __len__(self) -> int:
        return len(self._m._ids)


class CacheManager:
    """Block tables and state slots of all live requests over all groups."""

    def __init__(self, group_specs: Sequence[GroupSpec], page_tokens: int, num_pages: int,
                 num_slots: int):
        for spec in group_specs:
            if spec.kind not in ("full", "window"):
                raise ValueError(f"unknown cache group kind '{spec.kind}'")
            if spec.kind == "window" and (spec.window is None or spec.window <= 0):
                raise ValueError("a window group needs a positive window")
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self._lib = host_library()
        n = len(group_specs)
        kinds = (c_int * max(n, 1))(*[1 if s.kind == "window" else 0 for s in group_specs])
        windows = _ll([int(s.window or 0) for s in group_specs])
        handle = self._lib.leone_cache_create(n, kinds, windows, int(page_tokens), int(num_pages), int(num_slots))
        if not handle:
            raise ValueError("the cache manager's sizes must be positive")
        self._h = c_void_p(handle)
        self.page_tokens = page_tokens
        self._ids: Dict[Hashable, int] = {}
        self._next_id = 1
        self.groups = [CacheGroup(self, i, s, page_tokens) for i, s in enumerate(group_specs)]
        self.slots = _SlotsView(self)
        self.requests = _RequestsView(self)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.leone_cache_destroy(self._h)
            self._h = None

    def _id(self, rid: Hashable) -> int:
        if rid not in self._ids:
            raise CacheError(f"request {rid!r} is not open")
        return self._ids[rid]

    def _get_field(self, rid: Hashable, what: int) -> int:
        value = c_longlong(0)
        _check(self._lib.leone_cache_get(self._h, c_longlong(self._id(rid)), what, byref(value)))
        return int(value.value)

    # -- lifetime -------------------------------------------------------------------
    def open(self, rid: Hashable) -> int:
        if rid in self._ids:
            raise CacheError(f"request {rid!r} is already open")
        slot = c_int(-1)
        _check(self._lib.leone_cache_open(self._h, c_longlong(self._next_id), byref(slot)))
        self._ids[rid] = self._next_id
        self._next_id += 1
        return int(slot.value)

    def close(self, rid: Hashable) -> None:
        _check(self._lib.leone_cache_close(self._h, c_longlong(self._id(rid))))
        del self._ids[rid]

    def is_open(self, rid: Hashable) -> bool:
        return rid in self._ids

    def length(self, rid: Hashable) -> int:
        return self._get_field(rid, 0)

    def slot(self, rid: Hashable) -> int:
        return self._get_field(rid, 2)

    def table_version(self, rid: Hashable) -> int:
        """A number that changes whenever one of the request's block tables changes other than
        by growing at its end (a mirror of the tables may then append instead of rewriting)."""
        return self._get_field(rid, 4)

    # -- the step transaction -------------------------------------------------------
    def _pairs(self, wants: Dict[Hashable, int]):
        rids = [self._id(r) for r in wants]
        return len(rids), _ll(rids), _ll(int(v) for v in wants.values())

    def can_reserve(self, wants: Dict[Hashable, int]) -> bool:
        """Would ``reserve`` succeed for these (request → new length) pairs together?"""
        return bool(self._lib.leone_cache_can_reserve(self._h, *self._pairs(wants)))

    def reserve(self, wants: Dict[Hashable, int]) -> None:
        """Take pages so each request can hold ``new_len`` tokens.  All or nothing."""
        _check(self._lib.leone_cache_reserve(self._h, *self._pairs(wants)))

    def commit(self, rid: Hashable, new_len: int) -> None:
        """The step that wrote tokens up to ``new_len`` succeeded."""
        _check(self._lib.leone_cache_commit(self._h, c_longlong(self._id(rid)), c_longlong(new_len)))

    def reserve_steps(self, rids: Sequence[Hashable], steps: int):
        """Pages for ``steps`` more tokens of every request, all or nothing, in one call.
        Returns ``(lengths, versions, slots, table_lens)``: each request's committed length,
        table version and slot, and ``table_lens[g][i]``, the length of its block table in
        group ``g`` after the reservation."""
        n = len(rids)
        lengths = np.empty(max(n, 1), dtype=np.int64)
        versions = np.empty(max(n, 1), dtype=np.int64)
        slots = np.empty(max(n, 1), dtype=np.int32)
        table_lens = np.empty((len(self.groups), max(n, 1)), dtype=np.int32)
        ll, ci = ctypes.POINTER(c_longlong), ctypes.POINTER(c_int)
        _check(self._lib.leone_cache_reserve_steps(
            self._h, n, _ll(self._id(r) for r in rids), c_longlong(int(steps)), lengths.ctypes.data_as(ll),
            versions.ctypes.data_as(ll), slots.ctypes.data_as(ci), table_lens.ctypes.data_as(ci)))
        return lengths[:n], versions[:n], slots[:n], table_lens[:, :n]

    def commit_many(self, rids: Sequence[Hashable], new_lens: Sequence[int]) -> None:
        _check(self._lib.leone_cache_commit_many(self._h, len(rids), _ll(self._id(r) for r in rids),
                                                 _ll(int(v) for v in new_lens)))

    def rollback(self, rid: Hashable) -> None:
        """The step failed: return pages beyond the committed length."""
        _check(self._lib.leone_cache_truncate(self._h, c_longlong(self._id(rid)), c_longlong(-1)))

    def truncate(self, rid: Hashable, length: int) -> None:
        """Drop everything past ``length`` tokens (crates/leone/src/kv.rs:929-950)."""
        if length < 0:
            raise CacheError(f"request {rid!r}: cannot truncate to a negative length")
        _check(self._lib.leone_cache_truncate(self._h, c_longlong(self._id(rid)), c_longlong(length)))

    # -- views for the step function --------------------------------------------------
    def block_table(self, gid: int, rids: Sequence[Hashable], width: Optional[int] = None) -> np.ndarray:
        ids = [self._id(r) for r in rids]
        if width is None:
            width = max([int(self._lib.leone_cache_table_len(self._h, gid, c_longlong(i))) for i in ids] + [1])
        out = np.empty((len(ids), width), dtype=np.int32)
        _check(self._lib.leone_cache_block_table(self._h, gid, len(ids), _ll(ids), int(width),
                                                 out.ctypes.data_as(ctypes.POINTER(c_int))))
        return out

    # -- accounting -------------------------------------------------------------------
    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def pages_needed_for(self, total_len: int) -> List[int]:
        return [g.pages_for_request(total_len) for g in self.groups]

    def check_invariants(self) -> None:
        """Every page is either free or in exactly one table; counts add up."""
        _check(self._lib.leone_cache_check_invariants(self._h))

"""The engine: a model, its cache and the one step function.

``Engine.step`` takes a batch of (request, its next tokens, wanted places) —
portions of prompts beside single decoded tokens, cut anywhere — runs exactly
those tokens as one flat batch against what earlier steps left in the cache,
and returns the fp32 logits at the wanted places.  The reference runs prompt
portions one request at a time and then one shared decode pass
(crates/leone-cli/src/server.rs:3667-3938, crates/leone/src/runtime.rs:7461);
here both kinds of rows go through the same kernels in the same launches.

The step is a transaction on the cache (crates/leone/src/kv.rs:326-347):
pages for every token of the step are taken before anything runs, lengths
advance only after the step succeeded, and a failure gives the pages back.
"""
from __future__ import annotations

import os
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.pages import CacheManager, GroupSpec, OutOfPages
from ..cache.slots import SlotRecords
from ..parts.base import FixedState, PagedCacheView, PagedKV, Runtime, StateView
from ..parts.spec import ModelSpec
from ..registry import config_from_folder, spec_from_config
from ..weights.loader import check_names_and_shapes, load_checkpoint, target_dtype
from .budget import check_memory_budget, plan_memory
from .batch import StepContext, StepEntry, pack_metadata
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


class StepError(RuntimeError):
    """A kernel reported a fault through the status word (bad token id, bad page, ...)."""


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}")
    return _DTYPES[dtype]


def default_ops(device, dtype):
    """The CUDA kernels.  There is no other product path: this raises without them."""
    from ..ops.cuda import CudaOps
    return CudaOps(device, dtype)


class Engine:
    def __init__(self, spec: ModelSpec, tensors: Optional[Dict[str, torch.Tensor]] = None, *,
                 dtype="bfloat16", device="cuda:0", page_tokens: int = 16,
                 max_tokens: Optional[int] = None, num_pages: Optional[int] = None,
                 max_requests: int = 64, max_batch_tokens: int = 2048, ops=None,
                 folder: Optional[str] = None, random_seed: Optional[int] = None, free_bytes=None):
        """``free_bytes``: a callable that says how many bytes the device has free, for the
        memory budget (default: the CUDA driver's figure plus what torch's allocator holds
        unused; no check on a device without such a figure)."""
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        self.spec = spec
        if ops is None:
            ops = default_ops(self.device, self.dtype)
        self.ops = ops
        self.rt = Runtime(self.device, self.dtype, ops, max_batch_tokens)
        self.max_batch_tokens = max_batch_tokens
        self.model = Model(spec, self.rt)
        specs = self.model.weight_specs()

        # -- what the cache will hold (nothing is allocated yet) ------------------------------
        self.page_tokens = page_tokens
        if num_pages is None:
            if max_tokens is None:
                max_tokens = max_requests * 256
            num_pages = -(-max_tokens // page_tokens)
        self.num_pages = num_pages
        self.max_requests = max_requests
        plan = self.model.cache_plan()
        group_specs: List[GroupSpec] = []
        self._run_group: Dict[int, tuple] = {}      # run position -> (gid, index within group)
        self._run_state: Dict[int, torch.Tensor] = {}
        self._run_source: Dict[int, int] = {}       # run position -> position whose cache it reads
        state_shapes: Dict[int, tuple] = {}
        for pos, (req, source) in enumerate(plan):
            if source is not None:
                self._run_source[pos] = source
            elif isinstance(req, PagedKV):
                # the part says what it caches (widths, dtype, when pages go back); equal requests share a group
                r = req.resolved(self.dtype)
                gs = GroupSpec(r.lifetime, r.num_kv_heads, r.head_dim, r.window, value_head_dim=r.value_head_dim,
                               dtype=r.dtype, tag=r.tag)
                for gid, existing in enumerate(group_specs):
                    if existing.key() == gs.key():
                        break
                else:
                    gid = len(group_specs)
                    group_specs.append(gs)
                self._run_group[pos] = (gid, len(group_specs[gid].layers))
                group_specs[gid].layers.append(pos)
            elif isinstance(req, FixedState):
                state_shapes[pos] = (max_requests,) + tuple(int(d) for d in req.shape)
            elif req is not None:
                raise TypeError(f"run position {pos}: unknown cache request {req!r}")

        # -- the memory budget, before anything is uploaded -----------------------------------
        stored = None
        if tensors is None and folder is not None:
            from ..weights.safetensors import Checkpoint
            probe = Checkpoint(folder)
            notes = self.model.load_notes(set(probe.names()))
            stored = {n: e.dtype for n, e in probe.entries.items()}
            probe.close()
        elif tensors is not None:
            stored = {n: t.dtype for n, t in tensors.items()}
        self.memory_plan = plan_memory(self.model, specs, stored, self.dtype, group_specs, num_pages, page_tokens,
                                       state_shapes, max_requests, max_batch_tokens)
        if tensors is not None:
            # tensors already on the device are not uploaded again
            by_name = {s.name: s for s in specs}
            resident = sum(t.numel() * t.element_size() for n, t in tensors.items()
                           if n in by_name and t.device == self.device
                           and t.dtype == target_dtype(by_name[n], t.dtype, self.dtype))
            self.memory_plan["weights"] -= resident
            self.memory_plan["required"] -= resident
        check_memory_budget(self.memory_plan, self.device, free_bytes)

        # -- weights ------------------------------------------------------------------------------
        if tensors is None and folder is not None:
            tensors = load_checkpoint(folder, specs, self.dtype, self.device, notes)
        elif tensors is None:
            if random_seed is None:
                raise ValueError("an engine needs a model folder, tensors or a random seed")
            tensors = self._random_on_device(specs, random_seed)
        else:
            check_names_and_shapes(specs, tensors, self.model.load_notes(set(tensors)))
            by_name = {s.name: s for s in specs}
            tensors = {n: t.to(target_dtype(by_name[n], t.dtype, self.dtype)).to(self.device).contiguous()
                       for n, t in tensors.items()}
        self.model.load(tensors)        # empties the dict as the parts take their tensors
        del tensors

        # -- cache ----------------------------------------------------------------------------------
        for pos, shape in state_shapes.items():
            self._run_state[pos] = torch.zeros(shape, dtype=torch.float32, device=self.device)
        self.cache = CacheManager(group_specs, page_tokens, num_pages, max_requests)
        self.pools = []
        for gs in group_specs:
            k_el, v_el = gs.page_elements(page_tokens)
            head = (len(gs.layers), num_pages, gs.num_kv_heads, page_tokens)
            k_pool = torch.zeros(head + (gs.head_dim,), dtype=gs.dtype, device=self.device)
            v_pool = torch.zeros(head + (v_el // (gs.num_kv_heads * page_tokens),), dtype=gs.dtype,
                                 device=self.device) if v_el else None
            self.pools.append((k_pool, v_pool))
        self.slot_records = SlotRecords(max_requests, self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        if hasattr(self.ops, "bind_status"):
            self.ops.bind_status(self.status)
        self._meta_dev = None
        self._meta_host = None
        self._meta_event = None
        self.steps_run = 0
        self._sampler = None
        self._decode_graphs = {}
        # batch sizes whose captured decode steps are kept (a scheduler whose requests finish one
        # by one passes through every size, and a capture costs far more than a step); what a
        # size holds is small, because the logits buffer is shared
        self.max_decode_graphs = max(64, max_requests)
        self._decode_logits = None
        # a decode step launched before the step before it was read (see decode_steps)
        self._ahead = None
        self.lookahead = os.environ.get("LEONE_NO_LOOKAHEAD", "0") != "1"

    # -- construction helpers -----------------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str, **kw) -> "Engine":
        config = config_from_folder(folder)
        return cls(spec_from_config(config), folder=folder, **kw)

    @classmethod
    def from_config(cls, config, seed: int = 0, **kw) -> "Engine":
        """Random weights drawn on the device; nothing is written to disk."""
        return cls(spec_from_config(config), random_seed=seed, **kw)

    def _random_on_device(self, specs, seed):
        """Every tensor drawn in place in its storage dtype: the values are a function of
        (seed, name, index), the same on the device as in a folder written on the host."""
        from ..weights.loader import target_dtype
        from ..weights.random_init import draw
        return {spec.name: draw(spec, seed, self.device, target_dtype(spec, torch.float32, self.dtype))
                for spec in specs}

    # -- request lifetime ---------------------------------------------------------------
    def open(self, rid: Hashable) -> int:
        """A new request: block tables in every group and one state slot, whose record and
        fixed-size state rows start at zero."""
        self.drop_lookahead()
        slot = self.cache.open(rid)
        self.slot_records.open(slot)
        for state in self._run_state.values():
            state[slot].zero_()
        return slot

    def close(self, rid: Hashable) -> None:
        """The request's pages and its slot (with its record) go back."""
        self.drop_lookahead()
        slot = self.cache.slot(rid)
        self.cache.close(rid)
        self.slot_records.close(slot)

    def length(self, rid: Hashable) -> int:
        return self.cache.length(rid)

    # -- the step -----------------------------------------------------------------------
    def _stage(self, packed: np.ndarray) -> torch.Tensor:
        n = packed.size
        if self._meta_dev is None or self._meta_dev.numel() < n:
            cap = max(4096, 2 * n)
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            if self.device.type == "cuda":
                self._meta_host = torch.empty(cap, dtype=torch.int32, pin_memory=True)
                self._meta_event = torch.cuda.Event()
            else:
                self._meta_host = torch.empty(cap, dtype=torch.int32)
        elif self._meta_event is not None:
            self._meta_event.synchronize()     # the last copy out of the staging buffer is done
        self._meta_host[:n].numpy()[:] = packed
        self._meta_dev[:n].copy_(self._meta_host[:n], non_blocking=True)
        if self._meta_event is not None:
            self._meta_event.record()
        return self._meta_dev

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        rids = [e.rid for e in entries]
        starts = [self.cache.length(r) for r in rids]
        slots = [self.cache.slot(r) for r in rids]
        tables = [self.cache.block_table(g.gid, rids) for g in self.cache.groups]
        packed, offsets, bt_offsets, stats = pack_metadata(
            [e.tokens for e in entries], starts, slots, [e.want for e in entries], tables)
        dev = self._stage(packed)
        ctx = StepContext()
        for name, (o, s) in offsets.items():
            setattr(ctx, name, dev[o:o + s])
        ctx.block_tables = [dev[o:o + shape[0] * shape[1]].view(shape) for o, shape in bt_offsets]
        ctx.n_tokens, ctx.n_seqs, ctx.n_logit_rows = stats["n"], stats["b"], stats["m"]
        ctx.q_lens, ctx.starts, ctx.ctx_lens = stats["q_lens"], stats["starts"], stats["ctx_lens"]
        ctx.max_q_len, ctx.max_ctx_len = stats["max_q_len"], stats["max_ctx_len"]
        ctx.decode_only = stats["max_q_len"] == 1
        ctx.status = self.status
        self._attach_caches(ctx)
        return ctx

    def _attach_caches(self, ctx: StepContext) -> None:
        for pos in range(len(self.spec.run_order)):
            src = self._run_source.get(pos, pos)
            writes = pos not in self._run_source
            if src in self._run_group:
                gid, k = self._run_group[src]
                kp, vp = self.pools[gid]
                ctx.layer_caches[pos] = PagedCacheView(kp[k], None if vp is None else vp[k], ctx.block_tables[gid],
                                                       self.page_tokens, writes)
            elif src in self._run_state:
                ctx.layer_caches[pos] = StateView(self._run_state[src], writes)

    def step(self, entries: Sequence, check: bool = True) -> Optional[torch.Tensor]:
        """Run one batch.  ``entries``: ``StepEntry`` or ``(rid, tokens, want)`` tuples.

        Returns fp32 logits ``[wanted, vocab]`` in the order of the entries and of each
        entry's ``want`` (``None`` if nothing is wanted).  Raises :class:`OutOfPages`
        without changing anything if the pool cannot hold the step's tokens.
        """
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries:
            return None
        self.drop_lookahead()
        seen = set()
        total = 0
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.rid!r}: a step entry needs at least one token")
            ids = np.asarray(e.tokens, dtype=np.int64)
            if ids.size and (int(ids.min()) < 0 or int(ids.max()) >= self.spec.vocab_size):
                bad = [int(t) for t in ids[(ids < 0) | (ids >= self.spec.vocab_size)][:8]]
                raise ValueError(f"request {e.rid!r}: token ids {bad} are outside the "
                                 f"vocabulary of {self.spec.vocab_size}")
            total += len(e.tokens)
        if total > self.rt.max_tokens:
            raise ValueError(f"step has {total} tokens; this engine was built for at most "
                             f"{self.rt.max_tokens} per step")
        opened = []
        try:
            for e in entries:
                if not self.cache.is_open(e.rid):
                    self.open(e.rid)
                    opened.append(e.rid)
            wants = {}
            for e in entries:
                new_len = self.cache.length(e.rid) + len(e.tokens)
                if new_len > self.spec.max_positions:
                    raise ValueError(f"request {e.rid!r}: {new_len} tokens exceed the model's "
                                     f"{self.spec.max_positions} positions")
                wants[e.rid] = new_len
            self.cache.reserve(wants)
        except Exception:
            for rid in opened:
                self.cache.close(rid)
            raise
        saved = None
        try:
            if self._run_state:
                # fixed-size state is overwritten in place: keep the step's slots as they were,
                # so that a failed step leaves them (like the pages) as it found them
                rows = torch.tensor([self.cache.slot(e.rid) for e in entries], dtype=torch.long, device=self.device)
                saved = (rows, {pos: st.index_select(0, rows) for pos, st in self._run_state.items()})
            ctx = self.build_context(entries)
            logits = self.model.forward(ctx)
            if check:
                self.check_status()
        except Exception:
            if saved is not None:
                for pos, rows_before in saved[1].items():
                    self._run_state[pos].index_copy_(0, saved[0], rows_before)
            for e in entries:
                self.cache.rollback(e.rid)
            for rid in opened:
                self.cache.close(rid)
            raise
        for e in entries:
            self.cache.commit(e.rid, wants[e.rid])
        self.steps_run += 1
        return logits

    def sample(self, logits: torch.Tensor, params, positions, histories=None, states=None) -> List[int]:
        """One token per logits row (greedy, temperature, truncation stages; penalties if the
        rows' token histories are given, Mirostat if their sampler states are); returns host ints."""
        if self._sampler is None:
            from ..sampling.sampler import Sampler
            self._sampler = Sampler(self.ops, self.device)
        ids = self._sampler.sample(logits, params, positions, histories, states).tolist()
        if any(t < 0 for t in ids):
            raise ValueError("every logit of a row is non-finite, so no token can be sampled")
        return ids

    # -- decode quanta ------------------------------------------------------------------
    def decode_steps(self, rids: Sequence[Hashable], last_tokens: Sequence[int], params,
                     steps: int, use_graph: bool = True, expect_more: bool = True):
        """Decode ``steps`` tokens for every request in ``rids``: feed ``last_tokens`` at each
        request's current length, sample, feed the sample, and so on.  Returns the sampled ids
        as ``[steps][len(rids)]`` host ints.  Pages for all ``steps`` positions are taken first
        (:class:`OutOfPages` leaves everything as it was); lengths advance by ``steps``.
        ``expect_more``: the caller expects to ask for the step after this one with the same
        requests, so a single step may launch it before this one's ids are read
        (:meth:`_decode_one_ahead`); say False when a request ends with this step, or the
        step launched ahead is wasted GPU time before whatever comes next.
        """
        rids = list(rids)
        if steps <= 0 or not rids:
            return []
        # A step launched ahead and then dropped has run its kernels.  Pages it wrote are given
        # back and rewritten, but fixed-size state would have been advanced by a token for good,
        # and a window group would have released pages: such models decode without looking ahead.
        if (steps == 1 and use_graph and self.lookahead and self.device.type == "cuda"
                and not self._run_state and all(g.spec.kind == "full" for g in self.cache.groups)):
            return [self._decode_one_ahead(rids, [int(t) for t in last_tokens], list(params), expect_more)]
        self.drop_lookahead()
        if not (use_graph and self.device.type == "cuda") or steps > 64:
            if max(self.cache.length(r) for r in rids) + steps > self.spec.max_positions:
                raise ValueError("decode_steps would run past the model's positions")
            out = []
            toks = list(last_tokens)
            for _ in range(steps):
                logits = self.step([(r, [t], [0]) for r, t in zip(rids, toks)])
                toks = self.sample(logits, params, [self.cache.length(r) - 1 for r in rids])
                out.append(toks)
            return out
        # one call: pages for all the steps, and what the graph's buffers need to know
        lengths, versions, slots, table_lens = self.cache.reserve_steps(rids, steps)
        try:
            if int(lengths.max()) + steps > self.spec.max_positions:
                raise ValueError("decode_steps would run past the model's positions")
            state = dict(versions=versions, slots=slots, table_lens=table_lens)
            graph = self._decode_graph(rids, last_tokens, lengths, params, state, steps)
            graph.fill(rids, last_tokens, lengths, params, **state)
            tokens = graph.run(steps)       # also reads and checks the status word
        except Exception:
            for r in rids:
                self.cache.rollback(r)
            raise
        self.cache.commit_many(rids, lengths + steps)
        self.steps_run += steps
        return tokens.tolist()

    def decode_logits(self, rids: Sequence[Hashable], last_tokens: Sequence[int]) -> torch.Tensor:
        """One decode step of ``rids`` from the captured graph, for a caller that samples itself:
        returns the fp32 logits ``[len(rids), vocab]`` (the graph's own buffer, valid until the
        next decode step); lengths advance by one.  The graph's built-in greedy draw is ignored."""
        from ..sampling.sampler import SamplingParams
        rids = list(rids)
        self.drop_lookahead()
        if self.device.type != "cuda":
            return self.step([(r, [int(t)], [0]) for r, t in zip(rids, last_tokens)])
        params = [SamplingParams() for _ in rids]
        lengths, versions, slots, table_lens = self.cache.reserve_steps(rids, 1)
        try:
            if int(lengths.max()) + 1 > self.spec.max_positions:
                raise ValueError("decode_logits would run past the model's positions")
            state = dict(versions=versions, slots=slots, table_lens=table_lens)
            graph = self._decode_graph(rids, last_tokens, lengths, params, state)
            graph.fill(rids, last_tokens, lengths, params, **state)
            graph.run(1)                    # reads and checks the status word
        except Exception:
            for r in rids:
                self.cache.rollback(r)
            raise
        self.cache.commit_many(rids, lengths + 1)
        self.steps_run += 1
        return graph.logits

    def decode_logits_buffer(self) -> torch.Tensor:
        """fp32 ``[max_requests, vocab]``: the logits of a captured decode step of any batch size
        (its first ``batch`` rows), valid until the next decode step."""
        if self._decode_logits is None:
            self._decode_logits = torch.empty((self.max_requests, self.spec.vocab_size), dtype=torch.float32,
                                              device=self.device)
        return self._decode_logits

    def _decode_graph(self, rids, last_tokens, lengths, params, state, steps: int = 1):
        """The captured decode step for this batch size and for the context bucket that holds
        the longest sequence after ``steps`` more tokens, captured now if it is not yet.  One
        set of (small) buffers per batch size, one logits buffer for all; the least recently used
        batch size is dropped beyond ``max_decode_graphs`` of them."""
        graph = self._decode_graphs.pop(len(rids), None)
        if graph is None:
            from .decode_graph import DecodeGraph
            graph = DecodeGraph(self, len(rids))
        self._decode_graphs[len(rids)] = graph                 # most recently used last
        while len(self._decode_graphs) > self.max_decode_graphs:
            self._decode_graphs.pop(next(iter(self._decode_graphs)))
        bucket = graph.bucket_for(int(max(lengths)) + steps)
        if not graph.select(bucket):
            # capture needs valid tables: fill first, then warm up and capture on them
            graph.fill(rids, last_tokens, lengths, params, **state)
            graph.capture(bucket)
        return graph

    def _decode_one_ahead(self, rids: List[Hashable], last_tokens: List[int], params,
                          expect_more: bool = True) -> List[int]:
        """One decode step of ``rids``, with the step after it launched before this one's ids
        are read: the sampled ids are fed back on the device, so the next step needs nothing
        from the host but the pages it may write (reserved here, given back if the next call
        is not the expected one).  The next call finds its step already running if it names
        the same requests and feeds the ids this call returns; anything else the engine is
        asked to do in between (another step, opening or closing a request) drops it."""
        a, self._ahead = self._ahead, None
        if a is not None and a["rids"] == rids and a["feeds"] == last_tokens and a["params"] == params:
            graph, lengths, slot, event = a["graph"], a["lengths"], a["slot"], a["event"]
        else:
            self._ahead = a
            self.drop_lookahead()
            lengths, versions, slots, table_lens = self.cache.reserve_steps(rids, 1)
            try:
                if int(lengths.max()) + 1 > self.spec.max_positions:
                    raise ValueError("decode_steps would run past the model's positions")
                state = dict(versions=versions, slots=slots, table_lens=table_lens)
                graph = self._decode_graph(rids, last_tokens, lengths, params, state)
                graph.fill(rids, last_tokens, lengths, params, **state)
                slot, event = 0, graph.launch(0)
            except Exception:
                for r in rids:
                    self.cache.rollback(r)
                raise
        try:
            ahead = None
            # the step after this one must fit the captured step's context bucket (a new bucket
            # is captured by the next call, with nothing in flight)
            if (expect_more and slot + 1 < graph.max_quantum
                    and int(lengths.max()) + 2 <= min(self.spec.max_positions, graph.bucket)):
                try:
                    table_lens = self.cache.reserve_steps(rids, 2)[3]      # this step's token and the next one's
                except OutOfPages:
                    pass                                                   # the next call decides what gives way
                else:
                    graph.advance_from_host(rids, lengths + 1, table_lens, slot + 1)
                    ahead = dict(rids=rids, params=params, graph=graph, lengths=lengths + 1, slot=slot + 1,
                                 event=graph.launch(slot + 1))
            tokens = graph.collect(slot, event)
        except Exception:
            for r in rids:
                self.cache.rollback(r)
            raise
        self.cache.commit_many(rids, lengths + 1)
        if ahead is not None:
            ahead["feeds"] = tokens
            self._ahead = ahead
        self.steps_run += 1
        return tokens

    def drop_lookahead(self) -> None:
        """Forget a decode step that was launched ahead: what it reserved goes back.  Its kernels
        may still be running; whatever is launched next is ordered behind them on the stream."""
        a, self._ahead = self._ahead, None
        if a is not None:
            for r in a["rids"]:
                if self.cache.is_open(r):
                    self.cache.rollback(r)

    def check_status(self) -> None:
        word = self.status.tolist()
        if word[0] != 0:
            self.status.zero_()
            raise StepError(f"kernel status {word[0]:#x} (detail {word[1]}, {word[2]}, {word[3]}): "
                            + self.ops.describe_status(word[0]))

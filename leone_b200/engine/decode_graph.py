"""Decode steps replayed from a CUDA graph, with sampled tokens fed back on the device.

For a fixed set of B decoding requests the whole step — embedding, every layer, final norm,
output head, sampling, and the kernel that turns the sampled ids into the next step's inputs —
is captured once and replayed.  Everything that changes between steps (token ids, positions,
lengths, block tables, sampling positions) lives in device buffers that the captured kernels
read, so one captured step serves every context length up to the one it was captured for.
The reference captures its single-request decode chain the same way and keeps the position in a
device word (crates/leone/src/runtime.rs:7107-7291, crates/leone/src/backend.rs:1586-1595); it
re-captures when the context bucket changes (next power of two, at least 512:
crates/leone/src/backend.rs:1616, crates/leone/src/runtime.rs:5005-5009).  Here too a step is
captured per *context bucket* (same rule, capped by the model's positions): what is fixed at
capture is how the kernels are launched (how many ways the attention splits a sequence's keys),
and that is chosen for the bucket, not for the model's limit.  All buckets of a batch size share
one set of buffers.

A *quantum* of up to ``max_quantum`` steps runs without the host: pages for the whole quantum
are reserved and written into the block tables first, and the sampled ids of all its steps are
read back once (the reference's service quantum is 4 tokens, crates/leone-cli/src/server.rs:6190-6203).
"""
from __future__ import annotations

import gc
import weakref
from typing import Hashable, List, Sequence

import numpy as np
import torch

from .batch import StepContext, pack_metadata


class DecodeGraph:
    def __init__(self, engine, batch: int, max_quantum: int = 64):
        self.engine = weakref.proxy(engine)     # the engine owns this object: no reference cycle
        self.batch = batch
        self.max_quantum = max_quantum
        dev = engine.device
        self.widths = [-(-engine.spec.max_positions // engine.page_tokens) for _ in engine.cache.groups]
        tables = [np.full((batch, w), -1, dtype=np.int32) for w in self.widths]
        packed, self.offsets, self.bt_offsets, _ = pack_metadata(
            [[0]] * batch, [0] * batch, [0] * batch, [[0]] * batch, tables)
        self.size = packed.size
        self.meta = torch.zeros(self.size, dtype=torch.int32, device=dev)
        self.meta_host = torch.zeros(self.size, dtype=torch.int32, pin_memory=True)
        self.sampled = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.history = torch.zeros((max_quantum, batch), dtype=torch.int32, device=dev)
        self.history_host = torch.zeros((max_quantum, batch), dtype=torch.int32, pin_memory=True)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status_host = torch.zeros(4, dtype=torch.int32, pin_memory=True)
        self.logits = engine.decode_logits_buffer()[:batch]      # one buffer for every batch size
        self.ctx = self._context()
        self.graphs = {}                   # context bucket -> captured step
        self.graph = None                  # the selected bucket's
        self.bucket = None
        self._filled_rids = None           # what fill() last wrote into the host copy
        self._filled_pages = [[0] * batch for _ in engine.cache.groups]
        self._tables_at = min((o for o, _ in self.bt_offsets), default=None)   # where the block tables start
        self._events = [torch.cuda.Event(), torch.cuda.Event()]
        self._advance_host = [torch.zeros((2, batch), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.launches_per_step = 0
        self.stream = torch.cuda.Stream(device=dev)

    def bucket_for(self, longest: int) -> int:
        """The context bucket of a step whose longest sequence holds ``longest`` tokens after it:
        the next power of two, at least 512, at most the model's positions."""
        limit = self.engine.spec.max_positions
        bucket = 512
        while bucket < longest:
            bucket *= 2
        return min(bucket, limit)

    def select(self, bucket: int) -> bool:
        """Make ``bucket``'s captured step the one that is replayed; False if there is none yet."""
        graph = self.graphs.get(bucket)
        if graph is None:
            return False
        self.graph, self.bucket = graph, bucket
        return True

    def _view(self, name):
        o, s = self.offsets[name]
        return self.meta[o:o + s]

    def _context(self) -> StepContext:
        e = self.engine
        ctx = StepContext()
        for name in self.offsets:
            setattr(ctx, name, self._view(name))
        ctx.block_tables = [self.meta[o:o + shape[0] * shape[1]].view(shape) for o, shape in self.bt_offsets]
        ctx.n_tokens = ctx.n_seqs = ctx.n_logit_rows = self.batch
        ctx.max_q_len = 1
        ctx.max_ctx_len = e.spec.max_positions
        ctx.decode_only = True
        ctx.fixed_shapes = True
        ctx.status = e.status
        ctx.logits_out = self.logits
        e._attach_caches(ctx)
        return ctx

    def _one_step(self):
        e = self.engine
        b = self.batch
        logits = e.model.forward(self.ctx)
        # temperature, seed and position of every row come from its request's slot record, which
        # the advance kernel moves on by a token, like the step's own positions and lengths
        records = e.slot_records.on_device
        e.ops.sample_slots(logits, self.ctx.slot_ids, records, self.sampled)
        e.ops.decode_advance(self.ctx.token_ids, self.ctx.positions, self.ctx.ctx_len, None, self.sampled,
                             self.history, self.counter, slot_ids=self.ctx.slot_ids, records=records)

    def fill(self, rids: Sequence[Hashable], last_tokens: Sequence[int], lengths: Sequence[int], params,
             versions=None, slots=None, table_lens=None):
        """Host → device: this quantum's starting state.  The pinned host copy keeps what the
        last call wrote, so for the same requests in the same rows only what changed is
        rewritten: tokens, lengths, and the block-table entries of pages taken since.
        ``versions``, ``slots`` and ``table_lens`` (``[group][request]``) are what
        ``CacheManager.reserve_steps`` returned; without them the cache is asked."""
        e = self.engine
        b = self.batch
        host = self.meta_host.numpy()

        def put(name, values):
            o, s_ = self.offsets[name]
            host[o:o + s_] = values

        lengths = np.asarray(lengths, dtype=np.int32)
        put("token_ids", np.asarray(last_tokens, dtype=np.int32))
        put("positions", lengths)
        put("ctx_len", lengths + 1)
        if versions is None:
            versions = [e.cache.table_version(r) for r in rids]
        key = (tuple(rids), tuple(int(v) for v in versions))
        same = key == self._filled_rids
        if not same:
            put("seq_of_token", np.arange(b, dtype=np.int32))
            put("q_start", np.arange(b + 1, dtype=np.int32))
            put("slot_ids", np.asarray(slots if slots is not None else [e.cache.slot(r) for r in rids],
                                       dtype=np.int32))
            put("logit_rows", np.arange(b, dtype=np.int32))
        appended = []                       # [lo, hi) ranges of the host copy that gained entries
        for gi, (g, w, (o, shape)) in enumerate(zip(e.cache.groups, self.widths, self.bt_offsets)):
            view = host[o:o + shape[0] * shape[1]].reshape(shape)
            windowed = g.spec.kind == "window"
            if windowed:
                same = False                # a window's table also loses entries at its front: rewrite
            for i, r in enumerate(rids):
                n = int(table_lens[gi][i]) if table_lens is not None else g.tables.length(r)
                if n > w:
                    raise ValueError(f"block table needs {n} columns, only {w} given")
                done = 0 if (not same or windowed) else self._filled_pages[gi][i]
                if done == 0:
                    view[i, :] = -1
                if n > done:
                    view[i, done:n] = g.tables.tail(r, done)
                    appended.append((o + i * shape[1] + done, o + i * shape[1] + n))
                self._filled_pages[gi][i] = n
        self._filled_rids = key
        # the requests' slot records: sampling parameters, and where each stands (the position
        # of the token being fed is the position that is sampled at)
        records = e.slot_records
        row_slots = slots if slots is not None else [e.cache.slot(r) for r in rids]
        for slot, p, length, tok in zip(row_slots, params, lengths, last_tokens):
            records.set_sampling(int(slot), p.seed, p.temperature)
            records.set_progress(int(slot), int(length), int(length), int(tok))
        records.sync()
        if same and self._tables_at is not None:
            # same requests in the same rows: the per-token and per-sequence vectors, and the
            # block-table entries that were appended
            self.meta[:self._tables_at].copy_(self.meta_host[:self._tables_at], non_blocking=True)
            for lo, hi in appended:
                self.meta[lo:hi].copy_(self.meta_host[lo:hi], non_blocking=True)
        else:
            self.meta.copy_(self.meta_host, non_blocking=True)
        self.counter.zero_()

    def capture(self, bucket: int):
        """Run one step eagerly on the filled buffers (so every scratch buffer exists), then
        capture one step for contexts of up to ``bucket`` tokens and select it.  The caller fills
        the buffers again afterwards: the eager step has advanced them."""
        self.ctx.max_ctx_len = bucket
        cur = torch.cuda.current_stream(self.engine.device)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            # The eager step really runs.  What it writes into pages and into the step's own
            # buffers is written again by the first replayed step, but fixed-size state would
            # be advanced by a token for good: keep it and put it back.
            kept = {pos: state.clone() for pos, state in self.engine._run_state.items()}
            self._one_step()
            for pos, state in kept.items():
                self.engine._run_state[pos].copy_(state)
            self.stream.synchronize()
            before = self.engine.ops.launches
            self.graph = self.graphs[bucket] = torch.cuda.CUDAGraph()
            self.bucket = bucket
            # an object that the collector finalises in the middle of a capture (an older
            # graph, a freed pool) would invalidate the capture: keep the collector out
            was_enabled = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(self.graph, stream=self.stream, capture_error_mode="thread_local"):
                    self._one_step()
            finally:
                if was_enabled:
                    gc.enable()
            self.launches_per_step = self.engine.ops.launches - before
        cur.wait_stream(self.stream)
        self.counter.zero_()

    def advance_from_host(self, rids: Sequence[Hashable], lengths, table_lens, slot: int) -> None:
        """Inputs of a step that is launched before the step before it has been read: the host's
        own record of every request's position and length (the cache manager's; the device has
        advanced its copy to the same values) and the block-table entries of pages taken since
        the last :meth:`fill`.  The token ids are where the device put them.  The pinned staging
        rows alternate with ``slot``, so a row is rewritten only after the step that read it
        has been waited for."""
        e = self.engine
        b = self.batch
        stage = self._advance_host[slot & 1]
        stage[0].numpy()[:] = lengths                    # position of the token being fed
        stage[1].numpy()[:] = lengths + 1                # the sequence's length after the step
        self._view("positions").copy_(stage[0], non_blocking=True)
        self._view("ctx_len").copy_(stage[1], non_blocking=True)
        host = self.meta_host.numpy()
        for gi, (g, w, (o, shape)) in enumerate(zip(e.cache.groups, self.widths, self.bt_offsets)):
            for i, r in enumerate(rids):
                n, done = int(table_lens[gi][i]), self._filled_pages[gi][i]
                if n > w:
                    raise ValueError(f"block table needs {n} columns, only {w} given")
                if n > done:
                    # entries past `done` are read by no copy in flight: only this step needs them
                    at = o + i * shape[1]
                    host[at + done:at + n] = g.tables.tail(r, done)
                    self.meta[at + done:at + n].copy_(self.meta_host[at + done:at + n], non_blocking=True)
                    self._filled_pages[gi][i] = n

    def launch(self, slot: int) -> torch.cuda.Event:
        """Enqueue one step, whose sampled ids go to row ``slot`` of the history, and their
        read-back; returns the event that says the ids are on the host."""
        self.graph.replay()
        self.history_host[slot].copy_(self.history[slot], non_blocking=True)
        self.status_host.copy_(self.engine.status, non_blocking=True)
        event = self._events[slot & 1]
        event.record()
        return event

    def collect(self, slot: int, event: torch.cuda.Event) -> List[int]:
        """Wait for a launched step and return its sampled ids."""
        event.synchronize()
        if int(self.status_host[0]) != 0:
            self.engine.check_status()
        return self.history_host[slot].tolist()

    def run(self, steps: int) -> np.ndarray:
        """Replay ``steps`` steps and read the sampled ids back: int32 [steps, batch]."""
        for _ in range(steps):
            self.graph.replay()
        self.history_host[:steps].copy_(self.history[:steps], non_blocking=True)
        self.status_host.copy_(self.engine.status, non_blocking=True)
        torch.cuda.current_stream(self.engine.device).synchronize()
        if int(self.status_host[0]) != 0:
            self.engine.check_status()
        return self.history_host[:steps].numpy().copy()

"""The scheduler: admits requests, cuts prompts into portions, decodes, finishes and frees.

The decisions are C++ (``csrc/host_runtime.cpp``, ``leone_sched_*``): who is admitted, what
the next step holds, when a request ends, whom to preempt.  This module is their front: it
keeps the token ids, opens and closes requests in the engine as the planner decides, runs the
step function and the sampler, and mirrors each request's progress in a :class:`Request`.

Each call of :meth:`Scheduler.step` builds one batch for the engine's step function: one token
for every request that is decoding, then portions of waiting prompts in arrival order until
the token budget is used (``max_batch_tokens`` for the whole step, ``prefill_chunk_tokens``
per request).  With ``prefill_first`` decode rows are held back while any running request
still has prompt left, so requests that start together also decode together (larger decode
batches; the choice for offline generation).  The reference dispatches per request with a
token budget of ``min(remaining_prefill, prefill_chunk_tokens)`` or a decode quantum
(crates/leone/src/scheduler.rs:341-378) and runs prompt portions and decode rows in separate
passes; here they share one batch.

What happens when pages run out is a policy:

``reserve`` (default, the reference's own): a request is admitted only if pages for
    its whole life, ``ceil((prompt + max_new_tokens - 1) / page_tokens)``, can be set
    aside (crates/leone/src/scheduler.rs:652-667), so a running request can never run
    out; a request that does not fit waits in the queue.
``optimistic``: a request starts as soon as its next portion fits.  If a step cannot get
    its pages, the youngest running request is preempted: its pages are freed and it goes
    back to the front of the queue with what it has generated appended to its prompt, to
    be recomputed.  Sampling is keyed by (seed, position), so its tokens do not change.

Counting follows the reference: ``max_new_tokens`` counts emitted tokens including the
one sampled from the prompt, so N new tokens need the cache for P + N - 1 positions
(crates/leone/src/runtime.rs:3602-3607).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence

from ..cache.pages import OutOfPages, host_library
from ..sampling.sampler import SamplerState, SamplingParams

_REJECTS = {1: "duplicate", 2: "empty_prompt", 3: "output_limit", 4: "token_id", 5: "prompt_limit",
            6: "kv_capacity", 7: "queue_limit"}
_FINISH = {1: "eos", 2: "length", 3: "max_positions"}


class AdmissionError(ValueError):
    """A request that can never run; ``reason`` names why
    (the reference's ``AdmissionReject``, crates/leone/src/scheduler.rs:101-110)."""

    def __init__(self, reason: str, message: str):
        super().__init__(message)
        self.reason = reason


@dataclass
class SchedulerConfig:
    max_running: int = 64
    max_waiting: int = 1024
    max_batch_tokens: int = 2048
    prefill_chunk_tokens: int = 2048
    policy: str = "reserve"            # or "optimistic"
    decode_quantum: int = 1            # decode steps run without the host when only decoding
    prefill_first: bool = False        # True: no decode rows while a running request has prompt left
    use_graphs: bool = True            # replay decode-only steps from a CUDA graph

    def __post_init__(self):
        if self.policy not in ("reserve", "optimistic"):
            raise ValueError(f"unknown page policy '{self.policy}'")
        if min(self.max_running, self.max_batch_tokens, self.prefill_chunk_tokens) <= 0:
            raise ValueError("scheduler limits must be positive")


@dataclass
class Request:
    """A request as the caller sees it; the planner's counts are mirrored here after every call."""
    rid: Hashable
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    eos_token_id: Optional[int] = None                   # as given (an id, several, or None)
    stop_ids: tuple = ()                                 # every id that ends the request
    arrival: int = 0
    tokens: List[int] = field(default_factory=list)      # prompt + generated, what the cache must hold
    computed: int = 0                                    # tokens already in the cache
    generated: List[int] = field(default_factory=list)
    state: str = "waiting"                               # waiting | running | finished | cancelled
    finish_reason: Optional[str] = None
    reserved_pages: int = 0
    preemptions: int = 0
    cancel_requested: bool = False
    key: int = 0                                         # the planner's name for this request
    slot: Optional[int] = None                           # its state slot while it runs
    sampler_state: Optional[SamplerState] = None         # what the sampler remembers between tokens

    @property
    def remaining_new(self) -> int:
        return self.max_new_tokens - len(self.generated)


@dataclass
class StepOutput:
    rid: Hashable
    token: int
    finished: bool
    finish_reason: Optional[str] = None


class Scheduler:
    """Works on anything with the engine's interface: ``cache`` (a CacheManager), ``spec``
    (``vocab_size``, ``max_positions``), ``step(entries)``, ``open``, ``close`` and
    ``sample(logits, params, positions) -> list of ids``."""

    def __init__(self, engine, config: Optional[SchedulerConfig] = None):
        self.engine = engine
        self.config = cfg = config or SchedulerConfig()
        self._lib = lib = host_library()
        lib.leone_sched_create.restype = c_void_p
        for name in ("leone_sched_oldest_running", "leone_sched_decode_quantum", "leone_sched_get",
                     "leone_sched_count"):
            getattr(lib, name).restype = c_longlong
        cache_handle = getattr(engine.cache, "_h", None)
        self._h = c_void_p(lib.leone_sched_create(
            cache_handle, c_longlong(cfg.max_running), c_longlong(cfg.max_waiting),
            c_longlong(cfg.max_batch_tokens), c_longlong(cfg.prefill_chunk_tokens),
            0 if cfg.policy == "reserve" else 1, int(cfg.prefill_first), c_longlong(engine.spec.vocab_size),
            c_longlong(engine.spec.max_positions)))
        if not self._h:
            raise ValueError("scheduler limits must be positive")
        lib.leone_sched_set_decode_quantum(self._h, c_longlong(max(1, cfg.decode_quantum)))
        self.requests: Dict[Hashable, Request] = {}
        self._by_key: Dict[int, Request] = {}
        self._next_key = 1
        self._cap = cfg.max_running + 8
        self._buf = [(c_longlong * self._cap)() for _ in range(3)]
        self._steps = self._prefill_tokens = self._decode_tokens = self._max_batch_tokens_seen = 0

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.leone_sched_destroy(self._h)
            self._h = None

    # -- views -------------------------------------------------------------------------
    def _count(self, what: int) -> int:
        return int(self._lib.leone_sched_count(self._h, what))

    def _listed(self, which: int) -> List[Request]:
        n = max(self._count(which), 1)
        out = (c_longlong * n)()
        n = self._lib.leone_sched_list(self._h, which, out, n)
        return [self._by_key[k] for k in out[:n]]

    @property
    def waiting(self) -> List[Request]:
        return self._listed(0)

    @property
    def running(self) -> List[Request]:
        return self._listed(1)

    @property
    def stats(self) -> dict:
        return dict(steps=self._steps, prefill_tokens=self._prefill_tokens, decode_tokens=self._decode_tokens,
                    preemptions=self._count(5), admitted=self._count(2), finished=self._count(3),
                    cancelled=self._count(4), max_batch_tokens_seen=self._max_batch_tokens_seen)

    def forget(self, rid: Hashable) -> Optional[Request]:
        """Drop a finished or cancelled request from the scheduler's records (a long-lived
        scheduler would otherwise keep every request it ever saw).  Returns it, or None if it is
        unknown or still in flight."""
        req = self.requests.get(rid)
        if req is None or not self._lib.leone_sched_forget(self._h, c_longlong(req.key)):
            return None
        del self.requests[rid]
        del self._by_key[req.key]
        return req

    def has_work(self) -> bool:
        return self._count(0) + self._count(1) > 0

    # -- admission --------------------------------------------------------------------
    def add_request(self, rid: Hashable, prompt: Sequence[int], max_new_tokens: int,
                    sampling: Optional[SamplingParams] = None, eos_token_id=None) -> Request:
        """``eos_token_id``: one id or several (a list or tuple); sampling any of them ends the
        request (the reference stops on its tokenizer's end id, crates/leone/src/runtime.rs:5383)."""
        prompt = [int(t) for t in prompt]
        if eos_token_id is None:
            stop_ids = ()
        elif isinstance(eos_token_id, (list, tuple, set, frozenset)):
            stop_ids = tuple(int(t) for t in eos_token_id)
        else:
            stop_ids = (int(eos_token_id),)
        old = self.requests.get(rid)
        if old is not None and old.state in ("waiting", "running"):
            raise AdmissionError("duplicate", f"request id {rid!r} is already in flight")
        key = self._next_key
        ids = (c_longlong * max(len(prompt), 1))(*prompt)
        code = self._lib.leone_sched_add(self._h, c_longlong(key), ids, c_longlong(len(prompt)),
                                         c_longlong(int(max_new_tokens)))
        if code != 0:
            raise AdmissionError(_REJECTS[code], self._lib.leone_host_last_error().decode())
        self._next_key += 1
        req = Request(rid, prompt, max_new_tokens, sampling or SamplingParams(), eos_token_id, stop_ids,
                      arrival=int(self._lib.leone_sched_get(self._h, c_longlong(key), 6)),
                      tokens=list(prompt), key=key)
        if getattr(req.sampling, "mirostat", None):
            req.sampler_state = SamplerState(req.sampling)
        self.requests[rid] = req
        self._by_key[key] = req
        return req

    def cancel(self, rid: Hashable) -> None:
        """Queued: removed at once.  Running: stops at the next step boundary
        (crates/leone/src/scheduler.rs:540-554)."""
        req = self.requests.get(rid)
        if req is None:
            return
        what = self._lib.leone_sched_cancel(self._h, c_longlong(req.key))
        if what == 1:
            req.state, req.finish_reason = "cancelled", "cancelled"
        elif what == 2:
            req.cancel_requested = True
            self._record(req, cancel=True)

    # -- one step's decisions -----------------------------------------------------------
    def _keys(self, n: int) -> List[int]:
        return list(self._buf[0][:n])

    def _drop_cancelled(self) -> None:
        n = self._lib.leone_sched_drop_cancelled(self._h, self._buf[0], self._cap)
        for key in self._keys(n):
            req = self._by_key[key]
            self.engine.close(req.rid)
            req.state, req.finish_reason, req.reserved_pages, req.slot = "cancelled", "cancelled", 0, None

    def _record(self, req: Request, **fields) -> None:
        """Mirror the request's state into its slot record (``leone_b200.cache.slots``): the
        record is what the captured decode step reads, and where the request's sampling state,
        progress and cancellation flag live for as long as it holds its slot."""
        records = getattr(self.engine, "slot_records", None)
        if records is None or req.slot is None:
            return
        if "sampling" in fields:
            records.set_sampling(req.slot, req.sampling.seed, req.sampling.temperature)
        if "progress" in fields:
            records.set_progress(req.slot, req.computed, max(len(req.tokens) - 1, 0),
                                 req.tokens[-1] if req.tokens else None)
        if "cancel" in fields:
            records.request_cancel(req.slot)
        if "sampler" in fields and req.sampler_state is not None and req.sampler_state.maximum_surprise is not None:
            records.set_sampler_state(req.slot, req.sampler_state.maximum_surprise)

    def _try_admit(self) -> None:
        """Move requests from the queue to running, in arrival order, while they fit."""
        n = self._lib.leone_sched_admit(self._h, self._buf[0], self._cap)
        for key in self._keys(n):
            req = self._by_key[key]
            req.slot = self.engine.open(req.rid)
            self._record(req, sampling=True, progress=True, sampler=True)
            req.state, req.computed = "running", 0
            req.reserved_pages = int(self._lib.leone_sched_get(self._h, c_longlong(key), 4))

    def plan(self, admit: bool = True):
        """Entries of the next step as ``(request, first token index, count)`` triples."""
        self._drop_cancelled()
        if admit:
            self._try_admit()
        rids, starts, counts = self._buf
        n = self._lib.leone_sched_plan(self._h, rids, starts, counts, self._cap)
        return [(self._by_key[rids[i]], int(starts[i]), int(counts[i])) for i in range(n)]

    def _emitted(self, req: Request, tok: int) -> Optional[str]:
        """Book a sampled token; returns why the request ends now, if it does (it is closed then)."""
        req.generated.append(tok)
        req.tokens.append(tok)
        is_eos = tok in req.stop_ids
        code = self._lib.leone_sched_emitted(self._h, c_longlong(req.key), int(is_eos))
        if code <= 0:
            self._record(req, progress=True, sampler=True)
            return None
        self.engine.close(req.rid)
        req.state, req.finish_reason, req.reserved_pages, req.slot = "finished", _FINISH[code], 0, None
        return req.finish_reason

    def _preempt_youngest(self) -> bool:
        """The youngest running request other than the oldest goes back to the queue."""
        victim = c_longlong(-1)
        keep = self._lib.leone_sched_oldest_running(self._h)
        if not self._lib.leone_sched_preempt_youngest(self._h, c_longlong(keep), ctypes.byref(victim)):
            return False
        req = self._by_key[victim.value]
        self.engine.close(req.rid)
        req.state, req.computed, req.slot = "waiting", 0, None
        req.preemptions += 1
        return True

    # -- one step ---------------------------------------------------------------------------
    def step(self) -> List[StepOutput]:
        """Plan, run and account one batch.  Returns the tokens emitted in this step."""
        admit = True
        while True:
            plan = self.plan(admit)
            if not plan:
                if self._count(0) and not self._count(1):
                    raise RuntimeError("the head of the queue cannot be admitted into an empty engine")
                return []
            try:
                if self._decode_only(plan) and self.config.use_graphs and hasattr(self.engine, "decode_steps"):
                    return self._decode_quantum([req for req, _, _ in plan])
                if (self._decode_rows(plan) and self.config.use_graphs and hasattr(self.engine, "decode_logits")):
                    # requests whose sampler the captured step does not hold: the step still runs
                    # from the graph, and its logits are sampled below like any other step's
                    logits = self.engine.decode_logits([req.rid for req, _, _ in plan],
                                                       [req.tokens[-1] for req, _, _ in plan])
                    break
                entries = []
                for req, start, count in plan:
                    last = start + count == len(req.tokens)
                    entries.append((req.rid, req.tokens[start:start + count], [count - 1] if last else []))
                logits = self.engine.step(entries)
                break
            except OutOfPages:
                if self.config.policy != "optimistic" or not self._preempt_youngest():
                    raise
                admit = False          # the freed pages go to the requests that stay
        outputs: List[StepOutput] = []
        sampled_reqs = []
        for req, start, count in plan:
            if count == 1 and req.generated and start == len(req.tokens) - 1:
                self._decode_tokens += 1
            else:
                self._prefill_tokens += count
            self._lib.leone_sched_computed(self._h, c_longlong(req.key), c_longlong(count))
            req.computed = start + count
            if req.computed == len(req.tokens):
                sampled_reqs.append(req)
        self._steps += 1
        self._max_batch_tokens_seen = max(self._max_batch_tokens_seen, sum(c for _, _, c in plan))
        if sampled_reqs:
            kw = {}
            if any(getattr(r.sampling, "penalizes", False) for r in sampled_reqs):
                kw["histories"] = [r.tokens for r in sampled_reqs]      # the whole history, prompt included
            if any(r.sampler_state is not None for r in sampled_reqs):
                kw["states"] = [r.sampler_state for r in sampled_reqs]
            ids = self.engine.sample(logits, [r.sampling for r in sampled_reqs],
                                     [len(r.tokens) - 1 for r in sampled_reqs], **kw)
            for req, tok in zip(sampled_reqs, ids):
                reason = self._emitted(req, int(tok))
                outputs.append(StepOutput(req.rid, int(tok), reason is not None, reason))
        return outputs

    @staticmethod
    def _decode_rows(plan) -> bool:
        """Every entry feeds the one token its request sampled last."""
        return all(count == 1 and req.generated and start == len(req.tokens) - 1 for req, start, count in plan)

    @classmethod
    def _decode_only(cls, plan) -> bool:
        """Every entry is a decode row that the captured step can also sample (greedy or
        temperature; truncation stages, penalties and Mirostat run outside the graph)."""
        return cls._decode_rows(plan) and not any(getattr(req.sampling, "outside_graph", False)
                                                  for req, _, _ in plan)

    def _decode_quantum(self, reqs: List[Request]) -> List[StepOutput]:
        """Several decode steps of the same requests without the host in between.  A request
        that finishes inside the quantum drops the tokens sampled after its end (the reference
        bounds the same overshoot by its quantum, crates/leone/src/scheduler.rs:1334-1338)."""
        keys = (c_longlong * len(reqs))(*[r.key for r in reqs])
        q = int(self._lib.leone_sched_decode_quantum(self._h, len(reqs), keys, c_longlong(self.config.decode_quantum)))
        # no request reaches its limit in this quantum: the same batch decodes again
        more = all(r.remaining_new > q for r in reqs)
        steps = self.engine.decode_steps([r.rid for r in reqs], [r.tokens[-1] for r in reqs],
                                         [r.sampling for r in reqs], q, expect_more=more)
        outputs: List[StepOutput] = []
        live = list(range(len(reqs)))                   # rows whose request has not ended
        for row in steps:
            n = len(live)
            toks = [int(row[i]) for i in live]
            is_eos = (c_int * n)(*[int(t in reqs[i].stop_ids) for i, t in zip(live, toks)])
            reasons = (c_int * n)()
            code = self._lib.leone_sched_decoded(self._h, n, (c_longlong * n)(*[reqs[i].key for i in live]),
                                                 is_eos, reasons)       # the step's bookkeeping in one call
            if code != 0:
                raise RuntimeError(self._lib.leone_host_last_error().decode())
            still = []
            for i, tok, code in zip(live, toks, reasons):
                req = reqs[i]
                req.computed += 1
                req.generated.append(tok)
                req.tokens.append(tok)
                reason = None
                if code > 0:
                    self.engine.close(req.rid)
                    req.state, req.finish_reason, req.reserved_pages, req.slot = "finished", _FINISH[code], 0, None
                    reason = req.finish_reason
                else:
                    still.append(i)
                outputs.append(StepOutput(req.rid, tok, reason is not None, reason))
            self._decode_tokens += n
            live = still
        self._steps += q
        self._max_batch_tokens_seen = max(self._max_batch_tokens_seen, len(reqs))
        return outputs

    def run_to_completion(self, on_token: Optional[Callable[[StepOutput], None]] = None) -> None:
        while self.has_work():
            for out in self.step():
                if on_token:
                    on_token(out)

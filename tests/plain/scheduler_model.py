"""Plain model of the scheduler, in Python: what the engine's scheduler (decisions in C++) is
compared with.  Tests drive both with the same requests over the same fake engine and compare
every step's batch and every request's tokens and end.  It shares no code with the product and
works over the plain cache model beside it.

Each step: one token for every request that is decoding, then portions of waiting prompts in
arrival order until the token budget is used (crates/leone/src/scheduler.rs:341-378 dispatches
per request with min(remaining_prefill, prefill_chunk_tokens) or a decode quantum).  Policies
when pages run out: "reserve" sets pages aside for a request's whole life at admission
(crates/leone/src/scheduler.rs:652-667); "optimistic" preempts the youngest running request.
N new tokens need the cache for P + N - 1 positions (crates/leone/src/runtime.rs:3602-3607).
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence

from .cache_model import OutOfPages


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
    rid: Hashable
    prompt: List[int]
    max_new_tokens: int
    sampling: object = None
    eos_token_id: Optional[int] = None
    arrival: int = 0
    # progress
    tokens: List[int] = field(default_factory=list)      # prompt + generated, what the cache must hold
    computed: int = 0                                    # tokens already in the cache
    generated: List[int] = field(default_factory=list)
    state: str = "waiting"                               # waiting | running | finished | cancelled
    finish_reason: Optional[str] = None
    reserved_pages: int = 0
    preemptions: int = 0
    cancel_requested: bool = False

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
        self.config = config or SchedulerConfig()
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.requests: Dict[Hashable, Request] = {}
        self._arrivals = itertools.count()
        self._reserved_total = 0
        self._reserved_by_group: List[int] = []
        self.stats = dict(steps=0, prefill_tokens=0, decode_tokens=0, preemptions=0, admitted=0,
                          finished=0, cancelled=0, max_batch_tokens_seen=0)

    # -- admission --------------------------------------------------------------------
    def _needs(self, total: int) -> List[int]:
        """Per cache group, the most pages a request that comes to hold ``total`` tokens holds at
        one time: all its blocks in a full group; in a window group what lies between the first
        block a query can still see and the end of the step's tokens, at the worst alignment."""
        cfg = self.config
        portion = max(min(cfg.prefill_chunk_tokens, cfg.max_batch_tokens), cfg.decode_quantum)
        needs = []
        for g in self.engine.cache.groups:
            every = g.blocks_for(total)
            if g.spec.kind != "window":
                needs.append(every)
                continue
            w = g.spec.window
            most = max(g.blocks_for(c + portion) - g.first_live_block(c) for c in range(w, w + g.page_tokens))
            needs.append(min(every, most))
        return needs

    def add_request(self, rid: Hashable, prompt: Sequence[int], max_new_tokens: int,
                    sampling=None, eos_token_id: Optional[int] = None) -> Request:
        spec = self.engine.spec
        prompt = [int(t) for t in prompt]
        if rid in self.requests and self.requests[rid].state in ("waiting", "running"):
            raise AdmissionError("duplicate", f"request id {rid!r} is already in flight")
        if len(prompt) == 0:
            raise AdmissionError("empty_prompt", "a request needs at least one prompt token")
        if max_new_tokens <= 0:
            raise AdmissionError("output_limit", "max_new_tokens must be positive")
        bad = [t for t in prompt if not 0 <= t < spec.vocab_size]
        if bad:
            raise AdmissionError("token_id", f"token ids {bad[:8]} are outside the vocabulary "
                                             f"of {spec.vocab_size}")
        need_positions = len(prompt) + max_new_tokens - 1
        if need_positions > spec.max_positions:
            raise AdmissionError("prompt_limit", f"prompt ({len(prompt)}) + max_new_tokens "
                                 f"({max_new_tokens}) - 1 exceeds the model's {spec.max_positions} positions")
        for g, need in zip(self.engine.cache.groups, self._needs(need_positions)):
            if need > g.pool.num_pages:
                raise AdmissionError("kv_capacity", f"the request needs {need} pages; "
                                     f"the pool has {g.pool.num_pages} even when empty")
        if len(self.waiting) >= self.config.max_waiting:
            raise AdmissionError("queue_limit", f"{self.config.max_waiting} requests are already waiting")
        req = Request(rid, prompt, max_new_tokens, sampling, eos_token_id,
                      arrival=next(self._arrivals), tokens=list(prompt))
        self.requests[rid] = req
        self.waiting.append(req)
        return req

    def cancel(self, rid: Hashable) -> None:
        """Queued: removed at once.  Running: stops at the next step boundary
        (crates/leone/src/scheduler.rs:540-554)."""
        req = self.requests.get(rid)
        if req is None or req.state in ("finished", "cancelled"):
            return
        if req.state == "waiting":
            self.waiting.remove(req)
            req.state, req.finish_reason = "cancelled", "cancelled"
            self.stats["cancelled"] += 1
        else:
            req.cancel_requested = True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- one step's decisions -----------------------------------------------------------
    def _free_pages(self) -> int:
        return min(self.engine.cache.free_pages()) if self.engine.cache.groups else 1 << 30

    def _try_admit(self) -> None:
        """Move requests from the queue to running, in arrival order, while they fit."""
        cfg = self.config
        while self.waiting and len(self.running) < cfg.max_running:
            req = self.waiting[0]
            if self.engine.cache.slots.num_free == 0:
                break
            if cfg.policy == "reserve":
                needs = self._needs(len(req.tokens) + req.remaining_new - 1)
                groups = self.engine.cache.groups
                if len(self._reserved_by_group) != len(groups):
                    self._reserved_by_group = [0] * len(groups)
                if any(have + need > g.pool.num_pages
                       for have, need, g in zip(self._reserved_by_group, needs, groups)):
                    break
                self._reserved_by_group = [have + need for have, need in zip(self._reserved_by_group, needs)]
                req.needs = needs
                req.reserved_pages = max(needs, default=0)
                self._reserved_total += req.reserved_pages
            else:
                first = min(len(req.tokens), cfg.prefill_chunk_tokens)
                if self.running and any(g.blocks_for(first) > g.pool.num_free for g in self.engine.cache.groups):
                    break
            self.waiting.popleft()
            self.engine.open(req.rid)
            req.state = "running"
            req.computed = 0
            self.running.append(req)
            self.stats["admitted"] += 1

    def plan(self, admit: bool = True):
        """Entries of the next step as ``(request, first token index, count)`` triples."""
        self._drop_cancelled()
        if admit:
            self._try_admit()
        budget = self.config.max_batch_tokens
        plan = []
        decoding = lambda r: bool(r.generated) and r.computed == len(r.tokens) - 1   # noqa: E731
        hold_decodes = self.config.prefill_first and any(not decoding(r) for r in self.running)
        for req in self.running:                       # decode rows first
            if hold_decodes:
                break
            if req.computed == len(req.tokens) - 1 and req.generated and budget > 0:
                plan.append((req, req.computed, 1))
                budget -= 1
        for req in self.running:                       # then prompt portions, oldest first
            if budget <= 0:
                break
            left = len(req.tokens) - req.computed
            if left >= 1 and not (left == 1 and req.generated):
                count = min(left, self.config.prefill_chunk_tokens, budget)
                plan.append((req, req.computed, count))
                budget -= count
        return plan

    def _drop_cancelled(self) -> None:
        for req in [r for r in self.running if r.cancel_requested]:
            self._retire(req, "cancelled")

    def _retire(self, req: Request, reason: str) -> None:
        self.engine.close(req.rid)
        self.running.remove(req)
        self._reserved_total -= req.reserved_pages
        req.reserved_pages = 0
        for i, need in enumerate(getattr(req, "needs", [])):
            self._reserved_by_group[i] -= need
        req.needs = []
        req.state = "cancelled" if reason == "cancelled" else "finished"
        req.finish_reason = reason
        self.stats["cancelled" if reason == "cancelled" else "finished"] += 1

    def _preempt_youngest(self, keep: Optional[Request] = None) -> bool:
        victims = [r for r in self.running if r is not keep]
        if not victims:
            return False
        victim = max(victims, key=lambda r: r.arrival)
        self.engine.close(victim.rid)
        self.running.remove(victim)
        victim.state = "waiting"
        victim.computed = 0
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(victim)
        return True

    # -- one step ---------------------------------------------------------------------------
    def step(self) -> List[StepOutput]:
        """Plan, run and account one batch.  Returns the tokens emitted in this step."""
        admit = True
        while True:
            plan = self.plan(admit)
            if not plan:
                if self.waiting and not self.running:
                    raise RuntimeError("the head of the queue cannot be admitted into an empty engine")
                return []
            if self._decode_only(plan) and self.config.use_graphs and hasattr(self.engine, "decode_steps"):
                try:
                    return self._decode_quantum([req for req, _, _ in plan])
                except OutOfPages:
                    if self.config.policy != "optimistic":
                        raise
                    oldest = min(self.running, key=lambda r: r.arrival)
                    if not self._preempt_youngest(keep=oldest):
                        raise
                    admit = False
                    continue
            entries = []
            for req, start, count in plan:
                last = start + count == len(req.tokens)
                entries.append((req.rid, req.tokens[start:start + count], [count - 1] if last else []))
            try:
                logits = self.engine.step(entries)
                break
            except OutOfPages:
                if self.config.policy != "optimistic":
                    raise
                oldest = min(self.running, key=lambda r: r.arrival)
                if not self._preempt_youngest(keep=oldest):
                    raise
                admit = False          # the freed pages go to the requests that stay
        outputs: List[StepOutput] = []
        sampled_reqs = []
        for req, start, count in plan:
            req.computed = start + count
            if count == 1 and req.generated and start == len(req.tokens) - 1:
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prefill_tokens"] += count
            if req.computed == len(req.tokens):
                sampled_reqs.append(req)
        self.stats["steps"] += 1
        self.stats["max_batch_tokens_seen"] = max(self.stats["max_batch_tokens_seen"],
                                                  sum(c for _, _, c in plan))
        if sampled_reqs:
            ids = self.engine.sample(logits, [r.sampling for r in sampled_reqs],
                                     [len(r.tokens) - 1 for r in sampled_reqs])
            for req, tok in zip(sampled_reqs, ids):
                tok = int(tok)
                req.generated.append(tok)
                req.tokens.append(tok)
                reason = self._finish_reason(req, tok)
                if reason:
                    self._retire(req, reason)
                outputs.append(StepOutput(req.rid, tok, reason is not None, reason))
        return outputs

    @staticmethod
    def _decode_only(plan) -> bool:
        return all(count == 1 and req.generated and start == len(req.tokens) - 1
                   for req, start, count in plan)

    def _finish_reason(self, req: Request, tok: int) -> Optional[str]:
        if req.eos_token_id is not None and tok == req.eos_token_id:
            return "eos"
        if len(req.generated) >= req.max_new_tokens:
            return "length"
        if len(req.tokens) > self.engine.spec.max_positions:
            return "max_positions"
        return None

    def _decode_quantum(self, reqs: List[Request]) -> List[StepOutput]:
        """Several decode steps of the same requests without the host in between.  A request
        that finishes inside the quantum drops the tokens sampled after its end (the reference
        bounds the same overshoot by its quantum, crates/leone/src/scheduler.rs:1334-1338)."""
        q = min([self.config.decode_quantum] + [r.remaining_new for r in reqs] +
                [self.engine.spec.max_positions - len(r.tokens) + 1 for r in reqs])
        q = max(1, q)
        steps = self.engine.decode_steps([r.rid for r in reqs], [r.tokens[-1] for r in reqs],
                                         [r.sampling for r in reqs], q)
        outputs: List[StepOutput] = []
        done = set()
        for row in steps:
            for req, tok in zip(reqs, row):
                if req.rid in done:
                    continue
                tok = int(tok)
                req.generated.append(tok)
                req.tokens.append(tok)
                req.computed += 1
                self.stats["decode_tokens"] += 1
                reason = self._finish_reason(req, tok)
                if reason:
                    done.add(req.rid)
                    self._retire(req, reason)
                outputs.append(StepOutput(req.rid, tok, reason is not None, reason))
        self.stats["steps"] += q
        self.stats["max_batch_tokens_seen"] = max(self.stats["max_batch_tokens_seen"], len(reqs))
        return outputs

    def run_to_completion(self, on_token: Optional[Callable[[StepOutput], None]] = None) -> None:
        while self.has_work():
            for out in self.step():
                if on_token:
                    on_token(out)

"""The scheduler's decisions, with a fake step function (no model) and with the tiny model on
emulated kernels."""
import random

import pytest
import torch

from leone_b200.cache.pages import CacheManager, GroupSpec, OutOfPages
from leone_b200.engine.scheduler import AdmissionError, Scheduler, SchedulerConfig
from leone_b200.sampling.sampler import SamplingParams


class FakeSpec:
    vocab_size = 100
    max_positions = 64


class FakeEngine:
    """The engine's interface without a model: the 'next token' is a function of the request's
    tokens so far, so any scheduling must produce the same stream as running alone."""

    def __init__(self, pages=8, page_tokens=4, slots=4, cache_module=None, windows=(None,)):
        """``windows``: one cache group per entry; None is a full group, a number a window group."""
        self.spec = FakeSpec()
        make, group = (cache_module.CacheManager, cache_module.GroupSpec) if cache_module else (CacheManager, GroupSpec)
        self.cache = make([group("window", 1, 8, w) if w else group("full", 1, 8) for w in windows],
                          page_tokens, pages, slots)
        self.seen = {}
        self.batches = []

    def open(self, rid):
        self.cache.open(rid)
        self.seen[rid] = []

    def close(self, rid):
        self.cache.close(rid)

    def step(self, entries):
        wants = {rid: self.cache.length(rid) + len(toks) for rid, toks, _ in entries}
        self.cache.reserve(wants)
        rows = []
        for rid, toks, want in entries:
            assert len(self.seen[rid]) == self.cache.length(rid)
            self.seen[rid] = self.seen[rid] + list(toks)
            for w in want:
                prefix = self.seen[rid][:len(self.seen[rid]) - len(toks) + w + 1]
                rows.append(prefix)
            self.cache.commit(rid, wants[rid])
        self.batches.append([(rid, len(toks)) for rid, toks, _ in entries])
        self.cache.check_invariants()
        return rows

    def sample(self, rows, params, positions):
        assert [len(r) - 1 for r in rows] == list(positions)
        return [next_token(r) for r in rows]


class FakeGraphEngine(FakeEngine):
    """The same with the engine's ``decode_steps``: several decode steps without the scheduler
    in between, pages for all of them taken first."""

    def decode_steps(self, rids, last_tokens, params, steps, **_):
        wants = {r: self.cache.length(r) + steps for r in rids}
        self.cache.reserve(wants)
        rows = []
        toks = list(last_tokens)
        for _ in range(steps):
            for r, t in zip(rids, toks):
                self.seen[r] = self.seen[r] + [t]
            toks = [next_token(self.seen[r]) for r in rids]
            rows.append(toks)
        for r in rids:
            self.cache.commit(r, wants[r])
        self.batches.append([(r, steps) for r in rids])
        self.cache.check_invariants()
        return rows


def next_token(prefix):
    return (sum(prefix) * 31 + len(prefix) * 7) % 100


def alone(prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        out.append(next_token(toks))
        toks.append(out[-1])
    return out


def _run(sched):
    guard = 0
    while sched.has_work():
        sched.step()
        guard += 1
        assert guard < 10000
    return {rid: r.generated for rid, r in sched.requests.items()}


def test_typed_rejections():
    s = Scheduler(FakeEngine(), SchedulerConfig(max_waiting=1))
    for reason, args in [("empty_prompt", ([], 3)), ("output_limit", ([1], 0)), ("token_id", ([100], 2)),
                         ("prompt_limit", ([1] * 60, 10)), ("kv_capacity", ([1] * 30, 10))]:
        with pytest.raises(AdmissionError) as err:
            s.add_request("x", *args)
        assert err.value.reason == reason
    s.add_request("a", [1, 2], 2)
    with pytest.raises(AdmissionError) as err:
        s.add_request("a", [1], 1)
    assert err.value.reason == "duplicate"
    with pytest.raises(AdmissionError) as err:
        s.add_request("b", [1], 1)
    assert err.value.reason == "queue_limit"


def test_token_budget_and_portions():
    eng = FakeEngine(pages=16)
    s = Scheduler(eng, SchedulerConfig(max_batch_tokens=8, prefill_chunk_tokens=5))
    s.add_request("a", list(range(1, 14)), 3)       # 13 prompt tokens
    s.add_request("b", [5, 6, 7], 3)
    got = _run(s)
    assert got == {"a": alone(list(range(1, 14)), 3), "b": alone([5, 6, 7], 3)}
    assert all(sum(n for _, n in batch) <= 8 for batch in eng.batches)
    assert all(n <= 5 for batch in eng.batches for _, n in batch)
    # the first batch: a's first portion of 5 and b's whole prompt of 3
    assert eng.batches[0] == [("a", 5), ("b", 3)]
    # later, a decodes beside nothing or beside b: decode rows come first in a batch
    mixed = [b for b in eng.batches if len(b) == 2 and b[0][1] == 1 and b[1][1] > 1]
    assert mixed, "a decode row and a prompt portion never shared a batch"


def test_prefill_first_holds_decodes_until_prompts_are_done():
    eng = FakeEngine(pages=16)
    s = Scheduler(eng, SchedulerConfig(max_batch_tokens=8, prefill_chunk_tokens=5, prefill_first=True))
    s.add_request("a", list(range(1, 14)), 3)
    s.add_request("b", [5, 6, 7], 3)
    got = _run(s)
    assert got == {"a": alone(list(range(1, 14)), 3), "b": alone([5, 6, 7], 3)}
    prompt_steps = [i for i, b in enumerate(eng.batches) if any(n > 1 for _, n in b)]
    decode_steps = [i for i, b in enumerate(eng.batches) if all(n == 1 for _, n in b)]
    assert max(prompt_steps) < min(decode_steps)
    assert all(len(b) == 2 for b in eng.batches[min(decode_steps):min(decode_steps) + 2])


def test_reserve_policy_never_runs_out_and_queues_in_order():
    eng = FakeEngine(pages=6, page_tokens=4)
    s = Scheduler(eng, SchedulerConfig(policy="reserve"))
    prompts = {i: [i + 1] * 7 for i in range(4)}     # 7 + 6 - 1 = 12 tokens = 3 pages each
    for i, p in prompts.items():
        s.add_request(i, p, 6)
    s.step()
    assert [r.rid for r in s.running] == [0, 1] and [r.rid for r in s.waiting] == [2, 3]
    got = _run(s)
    assert got == {i: alone(p, 6) for i, p in prompts.items()}
    assert s.stats["preemptions"] == 0
    assert eng.cache.free_pages() == [6]


def test_optimistic_policy_preempts_the_youngest_and_recomputes():
    eng = FakeEngine(pages=5, page_tokens=4)
    s = Scheduler(eng, SchedulerConfig(policy="optimistic"))
    prompts = {i: [i + 3] * 6 for i in range(3)}     # each grows to 6 + 8 - 1 = 13 tokens = 4 pages
    for i, p in prompts.items():
        s.add_request(i, p, 8)
    got = _run(s)
    assert got == {i: alone(p, 8) for i, p in prompts.items()}
    assert s.stats["preemptions"] > 0
    assert s.requests[0].preemptions == 0            # the oldest is never the victim
    assert eng.cache.free_pages() == [5]


def test_cancel_waiting_and_running():
    eng = FakeEngine(pages=16)
    s = Scheduler(eng, SchedulerConfig(max_running=1))
    s.add_request("a", [1, 2, 3], 20)
    s.add_request("b", [4, 5], 5)
    s.step()
    s.cancel("b")                                    # still queued: gone at once
    assert s.requests["b"].state == "cancelled" and not s.waiting
    s.step()
    s.cancel("a")                                    # running: stops at the next step boundary
    before = len(s.requests["a"].generated)
    s.step()
    assert s.requests["a"].state == "cancelled" and len(s.requests["a"].generated) == before
    assert not s.has_work() and eng.cache.free_pages() == [16]


def test_eos_and_length():
    eng = FakeEngine(pages=16)
    s = Scheduler(eng)
    free = alone([9, 9], 6)
    s.add_request("a", [9, 9], 6, eos_token_id=free[2])
    s.add_request("b", [9, 9], 4)
    got = _run(s)
    assert got["a"] == free[:free.index(free[2]) + 1] and s.requests["a"].finish_reason == "eos"
    assert got["b"] == free[:4] and s.requests["b"].finish_reason == "length"


def test_any_of_several_stop_ids_ends_a_request():
    """A checkpoint may list several end ids; a request stops at the first one it samples."""
    eng = FakeEngine(pages=16)
    s = Scheduler(eng)
    free = alone([9, 9], 6)
    distinct = [t for i, t in enumerate(free) if t not in free[:i]]
    assert len(distinct) >= 3
    unused = next(t for t in range(1000) if t not in free)
    s.add_request("a", [9, 9], 6, eos_token_id=[unused, distinct[2]])
    s.add_request("b", [9, 9], 6, eos_token_id=(distinct[1], distinct[2]))
    got = _run(s)
    assert got["a"] == free[:free.index(distinct[2]) + 1] and s.requests["a"].finish_reason == "eos"
    assert got["b"] == free[:free.index(distinct[1]) + 1] and s.requests["b"].finish_reason == "eos"


@pytest.mark.parametrize("seed", range(5))
def test_interleaved_transcripts_equal_isolated_ones(seed):
    """A scripted arrival trace: whatever the interleaving, each request's tokens are the ones
    it produces alone (the reference checks the same, crates/leone/src/scheduler.rs:1227-1252)."""
    rng = random.Random(seed)
    eng = FakeEngine(pages=12, page_tokens=4, slots=3)
    s = Scheduler(eng, SchedulerConfig(max_running=3, max_batch_tokens=rng.choice([4, 6, 16]),
                                       prefill_chunk_tokens=rng.choice([2, 3, 7]),
                                       policy=rng.choice(["reserve", "optimistic"])))
    arrivals = sorted((rng.randint(0, 25), i) for i in range(7))
    specs = {i: ([rng.randrange(100) for _ in range(rng.randint(1, 12))], rng.randint(1, 9)) for _, i in arrivals}
    tick = 0
    while arrivals or s.has_work():
        while arrivals and arrivals[0][0] <= tick:
            _, i = arrivals.pop(0)
            s.add_request(i, *specs[i])
        if s.has_work():
            s.step()
        tick += 1
        assert tick < 5000
    for i, (prompt, n) in specs.items():
        assert s.requests[i].generated == alone(prompt, n), i
    assert eng.cache.free_pages() == [12]


def test_generation_with_the_tiny_model_on_emulated_kernels(tmp_path):
    """The scheduler over the real step function (CPU stand-in kernels): tiny A greedy and
    tiny B with temperature, both page policies, against the plain implementation."""
    from leone_b200.engine.engine import Engine
    from leone_b200.engine.generate import generate
    from tests import replay
    from tests.emulated_ops import EmulatedOps
    from tests.plain.model import PlainModel, generate as plain_generate
    from tests.tiny import PAGE_TOKENS, make_folder
    for which, temp, lens, n_new in (("A", 0.0, (5, 9, 13), 8), ("B", 0.8, (1, 7, 17, 30), 6)):
        folder = make_folder(tmp_path, which)
        plain = PlainModel(folder)
        prompts = [replay.random_tokens(plain.cfg["vocab_size"], n, 50 + n) for n in lens]
        want = [plain_generate(plain, p, n_new, temp, 7 + i) for i, p in enumerate(prompts)]
        for policy, pages in (("reserve", 14), ("optimistic", 9)):
            eng = Engine.from_folder(folder, dtype="float32", device="cpu", ops=EmulatedOps(),
                                     page_tokens=PAGE_TOKENS[which], num_pages=pages, max_requests=4,
                                     max_batch_tokens=16)
            for first in (False, True):
                got = generate(eng, prompts, n_new, temperature=temp, seed=7, prefill_chunk=6,
                               max_batch_tokens=16, policy=policy, eos_token_id=-1, prefill_first=first)
                assert got == want, (which, policy, first)
            eng.cache.check_invariants()
            assert eng.cache.free_pages()[0] == pages


@pytest.mark.parametrize("seed", range(12))
def test_the_native_planner_and_the_plain_scheduler_agree_step_by_step(seed):
    """The same arrivals, cancellations and limits go to the scheduler (decisions in C++, over the
    C++ cache manager) and to the Python model under tests/plain (over its own cache model):
    every step's batch, every emitted token, every request's end and the counters are equal."""
    from tests.plain import cache_model, scheduler_model
    rng = random.Random(500 + seed)
    policy = ["reserve", "optimistic"][seed % 2]
    pages, page_tokens, slots = rng.choice([5, 7, 12]), rng.choice([2, 4]), rng.choice([2, 3, 5])
    limits = dict(max_running=rng.choice([2, 3, 8]), max_waiting=rng.choice([3, 50]),
                  max_batch_tokens=rng.choice([4, 8, 32]), prefill_chunk_tokens=rng.choice([2, 5, 32]),
                  policy=policy, prefill_first=bool(seed % 3 == 0))
    make = FakeGraphEngine if seed % 4 >= 2 else FakeEngine       # with and without decode quanta
    limits["decode_quantum"] = rng.choice([1, 2, 4])
    windows = [(None,), (None, 6), (5,)][seed % 3]               # one full group; full + window; a window alone
    ea = make(pages, page_tokens, slots, windows=windows)
    eb = make(pages, page_tokens, slots, cache_module=cache_model, windows=windows)
    a = Scheduler(ea, SchedulerConfig(**limits))
    b = scheduler_model.Scheduler(eb, scheduler_model.SchedulerConfig(**limits))
    arrivals = 0
    for tick in range(300):
        for _ in range(rng.choice([0, 0, 1, 2])):
            rid = arrivals if rng.random() < 0.9 else rng.randrange(arrivals + 1)
            arrivals += 1
            prompt = [rng.randrange(0, 103) for _ in range(rng.choice([0, 1, 3, 9, 20, 70]))]
            new = rng.choice([0, 1, 2, 5, 9])
            eos = rng.choice([None, None, 7, 50])
            errs = []
            for s_, err in ((a, AdmissionError), (b, scheduler_model.AdmissionError)):
                try:
                    s_.add_request(rid, prompt, new, None, eos)
                    errs.append(None)
                except err as exc:
                    errs.append(exc.reason)
            assert errs[0] == errs[1], (rid, prompt, new, errs)
        if rng.random() < 0.1 and arrivals:
            rid = rng.randrange(arrivals)
            a.cancel(rid)
            b.cancel(rid)
        outs = []
        for s_ in (a, b):
            try:
                outs.append([(o.rid, o.token, o.finished, o.finish_reason) for o in s_.step()])
            except (OutOfPages, cache_model.OutOfPages):
                outs.append("out of pages")
            except RuntimeError as exc:
                outs.append(str(exc))
        assert outs[0] == outs[1], tick
        assert ea.batches == eb.batches
        assert [r.rid for r in a.running] == [r.rid for r in b.running]
        assert [r.rid for r in a.waiting] == [r.rid for r in b.waiting]
        assert a.stats == b.stats
        assert ea.cache.free_pages() == eb.cache.free_pages()
        if isinstance(outs[0], str):
            break
    for rid, rb in b.requests.items():
        ra = a.requests[rid]
        assert (ra.state, ra.finish_reason, ra.generated, ra.tokens, ra.computed, ra.preemptions, ra.reserved_pages) == \
               (rb.state, rb.finish_reason, rb.generated, rb.tokens, rb.computed, rb.preemptions, rb.reserved_pages), rid


@pytest.mark.parametrize("seed", range(6))
def test_admission_counts_each_group_and_a_reserved_request_never_runs_out(seed):
    """Under the reserve policy every group sets aside what a request holds there at its largest:
    all its blocks in a full group, a window's worth in a window group.  With a window group
    alone, more requests run at once than their full lengths would allow, and no step of an
    admitted request ever fails for pages."""
    rng = random.Random(900 + seed)
    page_tokens, window = rng.choice([2, 4]), rng.choice([3, 6, 9])
    cfg = SchedulerConfig(max_running=6, max_batch_tokens=rng.choice([6, 16]), prefill_chunk_tokens=rng.choice([3, 5]),
                          decode_quantum=rng.choice([1, 4]), policy="reserve")
    portion = max(min(cfg.prefill_chunk_tokens, cfg.max_batch_tokens), cfg.decode_quantum)
    worst = -(-(window + portion) // page_tokens) + 1
    make = FakeGraphEngine if cfg.decode_quantum > 1 else FakeEngine
    eng = make(pages=3 * worst, page_tokens=page_tokens, slots=6, windows=(window,))
    s = Scheduler(eng, cfg)
    specs = {i: ([rng.randrange(100) for _ in range(rng.randint(20, 40))], rng.randint(5, 20)) for i in range(6)}
    for i, (prompt, n) in specs.items():
        s.add_request(i, prompt, n)
    most_running = 0
    guard = 0
    while s.has_work():
        s.step()                                       # OutOfPages here would fail the test
        most_running = max(most_running, len(s.running))
        guard += 1
        assert guard < 5000
    # by full length each request would need at least 25 / page_tokens pages: fewer would fit
    by_full_length = (3 * worst) // -(-25 // page_tokens)
    assert most_running >= 3 and most_running >= by_full_length
    for i, (prompt, n) in specs.items():
        assert s.requests[i].generated == alone(prompt, n), i
    assert eng.cache.free_pages() == [3 * worst]
    # two groups: the full group is the one that limits
    eng2 = FakeEngine(pages=12, page_tokens=4, slots=6, windows=(None, 4))
    s2 = Scheduler(eng2, SchedulerConfig(max_running=6, policy="reserve"))
    for i in range(3):
        s2.add_request(i, [1] * 20, 4)                 # 23 positions: 6 pages of the full group each
    s2.step()
    assert len(s2.running) == 2 and len(s2.waiting) == 1


def test_sampler_options_through_the_scheduler_on_emulated_kernels(tmp_path):
    """Truncation stages, penalties and Mirostat through generate() and the scheduler (CPU
    stand-in kernels), with few pages under the optimistic policy, so that a preempted request
    is recomputed and its Mirostat state and history carry on: against the plain implementation
    run on each request alone."""
    from leone_b200.engine.engine import Engine
    from leone_b200.engine.generate import generate
    from leone_b200.sampling.sampler import Penalties
    from tests import replay
    from tests.emulated_ops import EmulatedOps
    from tests.plain.model import PlainModel, generate as plain_generate
    from tests.tiny import PAGE_TOKENS, make_folder
    folder = make_folder(tmp_path, "B")
    plain = PlainModel(folder)
    prompts = [replay.random_tokens(plain.cfg["vocab_size"], n, 90 + n) for n in (2, 9, 16)]
    stages = (("top_k", 20), ("typical", 0.9), ("min_p", 0.02))
    pen = dict(repetition=1.2, presence=0.1, window=16, dry_multiplier=0.6)
    cases = [dict(truncations=stages), dict(penalties=pen), dict(mirostat=(2.5, 0.3)),
             dict(truncations=stages, penalties=pen, mirostat=(1.5, 0.5))]
    for case in cases:
        want = [plain_generate(plain, p, 7, 0.9, 30 + i, **case) for i, p in enumerate(prompts)]
        product = dict(case)
        if "penalties" in product:
            product["penalties"] = Penalties(**pen)
        for policy, pages in (("reserve", 12), ("optimistic", 7)):
            eng = Engine.from_folder(folder, dtype="float32", device="cpu", ops=EmulatedOps(),
                                     page_tokens=PAGE_TOKENS["B"], num_pages=pages, max_requests=3,
                                     max_batch_tokens=16)
            got = generate(eng, prompts, 7, temperature=0.9, seed=30, prefill_chunk=6, max_batch_tokens=16,
                           policy=policy, eos_token_id=-1, prefill_first=False, **product)
            assert got == want, (sorted(case), policy)
            assert eng.cache.free_pages()[0] == pages
    # greedy takes no notice of truncation stages; penalties still apply to it
    want = [plain_generate(plain, p, 5, 0.0, 0, penalties=pen) for p in prompts]
    eng = Engine.from_folder(folder, dtype="float32", device="cpu", ops=EmulatedOps(), page_tokens=PAGE_TOKENS["B"],
                             num_pages=12, max_requests=3, max_batch_tokens=16)
    assert generate(eng, prompts, 5, eos_token_id=-1, truncations=stages, penalties=Penalties(**pen)) == want


def test_a_finished_request_can_be_forgotten():
    eng = FakeEngine(pages=16)
    s = Scheduler(eng, SchedulerConfig())
    s.add_request("a", [1, 2, 3], 2)
    s.add_request("b", [4], 50)
    assert s.forget("a") is None                    # still in flight
    while s.requests["a"].state != "finished":
        s.step()
    done = s.forget("a")
    assert done.generated == alone([1, 2, 3], 2) and "a" not in s.requests and s.forget("a") is None
    s.add_request("a", [9], 1)                      # the name is free again
    s.cancel("b")
    _run(s)
    assert s.forget("b").state == "cancelled" and s.requests["a"].generated == alone([9], 1)

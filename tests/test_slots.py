"""The per-request slot record: what it holds, who writes it, and that it goes with the slot."""
import pytest
import torch

from leone_b200.cache.slots import SlotRecords
from leone_b200.engine.engine import Engine
from leone_b200.engine.scheduler import Scheduler, SchedulerConfig
from leone_b200.sampling.sampler import SamplingParams
from tests.tiny import make_folder


def test_a_record_holds_what_was_written_and_starts_from_zero():
    rec = SlotRecords(4, "cpu")
    rec.open(2)
    assert rec.record(2) == dict(length=0, position=0, seed=0, temperature=0.0, last_token=0, cancel_requested=False,
                                 live=True, status=0, sampler=0.0)
    rec.set_sampling(2, (1 << 64) - 3, 0.8)
    rec.set_progress(2, 17, 16, 99)
    rec.set_sampler_state(2, 4.25)
    rec.request_cancel(2)
    got = rec.record(2)
    assert got["seed"] == (1 << 64) - 3 and abs(got["temperature"] - 0.8) < 1e-7 and got["sampler"] == 4.25
    assert (got["length"], got["position"], got["last_token"], got["cancel_requested"]) == (17, 16, 99, True)
    assert not rec.is_live(1)
    rec.sync()
    assert rec.read_device(2)["position"] == 16 and rec.read_device(2)["flags"] == 3
    rec.close(2)
    rec.open(2)                                           # the slot's next owner sees nothing of the last
    assert rec.record(2)["seed"] == 0 and not rec.cancel_requested(2)
    rec.sync()
    assert rec.read_device(2)["last_token"] == 0


def test_the_scheduler_keeps_each_running_request_in_its_slot_record(tmp_path):
    from tests.emulated_ops import EmulatedOps
    eng = Engine.from_folder(make_folder(tmp_path, "A"), dtype="float32", device="cpu", ops=EmulatedOps(),
                             page_tokens=4, num_pages=24, max_requests=3, max_batch_tokens=32)
    s = Scheduler(eng, SchedulerConfig(max_running=3, prefill_chunk_tokens=4, use_graphs=False))
    s.add_request("a", [1, 2, 3, 4, 5, 6], 5, SamplingParams(0.7, 41), -1)
    s.add_request("b", [9, 8], 5, SamplingParams(0.0, 5, mirostat=None), -1)
    s.step()
    a, b = s.requests["a"], s.requests["b"]
    assert a.slot is not None and a.slot != b.slot
    ra = eng.slot_records.record(a.slot)
    assert ra["live"] and ra["seed"] == 41 and abs(ra["temperature"] - 0.7) < 1e-7
    s.step()
    s.step()
    rb = eng.slot_records.record(b.slot)
    assert rb["length"] == b.computed and rb["last_token"] == b.tokens[-1] and rb["position"] == len(b.tokens) - 1
    s.cancel("a")
    assert eng.slot_records.cancel_requested(a.slot)
    slot_a = a.slot
    s.step()                                               # the cancelled request leaves at the step's start
    assert a.state == "cancelled" and a.slot is None and not eng.slot_records.is_live(slot_a)
    s.run_to_completion()
    assert all(not eng.slot_records.is_live(i) for i in range(3))
    assert eng.cache.slots.num_free == 3


@pytest.mark.gpu
def test_the_captured_decode_step_samples_from_and_advances_the_slot_records(tmp_path):
    """Temperature sampling through captured decode steps: the tokens are the plain sampler's,
    and afterwards each request's device record stands where the request stands."""
    from tests import replay
    from tests.plain.model import PlainModel, generate as plain_generate
    folder = make_folder(tmp_path, "B")
    plain = PlainModel(folder)
    eng = Engine.from_folder(folder, dtype="float32", page_tokens=8, max_tokens=256, max_requests=4, max_batch_tokens=64)
    prompts = [replay.random_tokens(384, n, 30 + n) for n in (5, 12)]
    params = [SamplingParams(0.9, 100 + i) for i in range(2)]
    want = [plain_generate(plain, p, 7, 0.9, 100 + i) for i, p in enumerate(prompts)]
    firsts = []
    for i, p in enumerate(prompts):
        logits = eng.step([(i, p, [len(p) - 1])])
        firsts.append(eng.sample(logits, [params[i]], [len(p) - 1])[0])
    toks = eng.decode_steps([0, 1], firsts, params, 4)            # a quantum
    toks += eng.decode_steps([0, 1], toks[-1], params, 1)         # single steps (one launched ahead)
    toks += eng.decode_steps([0, 1], toks[-1], params, 1)
    got = [[firsts[i]] + [row[i] for row in toks] for i in range(2)]
    assert got == want
    eng.drop_lookahead()
    torch.cuda.synchronize()
    for i, p in enumerate(prompts):
        rec = eng.slot_records.read_device(eng.cache.slot(i))
        assert rec["seed"] == 100 + i and abs(rec["temperature"] - 0.9) < 1e-6
        # a dropped look-ahead step may have moved the device copy one token further
        assert rec["length"] - eng.length(i) in (0, 1) and rec["position"] == rec["length"]

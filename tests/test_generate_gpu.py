"""Generation through the Python entry point on the GPU against the plain implementation."""
import pytest
import torch

from tests import replay
from tests.plain.model import PlainModel, generate as plain_generate
from tests.tiny import PAGE_TOKENS, make_folder

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("gen_models")
    return {w: make_folder(base, w) for w in "ABC"}


def _engine(folder, which, dtype, pages, **kw):
    from leone_b200.engine.engine import Engine
    return Engine.from_folder(folder, dtype=dtype, page_tokens=PAGE_TOKENS[which], num_pages=pages,
                              max_requests=4, max_batch_tokens=64, **kw)


def test_greedy_three_requests_fp32(folders):
    """Tiny A: prompts of 5/9/13 tokens, 8 new tokens each, greedy."""
    from leone_b200 import generate
    plain = PlainModel(folders["A"])
    prompts = [replay.random_tokens(256, n, 50 + n) for n in (5, 9, 13)]
    want = [plain_generate(plain, p, 8) for p in prompts]
    got = generate(folders["A"], prompts, 8, dtype="float32", page_tokens=4, eos_token_id=-1)
    assert got == want


@pytest.mark.parametrize("policy,pages", [("reserve", 14), ("optimistic", 9)])
@pytest.mark.parametrize("quantum", [1, 4])
def test_temperature_chunked_mixed_fp32(folders, policy, pages, quantum):
    """Tiny B: prompts of 1/7/17/30, prefill portions of 6 mixed with decode, 6 new tokens,
    temperature 0.8 with per-request seeds; few pages, both page policies."""
    from leone_b200 import generate
    plain = PlainModel(folders["B"])
    prompts = [replay.random_tokens(384, n, 60 + n) for n in (1, 7, 17, 30)]
    want = [plain_generate(plain, p, 6, 0.8, 7 + i) for i, p in enumerate(prompts)]
    eng = _engine(folders["B"], "B", "float32", pages)
    got, stats = generate(eng, prompts, 6, temperature=0.8, seed=7, prefill_chunk=6, max_batch_tokens=16,
                          policy=policy, return_stats=True, eos_token_id=-1, decode_quantum=quantum,
                          prefill_first=False)
    assert got == want
    if policy == "optimistic":
        assert stats.preemptions > 0
    eng.cache.check_invariants()
    assert eng.cache.free_pages()[0] == pages


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_greedy_bf16_stays_within_rounding(folders, which):
    from leone_b200 import generate
    plain = PlainModel(folders[which], matrices_as_bf16=True)
    vocab = plain.cfg["vocab_size"]
    prompts = [replay.random_tokens(vocab, n, 70 + n) for n in (3, 11, 24)]
    got = generate(folders[which], prompts, 8, dtype="bfloat16", page_tokens=PAGE_TOKENS[which],
                   eos_token_id=-1)
    for p, toks in zip(prompts, got):
        assert len(toks) == 8
        seq = list(p)
        for t in toks:
            logits = plain.logits(seq)[-1]
            assert float(logits.max() - logits[t]) <= 0.025 * float(logits.abs().max())
            seq.append(t)


def test_graph_decode_equals_eager_decode(folders):
    from leone_b200 import generate
    prompts = [replay.random_tokens(331, n, 80 + n) for n in (4, 19, 33, 8)]
    for dtype in ("float32", "bfloat16"):
        outs = []
        for kw in (dict(use_graphs=False), dict(use_graphs=True, decode_quantum=1),
                   dict(use_graphs=True, decode_quantum=5)):
            eng = _engine(folders["C"], "C", dtype, 40)
            outs.append(generate(eng, prompts, 12, temperature=0.7, seed=3, eos_token_id=-1, **kw))
        assert outs[0] == outs[1] == outs[2], dtype


def test_eos_stops_a_request(folders):
    from leone_b200 import generate
    plain = PlainModel(folders["A"])
    prompt = replay.random_tokens(256, 6, 5)
    free_run = plain_generate(plain, prompt, 8)
    eos = free_run[3]
    got = generate(folders["A"], [prompt], 8, dtype="float32", page_tokens=4, eos_token_id=eos)
    assert got[0] == free_run[:free_run.index(eos) + 1]


def test_a_captured_graph_survives_growth_of_the_scratch_buffers(folders):
    """A decode graph keeps the addresses of the split scratch it was captured with.  A later,
    larger batch outgrows that scratch; the small batch's graph must still be usable."""
    from leone_b200 import generate
    eng = _engine(folders["C"], "C", "bfloat16", 200)
    eng.ops.fast.min_scratch_floats = 1            # every growth reallocates
    eng.ops.fast.use_clusters = False              # the paths that keep partial results in scratch
    eng.ops.fast.force_decode_splits = 3           # ... whatever the dispatcher would choose here
    small = [replay.random_tokens(331, n, 90 + n) for n in (150, 140)]
    large = [replay.random_tokens(331, 150, 200 + i) for i in range(4)]
    first = generate(eng, small, 6, eos_token_id=-1)
    generate(eng, large, 6, eos_token_id=-1)       # larger batch: more scratch
    torch.cuda.empty_cache()
    again = generate(eng, small, 6, eos_token_id=-1)
    torch.cuda.synchronize()
    assert first == again
    assert len(eng.ops.fast._retired) > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing(folders, dtype):
    """A decode step launched before the step before it has been read: the same tokens as
    without, with requests that end at different steps (by length and by a stop token, so
    steps launched ahead are thrown away), few pages (new pages arrive while a step is in
    flight), and another step of the engine between two decode steps."""
    from leone_b200 import generate
    from leone_b200.sampling.sampler import SamplingParams
    prompts = [replay.random_tokens(331, n, 300 + n) for n in (5, 21, 34, 9)]
    outs, ahead_seen = [], []
    for lookahead in (False, True):
        eng = _engine(folders["C"], "C", dtype, 30)
        eng.lookahead = lookahead
        free = generate(eng, prompts, 40, temperature=0.9, seed=11, eos_token_id=-1)
        stop = free[1][17]                                # request 1 (and whoever else draws it) ends early
        got = generate(eng, prompts, 40, temperature=0.9, seed=11, eos_token_id=stop)
        assert got[1] == free[1][:free[1].index(stop) + 1]
        outs.append((free, got))
        assert eng.cache.free_pages() == [eng.num_pages] and eng._ahead is None
        # the engine's own interface: three decode steps, a prompt step of another request
        # in between, then more decode steps
        rids = ["p", "q"]
        firsts = []
        for r, p in zip(rids, prompts[:2]):
            logits = eng.step([(r, p, [len(p) - 1])])
            firsts.append(eng.sample(logits, [SamplingParams()], [len(p) - 1])[0])
        params = [SamplingParams(0.8, 5), SamplingParams(0.0, 0)]
        seq, last = [], firsts
        for i in range(9):
            if i == 3:
                eng.step([("other", prompts[2], [])])
            last = eng.decode_steps(rids, last, params, 1)[0]
            if i in (0, 4):
                ahead_seen.append(eng._ahead is not None)
            seq.append(last)
        outs.append(seq)
        for r in rids + ["other"]:
            eng.close(r)
        assert eng.cache.free_pages() == [eng.num_pages]
        eng.cache.check_invariants()
    assert outs[0] == outs[2] and outs[1] == outs[3]
    assert ahead_seen == [False, False, True, True]


def test_generation_with_truncation_stages(folders):
    """Temperature with top-k, top-p and min-p, and a pipeline with typical, through the entry
    point against the plain implementation; other requests of the batch sample without."""
    from leone_b200 import generate
    plain = PlainModel(folders["B"])
    prompts = [replay.random_tokens(384, n, 400 + n) for n in (3, 11, 20)]
    for stages in ((("top_k", 12), ("top_p", 0.9), ("min_p", 0.02)), (("top_n_sigma", 1.5), ("typical", 0.8))):
        want = [plain_generate(plain, p, 7, temperature=1.1, seed=21 + i, truncations=stages)
                for i, p in enumerate(prompts)]
        got = generate(folders["B"], prompts, 7, temperature=1.1, seed=21, dtype="float32", page_tokens=8,
                       eos_token_id=-1, truncations=stages)
        assert got == want
        unrestricted = generate(folders["B"], prompts, 7, temperature=1.1, seed=21, dtype="float32",
                                page_tokens=8, eos_token_id=-1)
        assert unrestricted != got


def test_generation_with_penalties(folders):
    """Greedy and temperature generation with repetition, frequency and repeated-suffix penalties
    over each request's own history, against the plain implementation; a prompt that repeats
    itself, so that the penalties bite from the first token."""
    from leone_b200 import generate
    from leone_b200.sampling.sampler import Penalties
    plain = PlainModel(folders["A"])
    base = replay.random_tokens(256, 6, 77)
    prompts = [base + base + base[:3], replay.random_tokens(256, 9, 78)]
    kw = dict(repetition=1.4, frequency=0.3, window=32, dry_multiplier=1.5, dry_allowed_length=2)
    for temperature in (0.0, 0.9):
        want = [plain_generate(plain, p, 10, temperature=temperature, seed=5 + i, penalties=kw)
                for i, p in enumerate(prompts)]
        got = generate(folders["A"], prompts, 10, temperature=temperature, seed=5, dtype="float32", page_tokens=4,
                       eos_token_id=-1, penalties=Penalties(**kw))
        assert got == want
        free = generate(folders["A"], prompts, 10, temperature=temperature, seed=5, dtype="float32", page_tokens=4,
                        eos_token_id=-1)
        assert free != got


def test_generation_with_mirostat(folders):
    """Mirostat v2 with and without truncation stages and penalties through the entry point:
    every request's maximum surprise follows its own tokens."""
    from leone_b200 import generate
    from leone_b200.sampling.sampler import Penalties
    plain = PlainModel(folders["B"])
    prompts = [replay.random_tokens(384, n, 500 + n) for n in (4, 13)]
    pen = dict(frequency=0.2, window=8)
    for case in (dict(mirostat=(3.0, 0.4)), dict(mirostat=(1.0, 1.0), truncations=(("top_p", 0.95),), penalties=pen)):
        want = [plain_generate(plain, p, 9, temperature=1.0, seed=40 + i, **case) for i, p in enumerate(prompts)]
        product = dict(case)
        if "penalties" in product:
            product["penalties"] = Penalties(**pen)
        got = generate(folders["B"], prompts, 9, temperature=1.0, seed=40, dtype="float32", page_tokens=8,
                       eos_token_id=-1, **product)
        assert got == want

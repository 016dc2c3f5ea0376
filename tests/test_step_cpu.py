"""The step function and cache on the CPU stand-in kernels, in every way of cutting the work."""
import pytest
import torch

from leone_b200.cache.pages import OutOfPages
from leone_b200.engine.engine import Engine
from tests import replay
from tests.emulated_ops import EmulatedOps
from tests.plain.model import PlainModel
from tests.tiny import PAGE_TOKENS, make_folder


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    base = tmp_path_factory.mktemp("cpu_models")
    folders = {w: make_folder(base, w) for w in "ABC"}
    return folders, {w: PlainModel(f) for w, f in folders.items()}


@pytest.mark.parametrize("which", ["A", "B", "C"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_every_cut_gives_the_plain_logits(setup, which, mode):
    folders, plains = setup
    plain = plains[which]
    reqs = {f"r{i}": replay.random_tokens(plain.cfg["vocab_size"], n, i) for i, n in enumerate([40, 7, 75, 33, 1, 50])}
    steps = {"whole": replay.trace_whole, "tail": replay.trace_decode_tail,
             "portions": replay.trace_portions, "mixed": replay.trace_mixed}[mode](reqs)
    eng = Engine.from_folder(folders[which], dtype="float32", device="cpu", ops=EmulatedOps(),
                             page_tokens=PAGE_TOKENS[which], max_tokens=replay.max_live_tokens(steps),
                             max_requests=8, max_batch_tokens=128)
    out = replay.run_trace_engine(eng, steps)
    replay.compare(steps, out, plain, reqs, 1e-5, 1e-5, f"{which}/{mode}")
    assert eng.cache.free_pages()[0] == eng.num_pages


def test_a_step_that_does_not_fit_changes_nothing(setup):
    folders, _ = setup
    eng = Engine.from_folder(folders["A"], dtype="float32", device="cpu", ops=EmulatedOps(),
                             page_tokens=4, num_pages=4, max_requests=3, max_batch_tokens=64)
    eng.step([("a", [1, 2, 3, 4, 5], [])])
    free = eng.cache.free_pages()
    with pytest.raises(OutOfPages):
        eng.step([("a", [6], [0]), ("b", list(range(1, 12)), [])])
    assert eng.cache.free_pages() == free and eng.length("a") == 5 and not eng.cache.is_open("b")
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step([("a", [999], [0])])
    big = Engine.from_folder(folders["A"], dtype="float32", device="cpu", ops=EmulatedOps(),
                             page_tokens=4, num_pages=40, max_requests=2, max_batch_tokens=64)
    big.step([("c", [1] * 64, [])])
    big.step([("c", [1] * 64, [])])
    with pytest.raises(ValueError, match="positions"):
        big.step([("c", [1], [])])
    with pytest.raises(ValueError, match="twice"):
        eng.step([("a", [1], []), ("a", [2], [])])
    eng.cache.check_invariants()


def test_run_order_may_repeat_a_layer_and_borrow_a_cache(setup, tmp_path):
    """Layer order is data: run a layer twice, and let one layer read another's cache."""
    from dataclasses import replace
    from leone_b200.config.qwen3 import Qwen3Config
    from leone_b200.registry import spec_from_config
    from leone_b200.weights.random_init import random_tensors
    from leone_b200.engine.model import weight_specs_for_config
    from tests.tiny import TINY_B
    cfg = Qwen3Config.from_dict(TINY_B)
    spec = spec_from_config(cfg)
    layers = tuple(replace(l, cache_of=0) if i == 2 else l for i, l in enumerate(spec.layers))
    spec2 = replace(spec, layers=layers, run_order=(0, 1, 1, 2))
    tensors = random_tensors(weight_specs_for_config(cfg), 3)
    toks = replay.random_tokens(384, 21, 1)

    def run(cuts):
        eng = Engine(spec2, dict(tensors), dtype="float32", device="cpu", ops=EmulatedOps(),
                     page_tokens=8, num_pages=8, max_requests=2, max_batch_tokens=32)
        assert len(eng.cache.groups[0].spec.layers) == 3       # three runs own a cache; layer 2 borrows
        outs, pos = [], 0
        for c in cuts:
            outs.append(eng.step([("x", toks[pos:pos + c], list(range(c)))]))
            pos += c
        return torch.cat(outs)

    whole, cut = run([21]), run([5, 2, 13, 1])
    assert torch.allclose(whole, cut, rtol=1e-5, atol=1e-6)
    plain_order = Engine(replace(spec, run_order=(0, 1, 2)), dict(tensors), dtype="float32", device="cpu",
                         ops=EmulatedOps(), page_tokens=8, num_pages=8, max_requests=2, max_batch_tokens=32)
    assert not torch.allclose(whole, plain_order.step([("x", toks, list(range(21)))]), atol=1e-4)


@pytest.mark.parametrize("seed", range(4))
def test_step_metadata_layout_against_a_plain_restatement(seed):
    """The packed int32 array of a step, field by field, against numpy written out here."""
    import numpy as np
    from leone_b200.engine.batch import pack_metadata
    rng = np.random.default_rng(seed)
    b = int(rng.integers(1, 5))
    token_lists = [list(rng.integers(0, 1000, int(rng.integers(1, 9)))) for _ in range(b)]
    starts = [int(rng.integers(0, 50)) for _ in range(b)]
    slots = list(rng.permutation(8)[:b])
    wants = [sorted(set(int(j) for j in rng.integers(0, len(t), int(rng.integers(0, 3))))) for t in token_lists]
    tables = [rng.integers(-1, 30, (b, 3 + g)).astype(np.int32) for g in range(2)]
    packed, offsets, bt_offsets, stats = pack_metadata(token_lists, starts, slots, wants, tables)

    def field(name):
        o, s = offsets[name]
        return packed[o:o + s].tolist()

    q_start = [0]
    for t in token_lists:
        q_start.append(q_start[-1] + len(t))
    assert field("token_ids") == [x for t in token_lists for x in t]
    assert field("positions") == [starts[i] + j for i, t in enumerate(token_lists) for j in range(len(t))]
    assert field("seq_of_token") == [i for i, t in enumerate(token_lists) for _ in t]
    assert field("q_start") == q_start
    assert field("ctx_len") == [starts[i] + len(t) for i, t in enumerate(token_lists)]
    assert field("slot_ids") == [int(s) for s in slots]
    assert field("logit_rows") == [q_start[i] + j for i, w in enumerate(wants) for j in w]
    for (o, shape), bt in zip(bt_offsets, tables):
        assert (packed[o:o + bt.size].reshape(shape) == bt).all()
    assert stats["n"] == q_start[-1] and stats["m"] == sum(len(w) for w in wants)
    with pytest.raises(ValueError, match="outside"):
        pack_metadata(token_lists, starts, slots, [[len(token_lists[0])]] + [[]] * (b - 1), tables)

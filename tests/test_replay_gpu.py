"""Replay on the GPU against the plain implementation: whole, decoded tail, portions, mixed;
in 32-bit and in bfloat16; through the engine in-process and through bin/trace_run."""
import os

import pytest
import torch

from tests import replay
from tests.plain.model import PlainModel
from tests.tiny import PAGE_TOKENS, make_folder

pytestmark = pytest.mark.gpu

FP32_TOL = dict(zip(("rtol", "atol_scale"), replay.FP32_TOL))
BF16_TOL = dict(zip(("rtol", "atol_scale"), replay.BF16_TOL))
LENGTHS = [40, 7, 75, 33, 1, 64, 50]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {w: make_folder(base, w) for w in "ABCD"}


@pytest.fixture(scope="module")
def plains(folders):
    return {(w, bf): PlainModel(folders[w], matrices_as_bf16=bf) for w in "ABCD" for bf in (False, True)}


def _requests(vocab, lengths=LENGTHS):
    return {f"r{i}": replay.random_tokens(vocab, n, 100 + i) for i, n in enumerate(lengths)}


def _traces(reqs):
    return {"whole": replay.trace_whole(reqs), "tail": replay.trace_decode_tail(reqs),
            "portions": replay.trace_portions(reqs), "mixed": replay.trace_mixed(reqs, seed=3)}


@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_in_process(folders, plains, which, dtype, mode):
    from leone_b200.engine.engine import Engine
    plain = plains[(which, dtype == "bfloat16")]
    reqs = _requests(plain.cfg["vocab_size"])
    steps = _traces(reqs)[mode]
    pool = replay.max_live_tokens(steps)
    engine = Engine.from_folder(folders[which], dtype=dtype, page_tokens=PAGE_TOKENS[which],
                                max_tokens=pool, max_requests=8, max_batch_tokens=128)
    out = replay.run_trace_engine(engine, steps)
    tol = FP32_TOL if dtype == "float32" else BF16_TOL
    worst = replay.compare(steps, out, plain, reqs, what=f"{which}/{dtype}/{mode}", **tol)
    replay.check_worst(("tiny", which, dtype, mode), worst)
    if mode == "mixed":
        pool_pages = engine.cache.groups[0].pool
        total_blocks = sum(-(-len(t) // engine.page_tokens) for t in reqs.values())
        assert total_blocks > pool_pages.num_pages, "the trace must force pages to be used again"
    assert engine.cache.groups[0].pool.num_free == engine.num_pages


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "float32")])
def test_replay_program(folders, plains, which, dtype, tmp_path):
    """bin/trace_run as a child process with its default page size."""
    plain = plains[(which, dtype == "bfloat16")]
    reqs = _requests(plain.cfg["vocab_size"], [40, 75, 33, 64, 50, 9])
    tol = FP32_TOL if dtype == "float32" else BF16_TOL
    for mode, steps in _traces(reqs).items():
        out_dir = os.path.join(str(tmp_path), mode)
        out = replay.run_trace_program(folders[which], dtype, steps, out_dir, replay.max_live_tokens(steps))
        replay.compare(steps, out, plain, reqs, what=f"trace_run {which}/{dtype}/{mode}", **tol)


@pytest.mark.parametrize("which", ["A", "C"])
def test_page_size_does_not_change_fp32_logits(folders, which):
    from leone_b200.engine.engine import Engine
    import numpy as np
    cfg_vocab = PlainModel(folders[which]).cfg["vocab_size"]
    reqs = _requests(cfg_vocab, [50, 21, 64])
    steps = replay.trace_mixed(reqs, seed=5)
    outs = []
    for pt in (4, 16, 64):
        engine = Engine.from_folder(folders[which], dtype="float32", page_tokens=pt,
                                    max_tokens=replay.max_live_tokens(steps), max_requests=8,
                                    max_batch_tokens=128)
        outs.append(replay.run_trace_engine(engine, steps))
    for k in outs[0]:
        assert np.array_equal(outs[0][k], outs[1][k]) and np.array_equal(outs[0][k], outs[2][k])


def test_first_tokens_and_long_decode(folders, plains):
    """Position 0 alone, then a long run of single-token steps across many pages."""
    from leone_b200.engine.engine import Engine
    for dtype, tol in (("float32", FP32_TOL), ("bfloat16", BF16_TOL)):
        plain = plains[("C", dtype == "bfloat16")]
        reqs = {"long": replay.random_tokens(plain.cfg["vocab_size"], 300, 77)}
        steps = replay.trace_decode_tail(reqs, tail=299)
        engine = Engine.from_folder(folders["C"], dtype=dtype, page_tokens=16, max_tokens=320,
                                    max_requests=2, max_batch_tokens=64)
        out = replay.run_trace_engine(engine, steps)
        replay.compare(steps, out, plain, reqs, what=f"long decode {dtype}", **tol)

"""Parts defined outside the framework are registered, built and stepped without touching it:
a mixer with per-request state, a feed-forward that routes tokens to experts, an unfused position
encoding, a windowed attention layer with partial rotary; three different mixers and two different
feed-forwards in three layers.  A second toy adds an embedding with a multiplier and learned
positions, a mixer whose paged cache holds one latent vector per token (its own width, no values,
its own dtype) and a tied head with a logit scale and a soft cap.  Both also run through the
scheduler with captured decode steps."""
import pytest
import torch

from leone_b200.engine.engine import Engine
from leone_b200.engine.model import Model
from leone_b200.parts.base import Runtime
from leone_b200.registry import config_from_dict, spec_from_config
from leone_b200.weights.random_init import random_tensors
from tests import replay, toy_parts


@pytest.fixture()
def toy():
    toy_parts.register()
    cfg = config_from_dict(toy_parts.TOY)
    spec = spec_from_config(cfg)
    specs = Model(spec, Runtime("cpu", torch.float32, None, 0)).weight_specs()
    tensors = random_tensors(specs, 11)
    for name in tensors:                                   # larger weights so every part matters
        if tensors[name].dim() == 2:
            tensors[name] = tensors[name] * 5
    yield cfg, spec, tensors
    toy_parts.unregister()


def _check(cfg, spec, tensors, device, ops, dtype, tol):
    reqs = {"a": replay.random_tokens(97, 45, 1), "b": replay.random_tokens(97, 30, 2),
            "c": replay.random_tokens(97, 17, 3)}
    want = {r: toy_parts.plain_logits(cfg, tensors if dtype == "float32" else
                                      {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in tensors.items()},
                                      t) for r, t in reqs.items()}

    class Plain:
        def logits(self, tokens):
            return want[[r for r, t in reqs.items() if t == list(tokens)][0]]

    for name, steps in (("whole", replay.trace_whole(reqs)), ("portions", replay.trace_portions(reqs)),
                        ("mixed", replay.trace_mixed(reqs, seed=2, max_live=3))):
        eng = Engine(spec, dict(tensors), dtype=dtype, device=device, ops=ops() if ops else None,
                     page_tokens=8, max_tokens=replay.max_live_tokens(steps), max_requests=3,
                     max_batch_tokens=64)
        kinds = sorted(g.spec.kind for g in eng.cache.groups)
        assert kinds == ["full", "window"] and len(eng._run_state) == 1
        out = replay.run_trace_engine(eng, steps)
        replay.compare(steps, out, Plain(), reqs, what=f"toy {name} {dtype}", **tol)
        assert eng.cache.free_pages() == [eng.num_pages] * 2


def test_toy_architecture_on_stand_in_kernels(toy):
    from tests.emulated_ops import EmulatedOps
    _check(*toy, "cpu", EmulatedOps, "float32", dict(rtol=1e-5, atol_scale=1e-5))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("float32", dict(rtol=2e-5, atol_scale=2e-5)),
                                       ("bfloat16", dict(rtol=3e-2, atol_scale=3e-2))])
def test_toy_architecture_on_the_gpu(toy, dtype, tol):
    _check(*toy, "cuda:0", None, dtype, tol)


def test_a_failed_step_leaves_fixed_state_as_it_found_it(toy):
    """The step is a transaction for fixed-size state too: a step that fails after its kernels
    ran gives the pages back and puts the slots' state back."""
    from tests.emulated_ops import EmulatedOps
    cfg, spec, tensors = toy
    eng = Engine(spec, dict(tensors), dtype="float32", device="cpu", ops=EmulatedOps(), page_tokens=8, max_tokens=128,
                 max_requests=3, max_batch_tokens=64)
    tokens = replay.random_tokens(97, 20, 9)
    eng.step([("a", tokens[:7], []), ("b", tokens[:3], [])])
    before = {pos: st.clone() for pos, st in eng._run_state.items()}
    free = eng.cache.free_pages()
    forward = eng.model.forward

    def failing(ctx):
        forward(ctx)
        raise RuntimeError("a fault found after the kernels ran")

    eng.model.forward = failing
    with pytest.raises(RuntimeError, match="fault found"):
        eng.step([("a", tokens[7:12], [4]), ("c", tokens[:4], [])])
    eng.model.forward = forward
    assert all(torch.equal(st, before[pos]) for pos, st in eng._run_state.items())
    assert eng.cache.free_pages() == free and eng.length("a") == 7 and not eng.cache.is_open("c")
    # and the request goes on as if nothing had happened
    want = toy_parts.plain_logits(cfg, tensors, tokens[:12])[-1]
    got = eng.step([("a", tokens[7:12], [4])])[0].double()
    assert (got - want).abs().max().item() <= 1e-5 * want.abs().max().item()


# -- the second toy: embedding and head hooks, a cache of another shape ---------------------------
@pytest.fixture()
def latent_toy():
    toy_parts.register()
    cfg = config_from_dict({**toy_parts.TOY, "architectures": ["ToyLatentLM"]})
    spec = spec_from_config(cfg)
    specs = Model(spec, Runtime("cpu", torch.float32, None, 0)).weight_specs()
    tensors = random_tensors(specs, 12)
    for name in tensors:
        if tensors[name].dim() == 2:
            tensors[name] = tensors[name] * 5
    yield cfg, spec, tensors
    toy_parts.unregister()


def _rounded(tensors, dtype):
    if dtype == "float32":
        return tensors
    return {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for k, v in tensors.items()}


def _check_latent(cfg, spec, tensors, device, ops, dtype, tol):
    reqs = {"a": replay.random_tokens(97, 45, 4), "b": replay.random_tokens(97, 30, 5),
            "c": replay.random_tokens(97, 17, 6)}
    want = {r: toy_parts.plain_logits_latent(cfg, _rounded(tensors, dtype), t) for r, t in reqs.items()}

    class Plain:
        def logits(self, tokens):
            return want[[r for r, t in reqs.items() if t == list(tokens)][0]]

    for name, steps in (("whole", replay.trace_whole(reqs)), ("portions", replay.trace_portions(reqs)),
                        ("mixed", replay.trace_mixed(reqs, seed=4, max_live=3))):
        eng = Engine(spec, dict(tensors), dtype=dtype, device=device, ops=ops() if ops else None,
                     page_tokens=8, max_tokens=replay.max_live_tokens(steps), max_requests=3, max_batch_tokens=64)
        # the mixer's own cache: one group, keys of its width in its dtype, no value pool
        (group,) = eng.cache.groups
        k_pool, v_pool = eng.pools[0]
        assert (group.spec.kind, group.spec.tag) == ("full", "latent") and v_pool is None
        assert k_pool.dtype == torch.float32 and tuple(k_pool.shape) == (1, eng.num_pages, 1, 8, 20)
        assert eng.memory_plan["cache"] == k_pool.numel() * 4 and eng.memory_plan["state"] == 2 * 3 * 48 * 4
        out = replay.run_trace_engine(eng, steps)
        replay.compare(steps, out, Plain(), reqs, what=f"latent toy {name} {dtype}", **tol)
        assert eng.cache.free_pages() == [eng.num_pages]


def test_latent_toy_on_stand_in_kernels(latent_toy):
    from tests.emulated_ops import EmulatedOps
    _check_latent(*latent_toy, "cpu", EmulatedOps, "float32", dict(rtol=1e-5, atol_scale=1e-5))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("float32", dict(rtol=2e-5, atol_scale=2e-5)),
                                       ("bfloat16", dict(rtol=3e-2, atol_scale=3e-2))])
def test_latent_toy_on_the_gpu(latent_toy, dtype, tol):
    _check_latent(*latent_toy, "cuda:0", None, dtype, tol)


def _plain_greedy(logits_fn, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        out.append(int(torch.argmax(logits_fn(toks)[-1])))
        toks.append(out[-1])
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["state", "latent"])
@pytest.mark.parametrize("quantum", [1, 4])
def test_toys_through_the_scheduler_with_captured_decode_steps(toy, which, quantum):
    """Both toys generate through the scheduler with decode steps replayed from CUDA graphs:
    fixed-size state advanced inside a captured step, a window group, the routed feed-forward,
    the mixer with its own cache.  Prompts are mixed with decode rows (so some decode steps are
    eager mixed steps and others captured), in 32-bit against the plain implementations."""
    from leone_b200.engine.generate import generate
    if which == "state":
        cfg, spec, tensors = toy
        plain = lambda toks: toy_parts.plain_logits(cfg, tensors, toks)
    else:
        cfg = config_from_dict({**toy_parts.TOY, "architectures": ["ToyLatentLM"]})
        spec = spec_from_config(cfg)
        tensors = random_tensors(Model(spec, Runtime("cpu", torch.float32, None, 0)).weight_specs(), 12)
        tensors = {k: (v * 5 if v.dim() == 2 else v) for k, v in tensors.items()}
        plain = lambda toks: toy_parts.plain_logits_latent(cfg, tensors, toks)
    prompts = [replay.random_tokens(97, n, 20 + n) for n in (3, 14, 29)]
    want = [_plain_greedy(plain, p, 9) for p in prompts]
    for first in (True, False):
        eng = Engine(spec, dict(tensors), dtype="float32", page_tokens=8, max_tokens=3 * 64, max_requests=3,
                     max_batch_tokens=32)
        got = generate(eng, prompts, 9, eos_token_id=-1, prefill_chunk=8, max_batch_tokens=16, decode_quantum=quantum,
                       prefill_first=first)
        assert got == want, (which, quantum, first)
        assert eng._decode_graphs, "decode steps were expected to run from captured graphs"
        assert eng.cache.free_pages() == [eng.num_pages] * len(eng.cache.groups)


@pytest.mark.gpu
def test_no_step_is_launched_ahead_when_a_mixer_keeps_state(toy):
    """A decode step launched ahead and then dropped would have advanced the state mixer's slot
    for good.  With fixed-size state (or a window group) the engine does not look ahead, so a
    single step followed by something else leaves the state as an eager step leaves it."""
    from leone_b200.sampling.sampler import SamplingParams
    cfg, spec, tensors = toy
    prompt = replay.random_tokens(97, 12, 77)
    results = []
    for lookahead in (True, False):
        eng = Engine(spec, dict(tensors), dtype="float32", page_tokens=8, max_tokens=64, max_requests=2, max_batch_tokens=32)
        eng.lookahead = lookahead
        eng.step([("r", prompt[:-1], [])])
        toks = eng.decode_steps(["r"], [prompt[-1]], [SamplingParams()], 1, expect_more=True)
        assert eng._ahead is None
        state = [s.clone() for s in eng._run_state.values()]
        # something else comes instead of the expected next decode step
        logits = eng.step([("r", [toks[0][0], 5, 6], [2])])
        results.append((toks, [s.cpu() for s in state], logits.cpu()))
    assert results[0][0] == results[1][0]
    assert all(torch.equal(a, b) for a, b in zip(results[0][1], results[1][1]))
    assert torch.equal(results[0][2], results[1][2])


# -- the adjacent-pair rotary encoding in a whole model ------------------------------------------
def _adjacent_case(which):
    """A tiny configuration's own spec with its position encoding swapped for the adjacent-pair
    one, its random tensors, and the plain implementation told the same."""
    import dataclasses
    from leone_b200.parts.spec import PartSpec
    from tests import tiny
    from tests.plain import model as plain
    cfg = tiny.tiny_config(which)
    spec = spec_from_config(cfg)
    rope = spec.position_encodings["rope"]
    spec = dataclasses.replace(spec, position_encodings={"rope": PartSpec("rotary_adjacent", dict(rope.params))})
    tensors = random_tensors(Model(spec, Runtime("cpu", torch.float32, None, 0)).weight_specs(), 29)
    for name in tensors:
        if tensors[name].dim() == 2:
            tensors[name] = tensors[name] * 3
    plain_cfg = dict(tiny.CONFIGS[which], rope_pairing="adjacent")
    return spec, tensors, plain_cfg, plain


def _adjacent_check(which, device, ops, dtype, tol):
    spec, tensors, plain_cfg, plain = _adjacent_case(which)
    vocab = plain_cfg["vocab_size"]
    reqs = {"a": replay.random_tokens(vocab, 70, 1), "b": replay.random_tokens(vocab, 41, 2)}
    w = tensors if dtype == "float32" else {k: (v.to(torch.bfloat16).float() if v.dim() == 2 else v)
                                           for k, v in tensors.items()}
    want = {r: plain.forward_logits(plain_cfg, {k: v.double() for k, v in w.items()}, t) for r, t in reqs.items()}
    half = {r: plain.forward_logits(dict(plain_cfg, rope_pairing="half_split"),
                                    {k: v.double() for k, v in w.items()}, t) for r, t in reqs.items()}
    assert float((want["a"] - half["a"]).abs().max()) > 0.05 * float(want["a"].abs().max()), \
        "the two pairings must give different logits for the test to mean anything"

    class Plain:
        def logits(self, tokens):
            return want[[r for r, t in reqs.items() if t == list(tokens)][0]]

    for name, steps in (("tail", replay.trace_decode_tail(reqs, tail=24)), ("portions", replay.trace_portions(reqs)),
                        ("mixed", replay.trace_mixed(reqs, seed=4, max_live=2))):
        eng = Engine(spec, dict(tensors), dtype=dtype, device=device, ops=ops() if ops else None,
                     page_tokens=8, max_tokens=replay.max_live_tokens(steps), max_requests=2, max_batch_tokens=96)
        out = replay.run_trace_engine(eng, steps)
        replay.compare(steps, out, Plain(), reqs, what=f"adjacent rotary {which} {name} {dtype}", **tol)


def test_adjacent_pair_rotary_on_stand_in_kernels():
    from tests.emulated_ops import EmulatedOps
    _adjacent_check("C", "cpu", EmulatedOps, "float32", dict(rtol=1e-5, atol_scale=1e-5))


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["C", "D"])            # head size 48: the any-size kernels; 64: the fused ones
@pytest.mark.parametrize("dtype,tol", [("float32", dict(rtol=2e-5, atol_scale=2e-5)),
                                       ("bfloat16", dict(rtol=3e-2, atol_scale=3e-2))])
def test_adjacent_pair_rotary_on_the_gpu(which, dtype, tol):
    _adjacent_check(which, "cuda:0", None, dtype, tol)

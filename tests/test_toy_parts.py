"""Parts defined outside the framework are registered, built and stepped without touching it:
a mixer with per-request state, a feed-forward that routes tokens to experts, an unfused position
encoding, a windowed attention layer with partial rotary; three different mixers and two different
feed-forwards in three layers."""
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

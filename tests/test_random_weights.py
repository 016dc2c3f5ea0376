"""Seeded random weights: a function of (seed, tensor name, element index) that gives the same
bits from the host routine, from the device kernel and from the tests' own numpy restatement."""
import numpy as np
import pytest
import torch

from leone_b200.parts.base import WeightSpec
from leone_b200.weights.random_init import draw, tensor_key
from tests.plain import random_draw as plain_draw

SPECS = [WeightSpec("model.layers.3.self_attn.q_proj.weight", (257, 96)),
         WeightSpec("model.norm.weight", (1031,), role="norm", std=0.1),
         WeightSpec("model.embed_tokens.weight", (331, 80), role="embedding"),
         WeightSpec("bias_like", (77,), role="vector", std=0.5),
         WeightSpec("lookup", (5, 41), role="int_table")]


def _plain(spec, seed, **kw):
    return plain_draw.draw(seed, spec.name, spec.shape, spec.role, spec.std, **kw)


@pytest.mark.parametrize("spec", SPECS, ids=lambda s: s.role)
def test_host_draw_equals_the_numpy_restatement_bit_for_bit(spec):
    got = draw(spec, 11).numpy()
    want = _plain(spec, 11)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert np.array_equal(got.view(np.int32), want.view(np.int32))
    assert tensor_key(11, spec.name) == plain_draw.tensor_key(11, spec.name)


def test_a_slice_is_the_same_values_and_tensors_do_not_depend_on_each_other():
    spec = WeightSpec("w", (123, 457))
    whole = draw(spec, 3).view(-1)
    for start, count in ((0, 1), (999, 4097), (123 * 457 - 5, 5)):
        assert torch.equal(draw(spec, 3, start=start, count=count), whole[start:start + count])
    assert not torch.equal(draw(spec, 4).view(-1), whole)
    assert not torch.equal(draw(WeightSpec("w2", (123, 457)), 3).view(-1), whole)
    with pytest.raises(ValueError):
        draw(spec, 3, start=10, count=123 * 457)


def test_the_draw_is_normal_with_the_asked_mean_and_deviation():
    z = (draw(WeightSpec("big", (2048, 2048)), 9).double().view(-1)) / 0.02
    n = z.numel()
    assert abs(z.mean().item()) < 4 / n ** 0.5 and abs(z.std().item() - 1) < 4 / (2 * n) ** 0.5
    assert abs((z ** 3).mean().item()) < 0.02 and abs((z ** 4).mean().item() - 3) < 0.03
    for x, p in ((1.0, 0.6826894921), (2.0, 0.9544997361), (3.0, 0.9973002039)):
        assert abs((z.abs() < x).double().mean().item() - p) < 1e-3
    # neighbours are uncorrelated
    assert abs((z[:-1] * z[1:]).mean().item()) < 4 / n ** 0.5
    norm = draw(WeightSpec("n", (100000,), role="norm", std=0.1), 9).double()
    assert abs(norm.mean().item() - 1) < 2e-3 and abs(norm.std().item() - 0.1) < 1e-3
    table = draw(WeightSpec("t", (100000,), role="int_table"), 9)
    assert table.dtype == torch.int32 and 0 <= int(table.min()) and int(table.max()) < 1 << 15


def test_bfloat16_storage_is_the_fp32_value_rounded_to_nearest_even():
    spec = WeightSpec("w", (64, 100))
    assert torch.equal(draw(spec, 1, dtype=torch.bfloat16), draw(spec, 1).to(torch.bfloat16))


def test_a_written_folder_holds_the_drawn_values(tmp_path):
    from leone_b200.weights.safetensors import Checkpoint
    from tests.plain.model import PlainModel, read_folder
    from tests.tiny import CONFIGS, make_folder
    folder = make_folder(tmp_path, "B", seed=77)
    cfg, on_disk = read_folder(folder)
    from_seed = PlainModel.from_seed(CONFIGS["B"], 77)
    assert set(on_disk) == set(from_seed.w)
    for name, t in on_disk.items():
        assert torch.equal(t, from_seed.w[name]), name


@pytest.mark.gpu
@pytest.mark.parametrize("spec", SPECS + [WeightSpec("wide.weight", (3000, 4099))], ids=lambda s: s.name)
def test_device_draw_equals_host_draw_bit_for_bit(spec):
    for dtype in (None, torch.bfloat16):
        on_device = draw(spec, 21, "cuda:0", dtype).cpu()
        on_host = draw(spec, 21, "cpu", dtype)
        assert on_device.dtype == on_host.dtype
        assert torch.equal(on_device.view(torch.int16 if on_host.dtype == torch.bfloat16 else torch.int32),
                           on_host.view(torch.int16 if on_host.dtype == torch.bfloat16 else torch.int32))


@pytest.mark.gpu
def test_device_draw_of_a_large_tensor_matches_host_slices():
    """A tensor of the real vocabulary's size, checked on slices (the draw is per element)."""
    spec = WeightSpec("model.embed_tokens.weight", (151936, 4096), role="embedding")
    big = draw(spec, 5, "cuda:0", torch.bfloat16).view(-1)
    numel = big.numel()
    for start in (0, 12345677, numel // 2 + 3, numel - 70000):
        want = draw(spec, 5, "cpu", torch.bfloat16, start=start, count=70000)
        assert torch.equal(big[start:start + 70000].cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
def test_an_engine_from_a_seed_is_the_engine_from_the_written_folder(tmp_path):
    """``Engine.from_config(config, seed)`` and ``write_random_model(config, folder, seed)`` are one
    model: same logits bit for bit in 32-bit, and the plain implementation with weights from
    the tests' own restatement of the draw agrees with both."""
    from leone_b200.engine.engine import Engine
    from tests import replay
    from tests.plain.model import PlainModel
    from tests.tiny import CONFIGS, PAGE_TOKENS, make_folder, tiny_config
    for which in "AB":
        folder = make_folder(tmp_path, which, seed=31)
        kw = dict(dtype="float32", page_tokens=PAGE_TOKENS[which], max_tokens=128, max_requests=2, max_batch_tokens=64)
        a = Engine.from_folder(folder, **kw)
        b = Engine.from_config(tiny_config(which), 31, **kw)
        tokens = replay.random_tokens(CONFIGS[which]["vocab_size"], 37, 4)
        la = a.step([("r", tokens, list(range(37)))])
        lb = b.step([("r", tokens, list(range(37)))])
        assert torch.equal(la, lb)
        want = PlainModel.from_seed(CONFIGS[which], 31).logits(tokens)
        err = (la.double().cpu() - want).abs().max().item()
        assert err <= 3e-5 * want.abs().max().item(), err


@pytest.mark.gpu
def test_generate_with_random_weights_needs_no_tensor_file(tmp_path):
    import json
    from leone_b200 import generate
    from leone_b200.cli import main
    from tests import replay
    from tests.plain.model import PlainModel, generate as plain_generate
    from tests.tiny import CONFIGS, tiny_config
    cfg = CONFIGS["B"]
    prompts = [replay.random_tokens(cfg["vocab_size"], n, 90 + n) for n in (4, 19)]
    plain = PlainModel.from_seed(cfg, 13)
    want = [plain_generate(plain, p, 6) for p in prompts]
    assert generate(tiny_config("B"), prompts, 6, dtype="float32", page_tokens=8, random_weights=True,
                    weights_seed=13, eos_token_id=-1) == want
    assert generate(dict(cfg), prompts, 6, seed=13, dtype="float32", page_tokens=8, random_weights=True,
                    eos_token_id=-1) == want
    folder = tmp_path / "only_config"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    out = tmp_path / "tokens.json"
    code = main(["generate", "-m", str(folder), "--random-weights", "--weights-seed", "13", "--dtype", "float32",
                 "--page-tokens", "8", "-n", "6", "--eos", "-1", "--debug-tokens", str(out)]
                + sum([["-t", ",".join(map(str, p))] for p in prompts], []))
    assert code == 0 and json.loads(out.read_text()) == want

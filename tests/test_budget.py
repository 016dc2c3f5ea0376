"""The memory budget that is checked before any tensor is uploaded
(the reference's ``check_weight_budget``, crates/leone/src/model.rs:350-366)."""
import pytest
import torch

from leone_b200.engine.budget import WeightBudgetError
from leone_b200.engine.engine import Engine
from tests.emulated_ops import EmulatedOps
from tests.tiny import CONFIGS, make_folder, tiny_config


def _engine(free, **kw):
    args = dict(dtype="float32", device="cpu", ops=EmulatedOps(), page_tokens=4, num_pages=10, max_requests=3,
                max_batch_tokens=32, free_bytes=(lambda: free))
    args.update(kw)
    return Engine.from_config(tiny_config("A"), 1, **args)


def test_the_plan_counts_weights_cache_and_scratch():
    eng = _engine(1 << 40)
    cfg = CONFIGS["A"]
    h, i, d, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"], cfg["vocab_size"]
    nq, nkv, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["num_hidden_layers"]
    per_layer = (nq + 2 * nkv) * d * h + h * nq * d + 3 * i * h + 2 * d + 2 * h
    assert eng.memory_plan["weights"] == 4 * (v * h + layers * per_layer + h)          # tied head: no second table
    assert eng.memory_plan["cache"] == layers * 10 * 2 * (nkv * 4 * d) * 4
    assert eng.memory_plan["load"] == 4 * 2 * i * h                                   # gate and up beside their fused copy
    assert eng.memory_plan["scratch"] > 0 and eng.memory_plan["state"] == 0
    assert eng.memory_plan["required"] == sum(v_ for k, v_ in eng.memory_plan.items() if k != "required")


def test_a_model_that_does_not_fit_is_refused_before_anything_is_loaded(monkeypatch, tmp_path):
    need = _engine(1 << 40).memory_plan["required"]
    loaded = []
    monkeypatch.setattr(Engine, "_random_on_device", lambda self, specs, seed: loaded.append(1) or {})
    with pytest.raises(WeightBudgetError) as err:
        _engine(need - 1)
    assert err.value.required_bytes == need and err.value.available_bytes == need - 1 and not loaded
    assert "nothing was loaded" in str(err.value) and str(need) in str(err.value)
    # a larger pool is what tips it over: the pools count
    monkeypatch.undo()
    _engine(need)
    with pytest.raises(WeightBudgetError):
        _engine(need, num_pages=11)
    # from a folder the stored dtypes are read from the file's header, nothing else
    folder = make_folder(tmp_path, "A", store_dtype=torch.bfloat16)
    import leone_b200.engine.engine as engine_module
    monkeypatch.setattr(engine_module, "load_checkpoint", lambda *a, **k: loaded.append(2))
    with pytest.raises(WeightBudgetError):
        Engine.from_folder(folder, dtype="float32", device="cpu", ops=EmulatedOps(), page_tokens=4, num_pages=10,
                           max_requests=3, max_batch_tokens=32, free_bytes=lambda: 1000)
    assert not loaded


def test_without_a_figure_for_free_memory_nothing_is_checked():
    eng = Engine.from_config(tiny_config("A"), 1, dtype="float32", device="cpu", ops=EmulatedOps(), page_tokens=4,
                             num_pages=10, max_requests=3, max_batch_tokens=32)
    assert eng.memory_plan["required"] > 0


@pytest.mark.gpu
def test_a_too_large_pool_at_real_layer_sizes_is_refused_before_allocation():
    """The 32B layer shape with a pool of 400 GB: refused with the figures, and the device's
    memory is as it was."""
    from leone_b200.config.qwen3 import Qwen3Config
    cfg = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=5120, num_attention_heads=64,
        num_key_value_heads=8, head_dim=128, intermediate_size=25600, vocab_size=151936, rope_theta=1e6,
        rms_norm_eps=1e-6, max_position_embeddings=4096, tie_word_embeddings=False))
    torch.cuda.empty_cache()
    before = torch.cuda.memory_allocated()
    free = torch.cuda.mem_get_info()[0]
    per_page = 2 * 2 * 8 * 16 * 128 * 2                 # layers x (k, v) x heads x tokens x dims x bytes
    with pytest.raises(WeightBudgetError) as err:
        Engine.from_config(cfg, 1, dtype="bfloat16", page_tokens=16, num_pages=(400 << 30) // per_page,
                           max_requests=4, max_batch_tokens=256)
    assert err.value.plan["cache"] >= 399 << 30 and err.value.available_bytes <= free + (1 << 30)
    assert torch.cuda.memory_allocated() == before


@pytest.mark.gpu
def test_scratch_does_not_grow_with_the_number_of_distinct_step_sizes():
    """200 steps of 200 different sizes: after the first few, no step allocates anything."""
    from leone_b200.config.qwen3 import Qwen3Config
    cfg = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=1024, num_attention_heads=8,
        num_key_value_heads=2, head_dim=128, intermediate_size=2048, vocab_size=1000, rope_theta=1e6,
        rms_norm_eps=1e-6, max_position_embeddings=1024, tie_word_embeddings=True))
    eng = Engine.from_config(cfg, 1, dtype="bfloat16", page_tokens=16, max_tokens=1024, max_requests=2,
                             max_batch_tokens=640)
    sizes = list(range(1, 33)) + list(range(257, 425))          # the sizes whose products carry a folded norm
    assert len(set(sizes)) == 200
    seen = []
    for n in [640, 32, 300] + sizes:
        eng.step([("r", [1] * n, [n - 1])])
        eng.close("r")
        torch.cuda.synchronize()
        seen.append((torch.cuda.memory_allocated(), eng.rt.allocated_bytes()))
    assert len(set(seen[3:])) == 1, sorted(set(seen[3:]))

"""Configuration reading and the architecture registry."""
import json
import os

import pytest

from leone_b200.config.base import (ConfigError, InvalidValue, MissingKey, UnsupportedArchitecture,
                                    UnsupportedField, WrongType)
from leone_b200.config.qwen3 import Qwen3Config
from leone_b200.registry import ARCHITECTURES, config_from_dict, config_from_folder, spec_from_config
from tests.tiny import CONFIGS, TINY_A, TINY_B


def test_tiny_configs_differ_in_every_size_and_option():
    a, b = Qwen3Config.from_dict(TINY_A), Qwen3Config.from_dict(TINY_B)
    for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                "head_dim", "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps",
                "max_position_embeddings", "tie_word_embeddings"):
        assert getattr(a, key) != getattr(b, key), key
    assert b.num_attention_heads * b.head_dim != b.hidden_size


@pytest.mark.parametrize("which", list(CONFIGS))
def test_roundtrip_through_a_folder(tmp_path, which):
    cfg = Qwen3Config.from_dict(CONFIGS[which])
    cfg.write(str(tmp_path))
    assert config_from_folder(str(tmp_path)) == cfg


def test_defaults():
    raw = dict(TINY_A)
    del raw["num_key_value_heads"], raw["head_dim"], raw["tie_word_embeddings"]
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads
    assert cfg.tie_word_embeddings is False


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads",
                                 "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps",
                                 "max_position_embeddings"])
def test_missing_key(key):
    raw = dict(TINY_B)
    del raw[key]
    with pytest.raises(MissingKey, match=key):
        Qwen3Config.from_dict(raw)


@pytest.mark.parametrize("patch,error", [
    ({"hidden_size": "64"}, WrongType), ({"num_hidden_layers": 0}, InvalidValue),
    ({"num_hidden_layers": True}, WrongType), ({"rope_theta": float("inf")}, InvalidValue),
    ({"rms_norm_eps": -1e-6}, InvalidValue), ({"num_key_value_heads": 4}, InvalidValue),
    ({"head_dim": 15}, InvalidValue), ({"rope_scaling": {"type": "yarn", "factor": 4}}, UnsupportedField),
    ({"use_sliding_window": True}, UnsupportedField), ({"attention_bias": True}, UnsupportedField),
    ({"hidden_act": "gelu"}, UnsupportedField), ({"tie_word_embeddings": "yes"}, WrongType),
    ({"eos_token_id": 99999}, InvalidValue),
])
def test_rejections(patch, error):
    raw = {**TINY_B, **patch}
    with pytest.raises(error):
        Qwen3Config.from_dict(raw)


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(UnsupportedArchitecture, match="Qwen3ForCausalLM"):
        config_from_dict({**TINY_A, "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(MissingKey):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_bad_json(tmp_path):
    with open(os.path.join(str(tmp_path), "config.json"), "w") as fh:
        fh.write("{not json")
    with pytest.raises(ConfigError):
        config_from_folder(str(tmp_path))
    with pytest.raises(ConfigError):
        config_from_folder(os.path.join(str(tmp_path), "nowhere"))


def test_spec_is_built_from_the_configuration_only():
    cfg = Qwen3Config.from_dict(TINY_B)
    spec = spec_from_config(cfg)
    assert len(spec.layers) == 3 and spec.run_order == (0, 1, 2)
    assert spec.lm_head_name == "lm_head.weight"
    assert spec_from_config(Qwen3Config.from_dict(TINY_A)).lm_head_name is None
    m = spec.layers[1].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["qk_norm_eps"]) == (6, 3, 32, 1e-5)
    assert spec.position_encodings["rope"].params["theta"] == 1e6
    assert "Qwen3ForCausalLM" in ARCHITECTURES.names()


def test_run_order_and_borrowed_caches_are_checked():
    from dataclasses import replace
    cfg = Qwen3Config.from_dict(TINY_B)
    spec = spec_from_config(cfg)
    replace(spec, run_order=(0, 1, 1, 2)).validate()
    with pytest.raises(ValueError):
        replace(spec, run_order=(0, 5)).validate()
    borrowed = tuple(replace(l, cache_of=0) if i == 2 else l for i, l in enumerate(spec.layers))
    replace(spec, layers=borrowed).validate()
    with pytest.raises(ValueError, match="before"):
        replace(spec, layers=borrowed, run_order=(2, 0, 1)).validate()


def test_cli_truncation_flags_keep_their_order():
    """Stages apply in the order their flags are given (crates/leone-cli/src/main.rs:1378-1430)."""
    from leone_b200.cli import build_parser
    from leone_b200.sampling.sampler import SamplingParams
    args = build_parser().parse_args(["generate", "-m", "x", "-t", "1,2", "-n", "4", "--temp", "0.8", "--min-p", "0.1",
                                      "--top-k", "40", "--typical", "0.9", "--top-k", "5"])
    assert args.truncations == [("min_p", 0.1), ("top_k", 40), ("typical", 0.9), ("top_k", 5)]
    params = SamplingParams(args.temp, args.seed, tuple(args.truncations))
    assert params.truncates and not SamplingParams(0.0, 0, tuple(args.truncations)).truncates
    assert build_parser().parse_args(["generate", "-m", "x", "-t", "1", "-n", "1"]).truncations is None


def test_stop_ids_may_be_a_list_and_come_from_generation_config(tmp_path):
    import json
    from leone_b200.config.base import InvalidValue, WrongType
    from leone_b200.registry import config_from_dict, config_from_folder, spec_from_config
    from tests.tiny import TINY_B
    cfg = config_from_dict({**TINY_B, "eos_token_id": [7, 9, 7]})
    assert cfg.eos_token_ids == (7, 9) and cfg.eos_token_id == 7
    assert spec_from_config(cfg).stop_ids() == (7, 9)
    assert config_from_dict(cfg.to_json_dict()).eos_token_ids == (7, 9)          # survives a round trip
    assert config_from_dict({**TINY_B, "eos_token_id": 5}).eos_token_ids == (5,)
    assert spec_from_config(config_from_dict(TINY_B)).stop_ids() == ()
    with pytest.raises(InvalidValue):
        config_from_dict({**TINY_B, "eos_token_id": [7, 100000]})
    with pytest.raises(WrongType):
        config_from_dict({**TINY_B, "eos_token_id": "7"})
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_B))
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 4]}))
    assert config_from_folder(str(folder)).eos_token_ids == (3, 4)

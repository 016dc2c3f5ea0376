"""Safetensors reading/writing, the loader's one error, and random-weight folders."""
import json
import os
import struct

import pytest
import torch

from leone_b200.config.qwen3 import Qwen3Config
from leone_b200.engine.model import weight_specs_for_config
from leone_b200.parts.base import WeightSpec
from leone_b200.weights.loader import WeightError, load_checkpoint, target_dtype
from leone_b200.weights.random_init import random_tensors, write_random_model
from leone_b200.weights.safetensors import Checkpoint, SafetensorsError, write_safetensors
from tests.tiny import TINY_A, TINY_B, make_folder


def test_safetensors_roundtrip(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "e": torch.zeros(0, 4)}
    path = os.path.join(str(tmp_path), "model.safetensors")
    write_safetensors(path, tensors)
    ckpt = Checkpoint(str(tmp_path))
    assert set(ckpt.names()) == set(tensors)
    for name, t in tensors.items():
        got = ckpt.read(name)
        assert got.dtype == t.dtype and torch.equal(got, t)
    ckpt.close()


def test_safetensors_agrees_with_the_installed_reader(tmp_path):
    safetensors = pytest.importorskip("safetensors.torch")
    tensors = {"x": torch.randn(4, 4), "y": torch.randn(3).to(torch.bfloat16)}
    path = os.path.join(str(tmp_path), "model.safetensors")
    write_safetensors(path, tensors)
    theirs = safetensors.load_file(path)
    assert all(torch.equal(theirs[k], v) for k, v in tensors.items())


def test_corrupt_files_are_refused(tmp_path):
    path = os.path.join(str(tmp_path), "model.safetensors")
    with open(path, "wb") as fh:
        fh.write(b"abc")
    with pytest.raises(SafetensorsError):
        Checkpoint(str(tmp_path))
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 99]}}).encode()
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(header)) + header + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="byte range"):
        Checkpoint(str(tmp_path))
    with pytest.raises(SafetensorsError):
        Checkpoint(os.path.join(str(tmp_path), "missing"))


def test_specs_name_every_tensor_of_the_architecture():
    cfg = Qwen3Config.from_dict(TINY_B)
    specs = weight_specs_for_config(cfg)
    names = {s.name: s for s in specs}
    assert len(specs) == 3 * 11 + 3                      # eleven per layer, table, final norm, head
    assert names["model.layers.2.self_attn.q_proj.weight"].shape == (6 * 32, 96)
    assert names["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert names["model.layers.0.self_attn.k_norm.weight"].role == "norm"
    assert names["model.layers.1.mlp.down_proj.weight"].shape == (96, 224)
    assert names["lm_head.weight"].shape == (384, 96)
    tied = {s.name for s in weight_specs_for_config(Qwen3Config.from_dict(TINY_A))}
    assert "lm_head.weight" not in tied


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_B)
    specs = weight_specs_for_config(cfg)
    tensors = random_tensors(specs, 1)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
    tensors["model.layers.2.self_attn.o_proj.weight"] = torch.zeros(96, 96)
    cfg.write(str(tmp_path))
    write_safetensors(os.path.join(str(tmp_path), "model.safetensors"), tensors)
    with pytest.raises(WeightError) as err:
        load_checkpoint(str(tmp_path), specs, torch.float32, "cpu")
    e = err.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"] or \
        set(e.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert len(e.wrong_shape) == 1 and "o_proj" in e.wrong_shape[0] and "[96, 192]" in e.wrong_shape[0]
    text = str(e)
    assert "missing tensors (2)" in text and "unexpected tensors (1)" in text and "wrong shapes (1)" in text


def test_tied_model_with_a_head_tensor_is_an_error(tmp_path):
    from leone_b200.engine.engine import Engine
    from tests.emulated_ops import EmulatedOps
    folder = make_folder(tmp_path, "A")
    ckpt = Checkpoint(folder)
    tensors = {n: ckpt.read(n) for n in ckpt.names()}
    ckpt.close()
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="ties the head"):
        Engine.from_folder(folder, dtype="float32", device="cpu", ops=EmulatedOps())


def test_dtype_policy():
    mat, norm, table = WeightSpec("m", (2, 2)), WeightSpec("n", (2,), "norm"), WeightSpec("t", (2,), "int_table")
    bf, f32 = torch.bfloat16, torch.float32
    assert target_dtype(mat, f32, bf) == bf and target_dtype(mat, bf, f32) == f32
    assert target_dtype(norm, f32, bf) == f32          # a tensor stored in 32 bits stays so
    assert target_dtype(norm, bf, bf) == bf and target_dtype(norm, torch.float16, f32) == f32
    assert target_dtype(table, torch.int64, bf) == torch.int32


def test_random_model_folder_is_seeded_and_loadable(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_A)
    a, b, c = (os.path.join(str(tmp_path), n) for n in "abc")
    write_random_model(cfg, a, seed=5)
    write_random_model(cfg, b, seed=5)
    write_random_model(cfg, c, seed=6)
    specs = weight_specs_for_config(cfg)
    ta, tb, tc = (load_checkpoint(f, specs, torch.float32, "cpu") for f in (a, b, c))
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert any(not torch.equal(ta[k], tc[k]) for k in ta)
    w = ta["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.003 and abs(float(w.mean())) < 0.002
    n = ta["model.layers.1.input_layernorm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.15
    assert os.path.isfile(os.path.join(a, "config.json"))

"""Seeded random weights.

Matrices and embedding tables are drawn N(0, 0.02), norm weights 1 + N(0, 0.1).
Each tensor has its own generator seeded from (seed, tensor name), so a
tensor's values do not depend on which other tensors exist.  The reference has
no random-weight mode (its tests use a zero-weight fixture,
crates/leone/tests/common/cpu_fixture.rs:67-106); this one is this engine's own.
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict, Sequence

import torch

from ..parts.base import WeightSpec
from .safetensors import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def draw(spec: WeightSpec, seed: int, device="cpu") -> torch.Tensor:
    """One tensor's fp32 values (int32 for tables) for this seed."""
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, spec.name))
    if spec.role == "int_table":
        return torch.randint(0, 1 << 15, spec.shape, generator=gen, device=device, dtype=torch.int32)
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    t.normal_(0.0, spec.std, generator=gen)
    if spec.role == "norm":
        t += 1.0
    return t


def random_tensors(specs: Sequence[WeightSpec], seed: int, store_dtype: torch.dtype = torch.float32,
                   device="cpu") -> Dict[str, torch.Tensor]:
    out = {}
    for spec in specs:
        t = draw(spec, seed, device)
        out[spec.name] = t if spec.role == "int_table" else t.to(store_dtype)
    return out


def write_random_model(config, folder: str, seed: int, store_dtype: torch.dtype = torch.float32) -> None:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded random weights."""
    from ..engine.model import weight_specs_for_config
    os.makedirs(folder, exist_ok=True)
    config.write(folder)
    specs = weight_specs_for_config(config)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(specs, seed, store_dtype),
                      metadata={"format": "pt", "seed": str(seed)})

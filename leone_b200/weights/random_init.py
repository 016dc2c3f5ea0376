"""Seeded random weights: a pure function of (seed, tensor name, element index).

Matrices and embedding tables are drawn N(0, 0.02), norm weights 1 + N(0, 0.1).  The draw
is counter-based (``csrc/random_draw.h`` defines it operation by operation): a tensor's key
is the first eight bytes of ``sha256("<seed>:<name>")``, and element ``i`` is a Box-Muller
normal made from two splitmix64 outputs of that key with arithmetic that rounds the same on
the host and on the device.  So a tensor's values do not depend on which other tensors
exist, any slice of a tensor can be drawn by itself, and the model that
:meth:`Engine.from_config` draws on the GPU is bit for bit the model that
:func:`write_random_model` writes to a folder for the same configuration and seed.

The reference has no random-weight mode (its tests use a zero-weight fixture,
crates/leone/tests/common/cpu_fixture.rs:67-106); this one is this engine's own.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
from ctypes import c_double, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Dict, Optional, Sequence

import torch

from ..parts.base import WeightSpec
from .safetensors import write_safetensors


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's stream."""
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little")


def _mean_std(spec: WeightSpec):
    return (1.0 if spec.role == "norm" else 0.0), float(spec.std)


def draw(spec: WeightSpec, seed: int, device="cpu", dtype: Optional[torch.dtype] = None,
         start: int = 0, count: Optional[int] = None) -> torch.Tensor:
    """One tensor's values for this seed: fp32 (or ``dtype``: bfloat16 is the fp32 value rounded
    to nearest even), int32 for integer tables.  ``start``/``count`` draw a flat slice of the
    tensor's elements instead of the whole tensor."""
    device = torch.device(device)
    numel = 1
    for s in spec.shape:
        numel *= int(s)
    whole = count is None and start == 0
    if count is None:
        count = numel - start
    if start < 0 or count < 0 or start + count > numel:
        raise ValueError(f"{spec.name}: slice [{start}, {start + count}) is outside its {numel} elements")
    key = tensor_key(seed, spec.name)
    mean, std = _mean_std(spec)
    table = spec.role == "int_table"
    if dtype is None or table:
        dtype = torch.int32 if table else torch.float32
    if dtype not in (torch.float32, torch.bfloat16, torch.int32):
        raise ValueError(f"random weights are drawn as float32, bfloat16 or int32, not {dtype}")
    if device.type == "cuda":
        from ..csrc.build import ensure_built
        lib = ctypes.CDLL(ensure_built("core"))
        out = torch.empty(count, dtype=dtype, device=device)
        kind = 2 if table else (1 if dtype == torch.bfloat16 else 0)
        with torch.cuda.device(device):
            code = lib.leone_random_fill_device(
                c_ulonglong(key), c_longlong(start), c_longlong(count), c_double(mean), c_double(std),
                c_int(kind), c_void_p(out.data_ptr()),
                c_void_p(torch.cuda.current_stream(device).cuda_stream))
        if code != 0:
            raise RuntimeError(f"random weights: the device kernel failed with code {code}")
    else:
        from ..cache.pages import host_library
        lib = host_library()
        out = torch.empty(count, dtype=torch.int32 if table else torch.float32)
        code = lib.leone_random_fill_host(c_ulonglong(key), c_longlong(start), c_longlong(count), c_double(mean),
                                          c_double(std), c_int(1 if table else 0), c_void_p(out.data_ptr()))
        if code != 0:
            raise RuntimeError(f"random weights: the host routine refused its arguments ({code})")
        if out.dtype != dtype:
            out = out.to(dtype)
    return out.view(spec.shape) if whole else out


def random_tensors(specs: Sequence[WeightSpec], seed: int, store_dtype: torch.dtype = torch.float32,
                   device="cpu") -> Dict[str, torch.Tensor]:
    return {spec.name: draw(spec, seed, device, store_dtype) for spec in specs}


def write_random_model(config, folder: str, seed: int, store_dtype: torch.dtype = torch.float32) -> None:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded random weights."""
    from ..engine.model import weight_specs_for_config
    os.makedirs(folder, exist_ok=True)
    config.write(folder)
    specs = weight_specs_for_config(config)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(specs, seed, store_dtype),
                      metadata={"format": "pt", "seed": str(seed)})

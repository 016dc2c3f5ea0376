"""Loading a model's tensors by name, with one error that says everything wrong.

The reference reads each tensor by name, checks shape and type, and rejects a
file that holds a tensor it did not consume (``require_tensor`` /
``check_shape`` crates/leone/src/model.rs:1060-1075; ``validate_loaded_tensors``
:697-714).  Here all findings are collected first and raised together.

Dtype policy.  Matrices and embedding tables are kept in the run dtype
(bfloat16 or float32).  Norm weights and other small vectors that the file
stores in 32 bits stay 32-bit even in a bfloat16 run; stored in 16 bits they
become bfloat16 (float32 in a 32-bit run).  Integer tables become int32.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from ..parts.base import WeightSpec
from .safetensors import Checkpoint


class WeightError(ValueError):
    """The checkpoint does not hold exactly the tensors the model needs."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str], wrong_shape: Sequence[str],
                 other: Sequence[str] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        if self.other:
            lines.extend("  " + o for o in self.other)
        super().__init__("\n".join(lines))


def target_dtype(spec: WeightSpec, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "int_table":
        return torch.int32
    if spec.role in ("matrix", "embedding"):
        return run_dtype
    if stored in (torch.float32, torch.float64) or run_dtype == torch.float32:
        return torch.float32
    return torch.bfloat16


def check_names_and_shapes(specs: Sequence[WeightSpec], entries: Dict[str, object],
                           notes: Sequence[str] = ()) -> None:
    """Raise :class:`WeightError` unless ``entries`` (name → object with .shape/.dtype) fits."""
    wanted = {s.name: s for s in specs}
    missing = [n for n in wanted if n not in entries]
    unexpected = sorted(n for n in entries if n not in wanted)
    wrong = []
    other = list(notes)
    for name, spec in wanted.items():
        if name not in entries:
            continue
        e = entries[name]
        if tuple(e.shape) != tuple(spec.shape):
            wrong.append(f"{name}: expected {list(spec.shape)}, file has {list(e.shape)}")
        is_int = e.dtype in (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)
        if (spec.role == "int_table") != is_int or e.dtype == torch.bool:
            other.append(f"{name}: dtype {e.dtype} does not fit a tensor of role '{spec.role}'")
    if missing or unexpected or wrong or other:
        raise WeightError(missing, unexpected, wrong, other)


def load_checkpoint(folder: str, specs: Sequence[WeightSpec], run_dtype: torch.dtype, device,
                    notes: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Read every tensor in ``specs`` from ``folder`` onto ``device``."""
    ckpt = Checkpoint(folder)
    try:
        check_names_and_shapes(specs, ckpt.entries, notes)
        out: Dict[str, torch.Tensor] = {}
        for spec in specs:
            t = ckpt.read(spec.name)
            out[spec.name] = t.to(target_dtype(spec, t.dtype, run_dtype)).to(device).contiguous()
        return out
    finally:
        ckpt.close()

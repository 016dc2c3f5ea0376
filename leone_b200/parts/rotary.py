"""Rotary position encoding, with half-split or adjacent pairing.

Pair ``i`` of a head is elements ``(i, i + rotary_dim/2)`` (half-split) or
``(2i, 2i + 1)`` (adjacent; crates/leone/src/backend.rs:1216-1222,
crates/leone/src/cpu.rs:1767-1770); its angle at
position ``p`` is ``p * theta^(-2i/rotary_dim)``, inverse frequency and angle
in float64 (crates/leone/src/cpu.rs:1735-1745 and 1747-1779); the rotation is
``x'_i = x_i cos - x_j sin``, ``x'_j = x_i sin + x_j cos``.  The reference's
CUDA path also rotates with an fp32 (cos, sin) table made from float64 trig
(crates/leone-cuda/cuda/ie_cuda.cu:2382-2402).  The table is a constant of the
part, built once for ``max_positions``.
"""
from __future__ import annotations

import torch

from ..registry import POSITION_ENCODINGS
from .base import PositionEncoding


def build_rotary_table(max_positions: int, rotary_dim: int, theta: float) -> torch.Tensor:
    half = rotary_dim // 2
    pair = torch.arange(half, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * pair / rotary_dim)
    pos = torch.arange(max_positions, dtype=torch.float64)
    angle = pos[:, None] * inv_freq[None, :]
    return torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32).contiguous()


@POSITION_ENCODINGS.register("rotary_half_split")
class RotaryHalfSplit(PositionEncoding):
    pairing = "half_split"

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim")
        self._table = None

    def rotary_table(self):
        if self._table is None:
            self._table = build_rotary_table(
                self.max_positions, self.rotary_dim, self.theta).to(self.rt.device)
        return self._table


@POSITION_ENCODINGS.register("rotary_adjacent")
class RotaryAdjacent(RotaryHalfSplit):
    """The same angles with pair ``i`` made of elements ``(2i, 2i + 1)``: the table is the same,
    the kernels are told which elements belong together."""
    pairing = "adjacent"

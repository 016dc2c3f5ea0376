"""Sampling from fp32 logits on the device.

Greedy takes the highest finite logit, lowest id on a tie
(crates/leone/src/sampler.rs:787-799).  Temperature ``t > 0`` draws from
``softmax(logits / t)`` with the uniform value
``uniform(seed, position, Select)`` of the reference's counter-based generator
(crates/leone/src/sampler.rs:84-94), where ``position`` is the absolute index
of the token whose logits are sampled (crates/leone/src/runtime.rs:4945), and
scans tokens in id order (crates/leone/src/sampler.rs:839-858).  A request's
stream therefore does not depend on how it was batched or cut.  The reference
samples on the host in float64 after reading the whole row back
(crates/leone/src/runtime.rs:9401); here the row stays on the device and only
the token id comes back.  Its truncation stages and penalties
(crates/leone/src/sampler.rs:184-234, crates/leone/src/penalty.rs) are not built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0     # 0 = greedy
    seed: int = 0

    def __post_init__(self):
        t = float(self.temperature)
        if not (t >= 0.0) or t == float("inf"):
            # crates/leone/src/sampler.rs:330-336: a temperature must be finite and > 0
            raise ValueError(f"temperature must be finite and >= 0 (0 = greedy), got {self.temperature}")


class Sampler:
    def __init__(self, ops, device, max_rows: int = 256):
        self.ops = ops
        self.device = torch.device(device)
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        self._cap = rows
        pin = self.device.type == "cuda"
        # one packed host buffer: temperature as float32 bits, then seed and position as int64
        self._host = torch.empty(rows * 3, dtype=torch.int64, pin_memory=pin)
        self._dev = torch.empty(rows * 3, dtype=torch.int64, device=self.device)
        self._out = torch.empty(rows, dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               positions: Sequence[int]) -> torch.Tensor:
        """One token id per logits row, as an int32 device tensor."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(positions):
            raise ValueError("sample: one SamplingParams and one position per logits row")
        if rows > self._cap:
            self._grow(max(rows, 2 * self._cap))
        host = self._host.numpy()
        temps = np.array([p.temperature for p in params], dtype=np.float32)
        host_f = self._host[:self._cap].view(torch.float32).numpy()      # first `cap` int64 = 2*cap floats
        host_f[:rows] = temps
        host[self._cap:self._cap + rows] = np.array([p.seed & 0xFFFF_FFFF_FFFF_FFFF for p in params],
                                                    dtype=np.uint64).view(np.int64)
        host[2 * self._cap:2 * self._cap + rows] = np.asarray(positions, dtype=np.int64)
        self._dev.copy_(self._host, non_blocking=True)
        t = self._dev[:self._cap].view(torch.float32)[:rows]
        seeds = self._dev[self._cap:self._cap + rows]
        pos = self._dev[2 * self._cap:2 * self._cap + rows]
        out = self._out[:rows]
        self.ops.sample(logits, t, seeds, pos, out)
        return out

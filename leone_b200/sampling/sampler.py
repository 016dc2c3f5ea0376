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
the token id comes back.

The reference's truncation stages (crates/leone/src/sampler.rs:184-234: top-k, top-p, min-p,
top-a, tail-free, typical, epsilon, eta, min-k, top-n-sigma, applied in the order given, each
on the renormalised survivors of the one before) run on the device too, in float64
(``csrc/sampling_pipeline.cu``: a sort of the row, block-wide sums and scans, an id-order
draw); rows that ask for them take that path, the others the single kernel.  Its penalties,
Mirostat and grammar constraint (crates/leone/src/penalty.rs, crates/leone/src/sampler.rs:97-164)
are not built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np
import torch


# stage name -> the kernel's stage number; the names are the reference's flags without dashes
# (crates/leone-cli/src/main.rs:836-845), "tfs" being tail-free sampling
TRUNCATION_STAGES = {"top_k": 0, "top_p": 1, "min_p": 2, "top_a": 3, "tfs": 4, "typical": 5, "epsilon": 6,
                     "eta": 7, "min_k": 8, "top_n_sigma": 9}
MAX_TRUNCATIONS = 16


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0     # 0 = greedy
    seed: int = 0
    # (stage name, value) pairs in the order they apply; greedy takes no notice of them
    # (crates/leone/src/sampler.rs:489-499 returns before any stage)
    truncations: Tuple[Tuple[str, float], ...] = ()

    def __post_init__(self):
        t = float(self.temperature)
        if not (t >= 0.0) or t == float("inf"):
            # crates/leone/src/sampler.rs:330-336: a temperature must be finite and > 0
            raise ValueError(f"temperature must be finite and >= 0 (0 = greedy), got {self.temperature}")
        stages = tuple((str(n), float(v)) for n, v in self.truncations)
        object.__setattr__(self, "truncations", stages)
        if len(stages) > MAX_TRUNCATIONS:
            raise ValueError(f"at most {MAX_TRUNCATIONS} truncation stages")
        for name, value in stages:
            # crates/leone/src/sampler.rs:243-262: top-k a positive count; min-k and top-n-sigma
            # finite and >= 0; every other stage finite in (0, 1]
            if name not in TRUNCATION_STAGES:
                raise ValueError(f"unknown truncation stage '{name}'; known: {', '.join(TRUNCATION_STAGES)}")
            if name == "top_k":
                ok = value >= 1 and value == int(value)
            elif name in ("min_k", "top_n_sigma"):
                ok = np.isfinite(value) and value >= 0.0
            else:
                ok = np.isfinite(value) and 0.0 < value <= 1.0
            if not ok:
                raise ValueError(f"the {name} parameter {value} is outside its valid range")

    @property
    def truncates(self) -> bool:
        return bool(self.truncations) and self.temperature > 0


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
        # rows with truncation stages: grouped by their stage list, through the fp64 pipeline
        groups = {}
        for i, p in enumerate(params):
            if p.truncates:
                groups.setdefault(p.truncations, []).append(i)
        for stages, members in groups.items():
            index = torch.tensor(members, dtype=torch.int64, device=logits.device)
            picked = self.ops.sample_truncated(
                logits.index_select(0, index), [float(params[i].temperature) for i in members],
                [params[i].seed for i in members], [int(positions[i]) for i in members],
                [(TRUNCATION_STAGES[n], v) for n, v in stages])
            out.index_copy_(0, index, picked)
        return out

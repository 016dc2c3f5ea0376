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
draw); rows that ask for them take that path, the others the single kernel.

Its penalties (crates/leone/src/penalty.rs: repetition, presence and frequency over a window of
the history, and the repeated-suffix penalty DRY) change the logits before any sampling, greedy
included: the host walks the history it owns and lists which tokens are touched and how
(:class:`Penalties`), a kernel does the arithmetic on the logits in float64.

Mirostat v2 (crates/leone/src/sampler.rs:97-164, 383-420) keeps one number per request, the
maximum surprise: after the stages, tokens more surprising than that are dropped, the draw is
made from the rest, and the number moves by ``learning_rate * (observed - target)`` with the
drawn token's surprise under the distribution before the drop (:class:`SamplerState`).  The
grammar constraint is not built.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import math
import sys

import numpy as np
import torch


# stage name -> the kernel's stage number; the names are the reference's flags without dashes
# (crates/leone-cli/src/main.rs:836-845), "tfs" being tail-free sampling
TRUNCATION_STAGES = {"top_k": 0, "top_p": 1, "min_p": 2, "top_a": 3, "tfs": 4, "typical": 5, "epsilon": 6,
                     "eta": 7, "min_k": 8, "top_n_sigma": 9}
MAX_TRUNCATIONS = 16


@dataclass(frozen=True)
class Penalties:
    """What is applied to a logit row before the sampler sees it
    (crates/leone/src/penalty.rs:116-126; defaults :130-138, 81-89)."""
    repetition: float = 1.0          # divides positive logits of seen tokens, multiplies the others; 1.0 is off
    presence: float = 0.0            # subtracted once from any seen token
    frequency: float = 0.0           # subtracted once per earlier occurrence
    window: Optional[int] = 64       # tokens of history the three look at; 0 disables, None is all
    dry_multiplier: float = 0.0      # the repeated-suffix penalty; 0.0 is off
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_window: int = 64
    dry_breakers: Tuple[int, ...] = ()

    def __post_init__(self):
        fin = np.isfinite
        # crates/leone/src/penalty.rs:147-158, 92-107
        if not (fin(self.repetition) and self.repetition > 0.0):
            raise ValueError("the repetition penalty must be finite and greater than zero")
        if not fin(self.presence):
            raise ValueError("the presence penalty must be finite")
        if not fin(self.frequency):
            raise ValueError("the frequency penalty must be finite")
        if self.window is not None and self.window < 0:
            raise ValueError("the penalty window cannot be negative")
        if not (fin(self.dry_multiplier) and self.dry_multiplier >= 0.0):
            raise ValueError("the DRY multiplier is outside its valid range")
        if not (fin(self.dry_base) and self.dry_base > 0.0):
            raise ValueError("the DRY base is outside its valid range")
        if self.dry_allowed_length < 1:
            raise ValueError("the DRY allowed length is outside its valid range")
        if self.dry_window < 0:
            raise ValueError("the DRY window cannot be negative")

    @property
    def counting(self) -> bool:
        return self.window != 0 and (self.repetition != 1.0 or self.presence != 0.0 or self.frequency != 0.0)

    @property
    def dry(self) -> bool:
        return self.dry_multiplier > 0.0 and self.dry_window > 0

    @property
    def active(self) -> bool:
        """Whether any penalty would change a logit (crates/leone/src/penalty.rs:141-145)."""
        return self.counting or self.dry

    def touched(self, context: Sequence[int]) -> Dict[int, Tuple[int, float]]:
        """token -> (occurrences in the counting window, DRY penalty) for the history ``context``
        (the whole of it, prompt included): which logits change; the arithmetic is the kernel's.
        DRY (crates/leone/src/penalty.rs:208-257): for every earlier place in its window that
        holds the last token, the length of the match that ends there against the history's end
        (not across a breaker); from ``dry_allowed_length`` on, the token that followed that place
        is charged ``multiplier * base ** (length - allowed)``, the largest charge if several."""
        out: Dict[int, List] = {}
        if self.counting:
            recent = context if self.window is None else context[max(0, len(context) - self.window):]
            for t in recent:
                out.setdefault(int(t), [0, 0.0])[0] += 1
        if self.dry:
            recent = list(context[max(0, len(context) - self.dry_window):])
            last = len(recent) - 1
            for start in range(last):
                if recent[start] != recent[last]:
                    continue
                length = 1
                while (length <= start and length <= last and recent[start - length] == recent[last - length]
                       and recent[last - length] not in self.dry_breakers):
                    length += 1
                if length < self.dry_allowed_length:
                    continue
                nxt = int(recent[start + 1])
                if nxt in self.dry_breakers:
                    continue
                charge = self.dry_multiplier * self.dry_base ** (length - self.dry_allowed_length)
                entry = out.setdefault(nxt, [0, 0.0])
                entry[1] = max(entry[1], charge)
        return {t: (c, d) for t, (c, d) in out.items()}


class SamplerState:
    """What a request's sampler remembers between its tokens: Mirostat's maximum surprise, which
    starts at twice the target (crates/leone/src/sampler.rs:138-144)."""

    def __init__(self, params: "SamplingParams"):
        self.maximum_surprise = 2.0 * params.mirostat[0] if params.mirostat else None

    def observe(self, params: "SamplingParams", probability: float) -> None:
        """The drawn token had this probability before the surprise filter
        (crates/leone/src/sampler.rs:392-396)."""
        target, rate = params.mirostat
        self.maximum_surprise -= rate * (-math.log(probability) - target)
        self.maximum_surprise = max(self.maximum_surprise, sys.float_info.epsilon)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0     # 0 = greedy
    seed: int = 0
    # (stage name, value) pairs in the order they apply; greedy takes no notice of them
    # (crates/leone/src/sampler.rs:489-499 returns before any stage)
    truncations: Tuple[Tuple[str, float], ...] = ()
    penalties: Optional[Penalties] = None
    mirostat: Optional[Tuple[float, float]] = None      # (target surprise in nats, learning rate)

    def __post_init__(self):
        if self.mirostat is not None:
            target, rate = (float(v) for v in self.mirostat)
            object.__setattr__(self, "mirostat", (target, rate))
            # crates/leone/src/sampler.rs:111-123
            if not (np.isfinite(target) and target > 0.0):
                raise ValueError("the Mirostat target must be finite and greater than zero")
            if not (np.isfinite(rate) and 0.0 < rate <= 1.0):
                raise ValueError("the Mirostat learning rate must be finite and in (0, 1]")
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

    @property
    def penalizes(self) -> bool:
        return self.penalties is not None and self.penalties.active

    @property
    def outside_graph(self) -> bool:
        """Whether a request samples with more than the captured decode step holds (greedy and
        temperature): truncation stages, penalties (which need the history), Mirostat (which
        keeps a number per request)."""
        return self.truncates or self.penalizes or self.mirostat is not None


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
               positions: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None,
               states: Optional[Sequence[Optional[SamplerState]]] = None) -> torch.Tensor:
        """One token id per logits row, as an int32 device tensor.  ``histories``: every row's
        whole token history (prompt included), needed by rows whose parameters hold penalties;
        their logits are changed in place.  ``states``: every row's :class:`SamplerState`,
        needed (and updated) by rows with Mirostat."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(positions):
            raise ValueError("sample: one SamplingParams and one position per logits row")
        if any(p.penalizes for p in params):
            if histories is None or len(histories) != rows:
                raise ValueError("sample: penalties need every row's token history")
            entries = [(i, t, c, d) for i, p in enumerate(params) if p.penalizes
                       for t, (c, d) in p.penalties.touched(histories[i]).items()]
            if entries:
                neutral = Penalties()
                self.ops.penalize(logits, entries, [(p.penalties or neutral) if p.penalizes else neutral
                                                    for p in params])
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
        if any(p.mirostat for p in params) and (states is None or len(states) != rows or any(
                p.mirostat and states[i] is None for i, p in enumerate(params))):
            raise ValueError("sample: Mirostat needs every such row's SamplerState")
        groups = {}
        for i, p in enumerate(params):
            if p.temperature > 0 and (p.truncations or p.mirostat):
                groups.setdefault((p.truncations, p.mirostat is not None), []).append(i)
        for (stages, surprise), members in groups.items():
            # the group's rows are sampled where they lie: the kernels read those rows of the
            # logits and write their ids over what the plain kernel left there
            got = self.ops.sample_truncated(
                logits, [float(params[i].temperature) for i in members],
                [params[i].seed for i in members], [int(positions[i]) for i in members],
                [(TRUNCATION_STAGES[n], v) for n, v in stages],
                maximum_surprise=[states[i].maximum_surprise for i in members] if surprise else None,
                rows=members, out=out)
            if surprise:
                for i, p_ in zip(members, got[1].tolist()):
                    states[i].observe(params[i], p_)
        for i, p in enumerate(params):
            if p.mirostat and not p.temperature > 0:
                states[i].observe(p, 1.0)       # greedy: the one token has probability one
        return out

"""Per-request state of fixed size: one record per state slot, on the host and mirrored on the device.

A live request owns one slot (``CacheManager.open`` hands it out with the request's block
tables and takes it back with its pages).  The slot is the row of every fixed-size thing the
request has: the rows of mixers' ``FixedState`` tensors, and the record kept here, eight 64-bit
words:

    0 length       tokens in the cache
    1 position     absolute position of the token being sampled next
    2 seed         the sampler's seed (the draw is f(seed, position), so nothing else is kept)
    3 temperature  fp32 bits in the low word; 0 is greedy
    4 last_token   the token sampled last (what the next decode step feeds)
    5 flags        bit 0: cancellation requested; bit 1: the slot is live
    6 status       the request's own status word (0 = fine)
    7 sampler      one fp64 of sampler feedback state (Mirostat's maximum surprise)

The reference keeps the same things with its session: position and device position
(crates/leone/src/kv.rs:64-65), evaluated tokens and sampler feedback state
(crates/leone/src/runtime.rs:600-616), the cancellation flag (crates/leone/src/runtime_service.rs:26);
its sampling draw is likewise a function of (seed, position) (crates/leone/src/sampler.rs:84-94).

The captured decode step reads temperature, seed and position from the device copy through the
step's slot ids and advances position, length and last token there itself, so a quantum of steps
needs nothing from the host.  The host copy is what the scheduler writes; ``sync`` brings the
rows that changed to the device.
"""
from __future__ import annotations

import struct
from typing import Iterable, Optional

import torch

FIELDS = 8
LENGTH, POSITION, SEED, TEMPERATURE, LAST_TOKEN, FLAGS, STATUS, SAMPLER = range(FIELDS)
CANCEL_REQUESTED = 1
LIVE = 2
_MASK = (1 << 64) - 1


def _signed(value: int) -> int:
    value &= _MASK
    return value - (1 << 64) if value >= 1 << 63 else value


class SlotRecords:
    def __init__(self, num_slots: int, device):
        self.device = torch.device(device)
        self.num_slots = num_slots
        pin = self.device.type == "cuda"
        self.host = torch.zeros((num_slots, FIELDS), dtype=torch.int64, pin_memory=pin)
        self.on_device = torch.zeros((num_slots, FIELDS), dtype=torch.int64, device=self.device)
        self._rows = self.host.numpy()
        self._dirty = set()

    # -- lifetime (the engine calls these beside CacheManager.open / close) ------------------
    def open(self, slot: int) -> None:
        self._rows[slot, :] = 0
        self._rows[slot, FLAGS] = LIVE
        self._dirty.add(slot)

    def close(self, slot: int) -> None:
        self._rows[slot, :] = 0
        self._dirty.add(slot)

    # -- what the scheduler and the decode loop write ------------------------------------------
    def set_sampling(self, slot: int, seed: int, temperature: float) -> None:
        self._rows[slot, SEED] = _signed(int(seed))
        self._rows[slot, TEMPERATURE] = struct.unpack("<I", struct.pack("<f", float(temperature)))[0]
        self._dirty.add(slot)

    def set_progress(self, slot: int, length: int, position: int, last_token: Optional[int] = None) -> None:
        self._rows[slot, LENGTH] = length
        self._rows[slot, POSITION] = position
        if last_token is not None:
            self._rows[slot, LAST_TOKEN] = last_token
        self._dirty.add(slot)

    def set_sampler_state(self, slot: int, value: float) -> None:
        self._rows[slot, SAMPLER] = struct.unpack("<q", struct.pack("<d", float(value)))[0]
        self._dirty.add(slot)

    def sampler_state(self, slot: int) -> float:
        return struct.unpack("<d", struct.pack("<q", int(self._rows[slot, SAMPLER])))[0]

    def request_cancel(self, slot: int) -> None:
        self._rows[slot, FLAGS] |= CANCEL_REQUESTED
        self._dirty.add(slot)

    def cancel_requested(self, slot: int) -> bool:
        return bool(int(self._rows[slot, FLAGS]) & CANCEL_REQUESTED)

    def is_live(self, slot: int) -> bool:
        return bool(int(self._rows[slot, FLAGS]) & LIVE)

    def record(self, slot: int) -> dict:
        """The host copy of one record, by field name."""
        r = self._rows[slot]
        return dict(length=int(r[LENGTH]), position=int(r[POSITION]), seed=int(r[SEED]) & _MASK,
                    temperature=struct.unpack("<f", struct.pack("<I", int(r[TEMPERATURE]) & 0xFFFFFFFF))[0],
                    last_token=int(r[LAST_TOKEN]), cancel_requested=self.cancel_requested(slot),
                    live=self.is_live(slot), status=int(r[STATUS]), sampler=self.sampler_state(slot))

    # -- host <-> device ---------------------------------------------------------------------------
    def sync(self, slots: Optional[Iterable[int]] = None) -> None:
        """Copy the rows that changed (or ``slots``) to the device copy, on the current stream."""
        rows = sorted(self._dirty if slots is None else set(slots) | self._dirty)
        self._dirty.clear()
        if not rows:
            return
        if len(rows) * 2 >= self.num_slots:
            self.on_device.copy_(self.host, non_blocking=True)
            return
        start = prev = rows[0]
        for r in rows[1:] + [None]:                     # runs of neighbouring rows go in one copy
            if r is not None and r == prev + 1:
                prev = r
                continue
            self.on_device[start:prev + 1].copy_(self.host[start:prev + 1], non_blocking=True)
            if r is not None:
                start = prev = r

    def read_device(self, slot: int) -> dict:
        """The device copy of one record (a synchronising read; for tests and diagnosis)."""
        r = self.on_device[slot].cpu().tolist()
        return dict(length=r[LENGTH], position=r[POSITION], seed=r[SEED] & _MASK,
                    temperature=struct.unpack("<f", struct.pack("<I", r[TEMPERATURE] & 0xFFFFFFFF))[0],
                    last_token=r[LAST_TOKEN], flags=r[FLAGS], status=r[STATUS])

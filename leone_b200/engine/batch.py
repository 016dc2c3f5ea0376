"""One step's batch as flat device arrays.

A step is a list of (request, its next tokens, wanted positions).  All tokens
of all entries form one flat list of ``N`` rows; per-token and per-sequence
index arrays say where each row belongs.  Everything that varies from step to
step lives in one int32 device buffer, filled by a single host→device copy:

    token_ids[N] positions[N] seq_of_token[N] q_start[B+1] ctx_len[B]
    slot_ids[B] logit_rows[M] block_table_g[B, W_g] for every cache group g

``positions`` are absolute (crates/leone/src/cpu.rs:1759-1765: prefill position
= start + t); ``ctx_len`` is a sequence's length after this step, so the query
at position p reads keys ``..p`` (the reference masks by loop bound,
crates/leone/src/cpu.rs:2372).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch



@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepContext:
    """Device views of one step's metadata plus what the parts need to find their caches."""

    def __init__(self):
        self.n_tokens = 0
        self.n_seqs = 0
        self.n_logit_rows = 0
        self.token_ids = self.positions = self.seq_of_token = None
        self.q_start = self.ctx_len = self.slot_ids = self.logit_rows = None
        self.block_tables: List[torch.Tensor] = []
        self.q_lens: np.ndarray = None
        self.starts: np.ndarray = None
        self.ctx_lens: np.ndarray = None
        self.max_q_len = 0
        self.max_ctx_len = 0
        self.decode_only = False
        self.status: torch.Tensor = None
        self.logits_out: Optional[torch.Tensor] = None
        self.layer_caches: Dict[int, object] = {}
        self.fixed_shapes = False      # True while a CUDA graph is captured or replayed

    def cache_view(self, run_position: int):
        """The cache of the layer at this position of the run order (None if it has none)."""
        return self.layer_caches.get(run_position)


def pack_metadata(token_lists: Sequence[Sequence[int]], starts: Sequence[int], slots: Sequence[int],
                  wants: Sequence[Sequence[int]], block_tables: Sequence[np.ndarray]):
    """Host side of the layout above, laid out by the C++ host runtime (``leone_pack_step``).
    Returns (packed int32 array, offsets dict, block-table offsets, host stats)."""
    from ..cache.pages import host_library
    lib = host_library()
    b = len(token_lists)
    q_lens = np.array([len(t) for t in token_lists], dtype=np.int64)
    n = int(q_lens.sum())
    starts = np.ascontiguousarray(starts, dtype=np.int64)
    token_ids = np.concatenate([np.asarray(t, dtype=np.int64) for t in token_lists]) if n else np.zeros(1, np.int64)
    want_start = np.zeros(b + 1, dtype=np.int64)
    np.cumsum([len(w) for w in wants], out=want_start[1:])
    m = int(want_start[b])
    flat_wants = np.array([j for w in wants for j in w] or [0], dtype=np.int64)
    slot_ids = np.ascontiguousarray(slots if b else [0], dtype=np.int64)
    sizes = [("token_ids", n), ("positions", n), ("seq_of_token", n), ("q_start", b + 1), ("ctx_len", b),
             ("slot_ids", b), ("logit_rows", m)]
    offsets = {}
    cursor = 0
    for name, size in sizes:
        offsets[name] = (cursor, size)
        cursor += size
    bt_offsets = []
    for bt in block_tables:
        bt_offsets.append((cursor, bt.shape))
        cursor += bt.size
    assert cursor == lib.leone_pack_step_size(b, ctypes.c_longlong(n), ctypes.c_longlong(m),
                                              ctypes.c_longlong(sum(bt.size for bt in block_tables)))
    packed = np.empty(max(cursor, 1), dtype=np.int32)

    def ptr(a):
        return a.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))

    code = lib.leone_pack_step(b, ptr(np.ascontiguousarray(q_lens if b else [0], dtype=np.int64)), ptr(token_ids),
                               ptr(starts if b else np.zeros(1, np.int64)), ptr(slot_ids), ptr(want_start),
                               ptr(flat_wants), packed.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
    if code != 0:
        raise ValueError(lib.leone_host_last_error().decode())
    for (o, shape), bt in zip(bt_offsets, block_tables):
        packed[o:o + bt.size] = bt.reshape(-1)
    ctx_len = starts + q_lens
    stats = dict(n=n, b=b, m=m, q_lens=q_lens, starts=starts, ctx_lens=ctx_len,
                 max_q_len=int(q_lens.max()) if b else 0, max_ctx_len=int(ctx_len.max()) if b else 0)
    return packed, offsets, bt_offsets, stats

"""The kernel table: Python calls into the engine's own CUDA libraries.

Every call checks shapes, dtypes and contiguity on the host, then launches on
the current torch stream through a C entry point of ``csrc`` (loaded with
ctypes; compiled on first use by :mod:`leone_b200.csrc.build`).  There is no
other implementation behind these calls: without a CUDA device or without the
compiled libraries, construction raises.  The reference has the same split
between checked wrappers and raw entry points
(crates/leone-cuda/src/cuda.rs, crates/leone-cuda/src/ffi.rs).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import numpy as np
import torch

from ..csrc.build import ensure_built

_STATUS_TEXT = {
    1: "a token id outside the vocabulary reached the embedding kernel",
    2: "a token's block has no valid page in its block table",
    3: "a position outside the position table",
    4: "a bounded wait inside a kernel ran out",
    5: "a token names a sequence outside the batch",
}
_REFUSALS = {
    -1: "a size this kernel does not take",
    -2: "a pointer or stride that is not aligned as the kernel needs",
    -3: "a dtype this kernel does not take",
}


class KernelError(RuntimeError):
    pass


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return 0
    if t == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {t}")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: refused — {_REFUSALS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


class PreparedMatrix:
    """A weight matrix ``[out, in]`` with what the kernels precompute for it."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        self.tma = None           # tensor map for the tensor-core kernel, made on first use

    @property
    def shape(self):
        return self.weight.shape

    @property
    def dtype(self):
        return self.weight.dtype


class CudaOps:
    def __init__(self, device, dtype: torch.dtype):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError(
                "leone_b200 runs on a CUDA device only (there is no CPU path); "
                f"asked for device '{device}', torch.cuda.is_available() = {torch.cuda.is_available()}")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; device reports sm_{major}{minor}")
        self.dtype = dtype
        self.core = ctypes.CDLL(ensure_built("core"))
        self.fast = None
        self._pinned_stream = None
        if dtype == torch.bfloat16:
            from .fast import FastKernels
            self.fast = FastKernels(self.device)
        self.launches = 0
        self._sample_scratch = None
        self.status = None
        # LEONE_NO_PDL=1 launches every kernel fully serialised after its predecessor
        self.set_pdl(os.environ.get("LEONE_NO_PDL", "0") != "1")

    def set_pdl(self, enabled: bool) -> None:
        """Programmatic dependent launch: a kernel may start (and fetch weights) while its
        predecessor in the stream still runs; it waits before touching the step's data."""
        self.core.leone_core_set_pdl(1 if enabled else 0)
        if self.fast is not None:
            self.fast.lib.leone_bf16_set_pdl(1 if enabled else 0)

    def bind_status(self, status: torch.Tensor) -> None:
        """The engine's status word; kernels with bounded waits report into it."""
        self.status = status
        if self.fast is not None:
            self.fast.status = status

    # -- helpers ------------------------------------------------------------------------
    def _stream(self):
        if self._pinned_stream is not None:        # (a handle of 0, the default stream, is a valid pin)
            return self._pinned_stream
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def pin_stream(self, on: bool) -> None:
        """Between ``pin_stream(True)`` and ``pin_stream(False)`` every launch goes to the stream
        that was current at the first call: a step looks its stream up once, not once per launch."""
        handle = c_void_p(torch.cuda.current_stream(self.device).cuda_stream) if on else None
        self._pinned_stream = handle
        if self.fast is not None:
            self.fast.pin_stream(handle)

    def describe_status(self, word: int) -> str:
        return _STATUS_TEXT.get(word, "unknown status")

    # -- weights ------------------------------------------------------------------------
    def scratch_bytes(self) -> int:
        """Device memory the ops allocate for themselves beyond the runtime's named buffers."""
        return self.fast.scratch_bytes() if self.fast is not None else 0

    def prepare_matrix(self, w: torch.Tensor) -> PreparedMatrix:
        _need(w.dim() == 2 and w.is_contiguous(), "a weight matrix must be contiguous [out, in]")
        return PreparedMatrix(w)

    def prepare_gate_up(self, gate: torch.Tensor, up: torch.Tensor) -> PreparedMatrix:
        _need(gate.shape == up.shape, "gate and up matrices differ in shape")
        if self.fast is not None:
            return self.fast.prepare_gate_up(gate, up)
        m = PreparedMatrix(torch.cat([gate, up], dim=0).contiguous())
        m.gate_up_layout = "stacked"
        return m

    # -- kernels ------------------------------------------------------------------------
    def embedding(self, table, ids, out, status, scale: float = 1.0):
        n, hidden = out.shape
        _need(out.dtype == torch.float32 and out.is_contiguous(), "embedding output must be fp32")
        _need(ids.dtype == torch.int32 and ids.numel() == n, "embedding ids must be int32 [N]")
        _need(table.shape[1] == hidden and table.is_contiguous(), "embedding table shape")
        self.launches += 1
        _check(self.core.leone_embedding(_dt(table.dtype), _ptr(table), _ptr(ids), _ptr(out), n,
                                         hidden, table.shape[0], c_float(scale), _ptr(status), self._stream()),
               "embedding")

    def logit_post(self, logits, scale: float = 1.0, soft_cap: Optional[float] = None):
        """In place: ``logits * scale``, then ``cap * tanh(. / cap)`` if a soft cap is given."""
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be contiguous fp32")
        _need(soft_cap is None or soft_cap > 0, "a soft cap must be positive")
        self.launches += 1
        _check(self.core.leone_logit_post(_ptr(logits), ctypes.c_longlong(logits.numel()), c_float(scale),
                                          c_float(soft_cap or 0.0), self._stream()), "logit_post")

    def rms_norm(self, x, weight, out, eps, rows=None):
        n_out, hidden = out.shape
        _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == hidden,
              "rms_norm input must be contiguous fp32 [*, hidden]")
        _need(weight.numel() == hidden and out.is_contiguous(), "rms_norm weight/output shape")
        if rows is not None:
            _need(rows.dtype == torch.int32 and rows.numel() == n_out, "rms_norm rows must be int32")
        else:
            _need(x.shape[0] >= n_out, "rms_norm input has fewer rows than the output")
        self.launches += 1
        _check(self.core.leone_rms_norm(_ptr(x), _ptr(rows), _ptr(weight), _dt(weight.dtype),
                                        _ptr(out), _dt(out.dtype), n_out, hidden, c_float(eps),
                                        self._stream()), "rms_norm")

    def _gemm_simt(self, x, w, out, epilogue, residual):
        m, k = x.shape
        n = w.shape[0]
        self.launches += 1
        _check(self.core.leone_gemm_simt(_dt(x.dtype), epilogue, _ptr(x), _ptr(w), _ptr(out),
                                         _ptr(residual), m, n, k, x.stride(0), w.stride(0),
                                         out.stride(0), self._stream()), "gemm_simt")

    def linear_fuses_norm(self, n_tokens: int, w: PreparedMatrix) -> bool:
        """True if a product of ``n_tokens`` tokens with ``w`` can take part in a fused RMSNorm:
        as the product before the norm (``linear(..., norm_out=d)`` also leaves
        ``d.xn = bf16(out * d.weight)`` and the sums of ``out^2`` in ``d.ss``) or as the one
        after it (``linear(d.xn, ..., norm_in=d)`` scales its rows by the norm's factor)."""
        wt = w.weight
        return (self.fast is not None and self.fast.fuses_norm(n_tokens, wt.shape[0], wt.shape[1])
                and wt.dtype == torch.bfloat16
                and wt.shape[0] % 8 == 0 and wt.shape[1] % 8 == 0 and wt.stride(0) % 8 == 0
                and wt.data_ptr() % 16 == 0)

    def norm_parts(self, n_tokens: int, n: int) -> int:
        """Rows of the ``ss`` buffer a product of ``n_tokens`` tokens with ``n`` outputs fills for
        the norm after it."""
        return self.fast.norm_parts(n_tokens, n)

    def _norm_args(self, m, w, norm_in, norm_out):
        ni = no = None
        if norm_in is not None:
            d = norm_in
            _need(self.linear_fuses_norm(m, w) and d.ss.dtype == torch.float32 and d.ss.is_contiguous()
                  and d.ss.shape == (d.parts, m), "linear: norm_in layout")
            ni = (d.ss, d.parts, d.eps)
        if norm_out is not None:
            d = norm_out
            _need(self.linear_fuses_norm(m, w) and d.weight.dtype == torch.float32 and d.weight.is_contiguous()
                  and d.weight.numel() == w.out_features and d.xn.dtype == torch.bfloat16
                  and d.xn.shape == (m, w.out_features) and d.xn.stride(1) == 1
                  and d.ss.dtype == torch.float32 and d.ss.is_contiguous()
                  and d.ss.shape == (self.norm_parts(m, w.out_features), m), "linear: norm_out layout")
            no = (d.xn, d.weight, d.ss)
        return ni, no

    def linear(self, x, w: PreparedMatrix, out, residual=None, norm_in=None, norm_out=None):
        """``out = x @ w.T`` (+ ``residual``).  ``out`` in x's dtype, or fp32 (then a fp32
        ``residual`` may be added; it may be ``out`` itself).  ``norm_in`` / ``norm_out``: see
        :meth:`linear_fuses_norm`."""
        m, k = x.shape
        _need(k == w.in_features and out.shape == (m, w.out_features), "linear: shapes do not chain")
        _need(x.dtype == w.dtype and x.stride(1) == 1 and out.stride(1) == 1, "linear: dtype/stride")
        if residual is not None:
            _need(out.dtype == torch.float32 and residual.dtype == torch.float32
                  and residual.shape == out.shape and residual.stride() == out.stride(),
                  "linear: a residual needs fp32 output of the same layout")
            epilogue = 2
        elif out.dtype == torch.float32 and x.dtype != torch.float32:
            epilogue = 1
        else:
            _need(out.dtype == x.dtype, "linear: output dtype")
            epilogue = 0
        if m == 0:
            return
        if norm_in is not None or norm_out is not None:
            _need(norm_out is None or epilogue in (1, 2), "linear: norm_out needs fp32 output")
            ni, no = self._norm_args(m, w, norm_in, norm_out)
            _need(self.fast.linear(x, w, out, epilogue, residual, ni, no), "linear: fused norm off the tensor-core path")
            self.launches += 1
            return
        if self.fast is not None and self.fast.linear(x, w, out, epilogue, residual):
            self.launches += 1
            return
        self._gemm_simt(x, w.weight, out, epilogue, residual)

    def linear_swiglu(self, x, w_gate_up: PreparedMatrix, out, norm_in=None):
        """``out = silu(x @ gate.T) * (x @ up.T)`` for a matrix from ``prepare_gate_up``."""
        m = x.shape[0]
        inter = w_gate_up.out_features // 2
        _need(out.shape == (m, inter) and out.dtype == x.dtype and out.is_contiguous(),
              "linear_swiglu: output shape")
        if m == 0:
            return
        if norm_in is not None:
            ni, _ = self._norm_args(m, w_gate_up, norm_in, None)
            _need(self.fast.linear_swiglu(x, w_gate_up, out, ni), "linear_swiglu: fused norm off the tensor-core path")
            self.launches += 1
            return
        if self.fast is not None and self.fast.linear_swiglu(x, w_gate_up, out):
            self.launches += 1
            return
        _need(getattr(w_gate_up, "gate_up_layout", None) == "stacked", "gate/up layout")
        scratch = self._scratch("gate_up", m, 2 * inter, x.dtype)
        self._gemm_simt(x, w_gate_up.weight, scratch, 0, None)
        self.launches += 1
        _check(self.core.leone_swiglu(_dt(x.dtype), _ptr(scratch), _ptr(out), m, inter,
                                      self._stream()), "swiglu")

    def swiglu(self, gate_up, out):
        m, two_i = gate_up.shape
        _need(out.shape == (m, two_i // 2) and gate_up.is_contiguous() and out.is_contiguous(),
              "swiglu shapes")
        self.launches += 1
        _check(self.core.leone_swiglu(_dt(gate_up.dtype), _ptr(gate_up), _ptr(out), m, two_i // 2,
                                      self._stream()), "swiglu")

    _scratch_bufs = None

    def _scratch(self, name, rows, cols, dtype):
        if self._scratch_bufs is None:
            self._scratch_bufs = {}
        key = (name, cols, dtype)
        buf = self._scratch_bufs.get(key)
        if buf is None or buf.shape[0] < rows:
            if buf is not None:
                self._scratch_bufs[("retired", id(buf))] = buf     # a captured graph may still use it
            buf = torch.empty((max(rows, 64), cols), dtype=dtype, device=self.device)
            self._scratch_bufs[key] = buf
        return buf[:rows]

    def qk_norm_rope_write(self, ctx, qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, table,
                           rotary_dim, cache, pairing="half_split"):
        """``pairing``: which elements of a head form rotation pair ``i``: ``(i, i + rotary_dim/2)``
        ("half_split") or ``(2i, 2i + 1)`` ("adjacent")."""
        _need(pairing in ("half_split", "adjacent"), f"rotary pairing '{pairing}'")
        n = qkv.shape[0]
        _need(qkv.is_contiguous() and qkv.shape[1] == (n_q + 2 * n_kv) * d, "qkv layout")
        w_dtype = 0
        if q_norm_w is not None:
            _need(k_norm_w is not None and q_norm_w.dtype == k_norm_w.dtype
                  and q_norm_w.numel() == d and k_norm_w.numel() == d, "q/k norm weights")
            w_dtype = _dt(q_norm_w.dtype)
        max_pos = 0
        if table is not None:
            _need(table.dtype == torch.float32 and table.is_contiguous() and table.dim() == 3
                  and table.shape[1] * 2 == rotary_dim and table.shape[2] == 2, "rotary table layout")
            max_pos = table.shape[0]
        if cache is not None:
            kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
            _need(kp.is_contiguous() and vp.is_contiguous() and kp.dtype == qkv.dtype
                  and kp.shape[1] == n_kv and kp.shape[3] == d and kp.shape[2] == cache.page_tokens,
                  "cache pool layout")
            _need(bt.dtype == torch.int32 and bt.is_contiguous(), "block table")
            pool_args = (_ptr(bt), bt.shape[1], bt.shape[0], _ptr(kp), _ptr(vp), kp.shape[0],
                         cache.page_tokens)
        else:
            pool_args = (c_void_p(0), 0, 0, c_void_p(0), c_void_p(0), 0, 0)
        self.launches += 1
        _check(self.core.leone_qk_norm_rope_write(
            _dt(qkv.dtype), _ptr(qkv), n, n_q, n_kv, d, _ptr(q_norm_w), _ptr(k_norm_w), w_dtype,
            c_float(eps), _ptr(table), rotary_dim, max_pos, _ptr(ctx.positions),
            _ptr(ctx.seq_of_token), pool_args[0], pool_args[1], pool_args[2], pool_args[3],
            pool_args[4], pool_args[5], pool_args[6], 1 if pairing == "adjacent" else 0, _ptr(ctx.status),
            self._stream()), "qk_norm_rope_write")

    def can_fuse_decode(self, ctx, qkv, n_q, n_kv, d) -> bool:
        """True if the attention kernel can do the q/k norm, rotation and cache write itself
        for this step (then ``qk_norm_rope_write`` is not called and ``attention`` gets
        ``fuse``: q_w, k_w (fp32 [d] or None), eps, rope ([positions, d/2, 2] fp32 or None),
        write_cache, and optionally pairing ("half_split" or "adjacent"))."""
        return self.fast is not None and self.fast.decode_fusable(ctx, qkv.dtype, n_q, n_kv, d, qkv.stride(0))

    def attention(self, ctx, qkv, out, n_q, n_kv, d, scale, window, cache, fuse=None):
        n = qkv.shape[0]
        kp, vp, bt = cache.k_pool, cache.v_pool, cache.block_table
        _need(out.shape == (n, n_q * d) and out.is_contiguous() and out.dtype == qkv.dtype,
              "attention output layout")
        _need(kp.is_contiguous() and vp.is_contiguous() and kp.dtype == qkv.dtype
              and kp.shape[1] == n_kv and kp.shape[3] == d, "cache pool layout")
        if self.fast is not None and self.fast.attention(ctx, qkv, out, n_q, n_kv, d, scale,
                                                         window, cache, fuse):
            self.launches += 1
            return
        _need(fuse is None, "the any-size attention kernel needs q/k norm and cache write done before")
        self.launches += 1
        _check(self.core.leone_attention_generic(
            _dt(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(kp), _ptr(vp),
            _ptr(bt), bt.shape[1], _ptr(ctx.seq_of_token), _ptr(ctx.positions), n, n_q, n_kv, d,
            c_float(scale), int(window or 0), cache.page_tokens, kp.shape[0], bt.shape[0],
            _ptr(ctx.status), self._stream()), "attention_generic")

    def sample(self, logits, temperature, seeds, positions, out):
        rows, vocab = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be fp32")
        _need(temperature.dtype == torch.float32 and seeds.dtype == torch.int64
              and positions.dtype == torch.int64 and out.dtype == torch.int32, "sample arguments")
        _need(temperature.numel() >= rows and seeds.numel() >= rows and positions.numel() >= rows
              and out.numel() >= rows, "sample argument lengths")
        self.launches += 1
        _check(self.core.leone_sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(seeds),
                                      _ptr(positions), _ptr(out), self._stream()), "sample")

    def sample_slots(self, logits, slot_ids, records, out):
        """One token per row with the row's temperature, seed and position taken from the slot
        record of its request (``records``: int64 ``[slots, 8]`` on the device, see
        :mod:`leone_b200.cache.slots`)."""
        rows, vocab = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be fp32")
        _need(slot_ids.dtype == torch.int32 and slot_ids.numel() >= rows and records.dtype == torch.int64
              and records.is_contiguous() and records.shape[1] == 8 and out.dtype == torch.int32
              and out.numel() >= rows, "sample_slots arguments")
        self.launches += 1
        _check(self.core.leone_sample_slots(_ptr(logits), rows, vocab, _ptr(slot_ids), _ptr(records), _ptr(out),
                                            self._stream()), "sample_slots")

    def penalize(self, logits, entries, penalties):
        """Penalties from the decode history, in place: ``entries`` lists (row, token, occurrences
        in the row's window, DRY penalty), each (row, token) once; ``penalties[row]`` holds the
        row's repetition, presence and frequency factors (``csrc/sampling_pipeline.cu``)."""
        rows, vocab = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be fp32")
        _need(len(penalties) == rows and all(0 <= e[0] < rows for e in entries), "penalize: rows")
        dev = self.device
        ints = torch.tensor([[e[0] for e in entries], [e[1] for e in entries], [e[2] for e in entries]],
                            dtype=torch.int32, device=dev)
        dry = torch.tensor([e[3] for e in entries], dtype=torch.float64, device=dev)
        per_row = torch.tensor([[p.repetition for p in penalties], [p.presence for p in penalties],
                                [p.frequency for p in penalties]], dtype=torch.float64, device=dev)
        self.launches += 1
        _check(self.core.leone_penalize(_ptr(logits), vocab, len(entries), _ptr(ints[0]), _ptr(ints[1]),
                                        _ptr(ints[2]), _ptr(dry), _ptr(per_row[0]), _ptr(per_row[1]),
                                        _ptr(per_row[2]), self._stream()), "penalize")

    def sample_truncated(self, logits, temperatures, seeds, positions, stages, want_probs: bool = False,
                         maximum_surprise=None, rows=None, out=None):
        """Rows that sample through truncation stages: ``stages`` is a list of (stage number,
        value) applied in order to every row (``csrc/sampling_pipeline.cu``).  ``rows``: which
        rows of ``logits`` take part (default: all); their ids are written to ``out`` at the same
        row numbers (``out``: int32 device tensor with a place per logits row; default: a new
        one).  Returns ``out`` (and the fp64 distribution the draws were made from, one row per
        participating row).  ``maximum_surprise`` (one per participating row): Mirostat's filter
        after the stages; the drawn tokens' probabilities before that filter are returned too
        (fp64 device tensor).  A row whose logits are all non-finite gets the id -1."""
        import ctypes
        n_rows, vocab = logits.shape
        members = list(range(n_rows)) if rows is None else [int(r) for r in rows]
        count = len(members)
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logits must be fp32")
        _need(count == len(temperatures) == len(seeds) == len(positions), "one temperature, seed and position a row")
        _need(all(0 <= r < n_rows for r in members) and len(set(members)) == count, "rows must be distinct rows of the logits")
        _need(all(t > 0 for t in temperatures), "truncation stages need a temperature")
        self.core.leone_sample_truncated_scratch.restype = ctypes.c_longlong
        need = int(self.core.leone_sample_truncated_scratch(count, vocab))
        if self._sample_scratch is None or self._sample_scratch.numel() < need:
            self._sample_scratch = torch.empty(need, dtype=torch.uint8, device=self.device)
        dev = self.device
        t = torch.tensor(temperatures, dtype=torch.float64, device=dev)
        sd = torch.tensor(np.array([s_ & 0xFFFF_FFFF_FFFF_FFFF for s_ in seeds], dtype=np.uint64).view(np.int64),
                          device=dev)
        pos = torch.tensor(positions, dtype=torch.int64, device=dev)
        row_map = None if rows is None else torch.tensor(members, dtype=torch.int32, device=dev)
        if out is None:
            out = torch.empty(n_rows, dtype=torch.int32, device=dev)
        _need(out.dtype == torch.int32 and out.numel() >= n_rows and out.is_contiguous(), "out: int32, a place per logits row")
        probs = torch.empty((count, vocab), dtype=torch.float64, device=dev) if want_probs else None
        mu = chosen = None
        if maximum_surprise is not None:
            _need(len(maximum_surprise) == count, "one maximum surprise a row")
            mu = torch.tensor([float(m) for m in maximum_surprise], dtype=torch.float64, device=dev)
            chosen = torch.zeros(count, dtype=torch.float64, device=dev)
        n = len(stages)
        types = (ctypes.c_int * max(n, 1))(*[int(a) for a, _ in stages])
        values = (ctypes.c_double * max(n, 1))(*[float(b) for _, b in stages])
        self.launches += 1
        _check(self.core.leone_sample_truncated(_ptr(logits), count, vocab, _ptr(t), _ptr(sd), _ptr(pos), n,
                                                types, values, _ptr(self._sample_scratch), _ptr(out),
                                                _ptr(probs), _ptr(mu), _ptr(chosen), _ptr(row_map), self._stream()),
               "sample_truncated")
        result = (out,) + ((probs,) if want_probs else ()) + ((chosen,) if mu is not None else ())
        return result if len(result) > 1 else out

    def decode_advance(self, token_ids, positions, ctx_len, sample_pos, sampled, history, counter,
                       slot_ids=None, records=None):
        """Feeds the sampled ids back as the next step's inputs.  Either ``sample_pos`` (int64 per
        row) is advanced, or, with ``slot_ids`` and ``records``, each request's slot record."""
        n = token_ids.numel()
        _need(history.dtype == torch.int32 and history.shape[1] == n and counter.dtype == torch.int32,
              "decode_advance arguments")
        if records is not None:
            _need(sample_pos is None and slot_ids is not None and slot_ids.dtype == torch.int32
                  and records.dtype == torch.int64 and records.shape[1] == 8, "decode_advance: slot records")
        else:
            _need(sample_pos is not None and sample_pos.dtype == torch.int64, "decode_advance: sample positions")
        self.launches += 1
        _check(self.core.leone_decode_advance(_ptr(token_ids), _ptr(positions), _ptr(ctx_len),
                                              _ptr(sample_pos), _ptr(sampled), _ptr(history),
                                              _ptr(counter), n, history.shape[0], _ptr(slot_ids), _ptr(records),
                                              self._stream()),
               "decode_advance")

"""Interfaces of the parts a layer is built from.

A part is constructed from ``(PartSpec.params, Runtime)`` and never learns
which model it is in.  It names the tensors it needs (:class:`WeightSpec`,
relative to the layer's prefix), receives them in ``load`` and runs in
``forward``.  Kinds are looked up in the registries of
:mod:`leone_b200.registry`.

Interfaces, by kind:

``Norm.forward(ctx, hidden, rows=None) -> Tensor``
    ``hidden`` is the fp32 residual stream ``[N, size]``; returns the normed
    rows in the run dtype (``rows``: optional int32 device indices to gather).

``Mixer.forward(ctx, cache, x, hidden) -> None``
    ``x`` are the normed tokens ``[N, hidden]``; the mixer adds its output to the
    fp32 ``hidden`` in place.  Optional fusion of the norms around it: a mixer
    that sets ``accepts_deferred_norm`` may be given a :class:`DeferredNorm`
    as ``x``; one that sets ``fuses_following_norm`` takes ``then=`` (the
    :class:`DeferredNorm` of the norm after its residual add, or ``None``).  ``cache`` is what ``cache_request()`` asked
    for: a :class:`PagedCacheView`, a :class:`StateView` or ``None``.

``FeedForward.forward(ctx, x, hidden) -> None``
    Same contract without a cache.

``PositionEncoding``
    Either offers ``rotary_table()`` (a ``[max_positions, rotary_dim/2, 2]``
    fp32 cos/sin table that an attention kernel applies itself, with
    ``pairing`` saying which elements form a pair) or implements
    ``apply(ctx, q, k)`` on ``[N, heads, head_dim]`` views in place.

``Block.forward(ctx, cache, hidden) -> None``
    The arrangement of norm, mixer and feed-forward around the residual stream.

``Embedding.forward(ctx, hidden) -> None`` / ``Head.forward(ctx, x, out) -> None``
    What stands before the first layer (token ids → fp32 residual stream) and after the final
    norm (normed wanted rows → fp32 logits).  A multiplier, learned positions added to the
    token rows, a logit scale or soft cap live in parts of these two kinds.

A mixer whose ``__init__`` takes a ``position_encodings`` keyword is given the model's named
position encodings (a dict) when it is built; one without it is built from ``(params, rt)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part reads.  ``role`` decides dtype policy and random init:

    ``matrix``/``embedding``: kept in the run dtype, drawn N(0, std);
    ``norm``: a 32-bit tensor stays 32-bit, drawn 1 + N(0, std);
    ``vector``: like ``norm`` but drawn N(0, std);
    ``int_table``: int32.
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    std: float = 0.02


@dataclass
class PagedKV:
    """A mixer's request for a paged cache: per token and KV head one key row of ``head_dim``
    elements and one value row of ``value_head_dim`` elements.

    ``value_head_dim``: ``None`` = as wide as the key; 0 = no value pool at all (a mixer that
    caches one vector per token, a latent, and derives the rest).  ``dtype``: storage dtype of
    the pages (``None`` = the run dtype).  ``lifetime``: when pages go back to the pool:
    ``"full"`` (at the request's end) or ``"window"`` (as soon as every later query lies more
    than ``window`` tokens past the page); ``None`` = ``"window"`` if a window is given.
    ``tag``: requests with different tags never share a group (a pool and a block table).
    Layers whose requests are equal share a group."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_head_dim: Optional[int] = None
    dtype: Optional[torch.dtype] = None
    lifetime: Optional[str] = None
    tag: str = ""

    def resolved(self, run_dtype: torch.dtype) -> "PagedKV":
        lifetime = self.lifetime or ("window" if self.window else "full")
        if lifetime not in ("full", "window"):
            raise ValueError(f"a paged cache's lifetime is 'full' or 'window', not '{lifetime}'")
        if lifetime == "window" and not self.window:
            raise ValueError("a paged cache with lifetime 'window' needs a window")
        vd = self.head_dim if self.value_head_dim is None else int(self.value_head_dim)
        if self.num_kv_heads <= 0 or self.head_dim <= 0 or vd < 0:
            raise ValueError(f"a paged cache needs positive sizes, got {self}")
        return PagedKV(self.num_kv_heads, self.head_dim, self.window if lifetime == "window" else None,
                       vd, self.dtype or run_dtype, lifetime, self.tag)


@dataclass
class FixedState:
    """A mixer's request for fixed-size per-request state, ``shape`` per request, fp32."""
    shape: Tuple[int, ...]


@dataclass
class PagedCacheView:
    """What a mixer sees of a paged group for one layer in one step."""
    k_pool: torch.Tensor          # [pages, kv_heads, page_tokens, head_dim]
    v_pool: Optional[torch.Tensor]  # [pages, kv_heads, page_tokens, value_head_dim]; None if the request had no values
    block_table: torch.Tensor     # int32 [B, max_blocks]; -1 where no page
    page_tokens: int
    writes: bool = True           # False for a layer that borrows another layer's cache


@dataclass
class StateView:
    """Fixed-size state for one layer: row ``slot`` belongs to the request in that slot."""
    state: torch.Tensor           # [num_slots, *shape] fp32
    writes: bool = True


@dataclass
class DeferredNorm:
    """An RMSNorm folded into the products around it instead of run as a kernel.

    The part whose last product writes the residual stream (``fuses_following_norm``) is handed
    this object as ``then``; if its product can, it calls :meth:`prepare`, passes the object as
    ``norm_out`` (the product then also leaves ``xn = bf16(hidden * weight)`` and the sums of
    ``hidden^2`` in ``ss``) and sets ``ready``.  The part that consumes the normed tokens
    (``accepts_deferred_norm``) is given the object instead of a tensor: if ``ready`` it feeds
    ``xn`` to its first product with ``norm_in=self``; otherwise it calls :meth:`materialize`,
    which runs the norm as a kernel of its own."""
    norm: "Norm"
    ctx: object
    hidden: torch.Tensor
    weight: torch.Tensor          # fp32
    eps: float
    tag: str = "a"                # names the buffers: two deferred norms alive together differ in it
    xn: Optional[torch.Tensor] = None
    ss: Optional[torch.Tensor] = None
    parts: int = 0
    ready: bool = False

    def prepare(self, rt, parts: int) -> None:
        """Buffers for a step of ``n`` tokens: ``xn [n, size]`` and the partial sums ``ss
        [parts, n]``, a view of one flat allocation per tag that is large enough for any step
        (``parts`` never exceeds the row width; a step never exceeds ``rt.max_tokens``), so its
        address is the same for every step size and a captured graph keeps seeing it."""
        n, size = self.hidden.shape
        self.parts = parts
        self.xn = rt.buffer(f"deferred_norm_x_{self.tag}", n, size, rt.dtype)
        # up to 32 tokens a part is 32 weight rows (parts * n <= size); prompt-sized steps have a
        # part per tile of at least 240 weight rows: reserve for the larger of the two at once
        flat = rt.flat_buffer(f"deferred_norm_ss_{self.tag}", parts * n, torch.float32,
                              reserve=max(size, (size // 240 + 2) * rt.max_tokens))
        self.ss = flat[:parts * n].view(parts, n)

    def materialize(self) -> torch.Tensor:
        return self.norm.forward(self.ctx, self.hidden)


class Runtime:
    """What every part gets at construction: device, run dtype, kernels and scratch buffers."""

    def __init__(self, device, dtype: torch.dtype, ops, max_tokens: int):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype
        self.ops = ops
        self.max_tokens = max_tokens
        self._buffers: Dict[str, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}

    def buffer(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """A scratch ``[rows, cols]`` view; one allocation per name, sized for ``max_tokens`` rows.

        The contents are whatever the last user left.  Two buffers of different
        names never overlap; the same name is the same memory.
        """
        vkey = (name, rows, cols, dtype)
        view = self._views.get(vkey)                  # a step asks for the same views layer after layer
        if view is not None:
            return view
        cap_rows = max(rows, self.max_tokens)
        key = f"{name}/{cols}/{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < cap_rows:
            if buf is not None:
                self._buffers[f"retired/{id(buf)}"] = buf    # a captured graph may still use it
            buf = torch.empty((cap_rows, cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self._views.clear()
        if len(self._views) > 4096:
            self._views.clear()
        view = self._views[vkey] = buf[:rows]
        return view


    def flat_buffer(self, name: str, numel: int, dtype: torch.dtype, reserve: int = 0) -> torch.Tensor:
        """A scratch vector of at least ``numel`` elements under ``name`` (``reserve``: what to
        allocate at once, so that later, larger asks need no new allocation).  It only ever
        grows (by at least a factor of two), and an outgrown allocation is kept alive for
        captured graphs that may still use it."""
        key = f"flat/{name}/{dtype}"
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._buffers[f"retired/{id(buf)}"] = buf
            cap = max(numel, reserve, 2 * buf.numel() if buf is not None else 0)
            buf = torch.empty(cap, dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf

    def allocated_bytes(self) -> int:
        """Bytes of all scratch buffers alive (retired ones included)."""
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class Part:
    def __init__(self, params: dict, rt: Runtime):
        self.params = params
        self.rt = rt

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def scratch_bytes(self, max_tokens: int) -> int:
        """Bytes of scratch buffers this part asks the runtime for in a step of ``max_tokens``
        tokens (an estimate for the memory budget that is checked before anything is loaded)."""
        return 0

    def load_transient_bytes(self) -> int:
        """Bytes ``load`` holds on top of the tensors it was given while it runs (a fused copy
        next to its sources); for the same budget."""
        return 0


class Norm(Part):
    def forward(self, ctx, hidden, rows=None):
        raise NotImplementedError

    def defer(self, ctx, hidden, tag="a") -> Optional[DeferredNorm]:
        """A :class:`DeferredNorm` if this norm is ``x * w / sqrt(mean(x^2) + eps)`` and may be
        folded into the products around it; ``None`` (the default) if it must run itself."""
        return None


class Mixer(Part):
    # True if ``forward`` copes with ``x`` being a DeferredNorm instead of the normed tokens
    accepts_deferred_norm = False
    # True if ``forward`` takes ``then=DeferredNorm`` (the norm that follows its residual add)
    fuses_following_norm = False

    def cache_request(self):
        return None

    def forward(self, ctx, cache, x, hidden):
        raise NotImplementedError


class FeedForward(Part):
    accepts_deferred_norm = False     # as for Mixer
    fuses_following_norm = False

    def forward(self, ctx, x, hidden):
        raise NotImplementedError


class PositionEncoding(Part):
    pairing: Optional[str] = None

    def rotary_table(self) -> Optional[torch.Tensor]:
        return None

    def apply(self, ctx, q, k):
        raise NotImplementedError


class Embedding(Part):
    """Token ids → the fp32 residual stream.  Its tensors are named in full (no layer prefix).
    ``params`` always hold ``vocab_size`` and ``hidden_size``."""

    def forward(self, ctx, hidden) -> None:
        """Fill ``hidden`` (fp32 ``[N, hidden_size]``) for the step's ``ctx.token_ids`` (at
        ``ctx.positions``); an id outside the vocabulary sets ``ctx.status`` and zeroes the row."""
        raise NotImplementedError

    def table(self) -> Optional[torch.Tensor]:
        """The ``[vocab, hidden]`` token table, for an output head that is tied to it."""
        return None


class Head(Part):
    """Normed rows → fp32 logits.  Its tensors are named in full.  ``params`` always hold
    ``vocab_size`` and ``hidden_size``."""

    def load(self, tensors: Dict[str, torch.Tensor], embedding: Optional[Embedding] = None) -> None:
        pass

    def forward(self, ctx, x, out) -> None:
        """``x``: the final norm's output for the wanted rows ``[M, hidden]`` in the run dtype;
        ``out``: fp32 ``[M, vocab]`` to fill."""
        raise NotImplementedError

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads here."""
        return 0


class Block:
    """``feed_forward`` and either norm are ``None`` where the layer's spec has none; further
    named parts of the layer (``LayerSpec.extra``) arrive as keyword arguments."""

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], mixer_norm: Optional[Norm],
                 ffn_norm: Optional[Norm], **extra):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm
        for name, part in extra.items():
            setattr(self, name, part)

    def forward(self, ctx, cache, hidden):
        raise NotImplementedError

"""The description of a model as data.

A :class:`ModelSpec` is what an architecture's ``build_spec(config)`` returns:
which parts each layer is made of (by registered kind name, each with its own
sizes and constants), and in which order layers run.  The engine builds the
model from this description only; it never asks which architecture it runs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the registered kind and the constants it is built with."""
    kind: str
    params: Dict[str, object] = field(default_factory=dict)

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement of a mixer, a feed-forward and their norms.

    ``prefix`` is the layer's tensor-name prefix in the checkpoint.  The feed-forward and either
    norm may be ``None`` for an arrangement that has none (the block then gets ``None`` in its
    place); ``extra`` holds further named parts of the arrangement, each as ``(registry, spec)``
    with ``registry`` one of ``"mixer"``, ``"feed_forward"``, ``"norm"`` (a second norm after the
    mixer, a parallel branch), given to the block as keyword arguments.
    ``cache_of`` names another layer whose cache this layer's mixer reads
    instead of owning one (it then writes nothing).  A layer named twice in the
    run order shares its weights between the runs; each run owns its own cache.
    """
    prefix: str
    block: str
    mixer: PartSpec
    feed_forward: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None
    cache_of: Optional[int] = None
    extra: Dict[str, Tuple[str, PartSpec]] = field(default_factory=dict)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_name: str                       # tensor name of the token table
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[int, ...]                # indices into ``layers``; may repeat
    final_norm: PartSpec
    final_norm_name: str
    lm_head_name: Optional[str]               # None: tied to the embedding table
    position_encodings: Dict[str, PartSpec] = field(default_factory=dict)
    eos_token_id: Optional[int] = None        # the first of ``eos_token_ids`` (kept for callers that want one)
    eos_token_ids: Tuple[int, ...] = ()       # every id that ends a request
    # What stands before the first layer and after the final norm.  ``None``: the built-in
    # ``token_embedding`` of ``embedding_name`` and ``linear_head`` of ``lm_head_name``.  The
    # engine adds ``vocab_size`` and ``hidden_size`` to the params of either.
    embedding: Optional[PartSpec] = None
    head: Optional[PartSpec] = None

    def embedding_spec(self) -> PartSpec:
        base = self.embedding or PartSpec("token_embedding", {"name": self.embedding_name})
        return PartSpec(base.kind, {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, **base.params})

    def head_spec(self) -> PartSpec:
        base = self.head or PartSpec("linear_head", {"name": self.lm_head_name})
        return PartSpec(base.kind, {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size, **base.params})

    def stop_ids(self) -> Tuple[int, ...]:
        if self.eos_token_ids:
            return tuple(self.eos_token_ids)
        return () if self.eos_token_id is None else (self.eos_token_id,)

    def validate(self) -> None:
        n = len(self.layers)
        if n == 0:
            raise ValueError("a model needs at least one layer")
        for idx in self.run_order:
            if not 0 <= idx < n:
                raise ValueError(f"run_order names layer {idx}, but there are {n} layers")
        first_run = {}
        for step, idx in enumerate(self.run_order):
            first_run.setdefault(idx, step)
        for i, layer in enumerate(self.layers):
            src = layer.cache_of
            if src is None:
                continue
            if not 0 <= src < n or src == i:
                raise ValueError(f"layer {i}: cache_of={src} is not another layer")
            if self.layers[src].cache_of is not None:
                raise ValueError(f"layer {i}: cache_of={src} which itself borrows a cache")
            if i in first_run and (src not in first_run or first_run[src] > first_run[i]):
                raise ValueError(
                    f"layer {i} reads layer {src}'s cache but runs before it writes")

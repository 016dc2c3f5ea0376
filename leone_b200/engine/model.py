"""A model built from a :class:`ModelSpec`: embedding, layers in run order, final norm, head.

The forward pass runs only the tokens of the step: the embedding part
(crates/leone/src/runtime.rs:6686-6692), the layers in ``run_order``, then the
final norm and the head part on the wanted rows only
(crates/leone/src/runtime.rs:7428-7452, 6542-6608).  A tied head reads the
embedding table (crates/leone/src/model.rs:452-471).  Embedding and head are
parts like the others, chosen by kind from the spec.
"""
from __future__ import annotations

import inspect
from typing import Dict, List, Optional

import torch

from .. import parts as _parts  # noqa: F401  (registers built-in parts)
from ..parts.base import FixedState, PagedKV, Runtime, WeightSpec
from ..parts.spec import ModelSpec
from ..registry import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                        spec_from_config)


class _Prefixed:
    """Gives a part its tensors under the names it declared, from the checkpoint's full names."""

    def __init__(self, prefix: str, part):
        self.prefix = prefix
        self.part = part

    def full_specs(self) -> List[WeightSpec]:
        return [WeightSpec(f"{self.prefix}.{s.name}", s.shape, s.role, s.std)
                for s in self.part.weight_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hands the part its tensors and takes them out of ``tensors``: what the part keeps it
        holds itself, what it fused into a copy is freed at once."""
        self.part.load({s.name: tensors.pop(f"{self.prefix}.{s.name}") for s in self.part.weight_specs()})


def _build_mixer(spec, rt, position_encodings):
    cls = MIXERS.get(spec.kind)
    if "position_encodings" in inspect.signature(cls.__init__).parameters:
        return cls(dict(spec.params), rt, position_encodings=position_encodings)
    return cls(dict(spec.params), rt)


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.position_encodings = {
            name: POSITION_ENCODINGS.get(ps.kind)(dict(ps.params), rt)
            for name, ps in spec.position_encodings.items()}
        self.blocks = []
        self._holders: List[_Prefixed] = []
        for layer in spec.layers:
            def build(registry, part_spec):
                if part_spec is None:
                    return None
                if registry == "mixer":
                    return _build_mixer(part_spec, rt, self.position_encodings)
                table = {"feed_forward": FEED_FORWARDS, "norm": NORMS}.get(registry)
                if table is None:
                    raise ValueError(f"layer {layer.prefix}: no registry '{registry}' for an extra part")
                return table.get(part_spec.kind)(dict(part_spec.params), rt)

            mixer = build("mixer", layer.mixer)
            ffn = build("feed_forward", layer.feed_forward)
            n1, n2 = build("norm", layer.mixer_norm), build("norm", layer.ffn_norm)
            extra = {name: build(registry, ps) for name, (registry, ps) in layer.extra.items()}
            block = BLOCKS.get(layer.block)(mixer, ffn, n1, n2, **extra)
            block.extra_parts = extra
            self.blocks.append(block)
            self._holders += [_Prefixed(layer.prefix, p) for p in (mixer, ffn, n1, n2, *extra.values())
                              if p is not None]
        self.final_norm = NORMS.get(spec.final_norm.kind)(
            {**spec.final_norm.params, "name": spec.final_norm_name}, rt)
        es, hs = spec.embedding_spec(), spec.head_spec()
        self.embedding = EMBEDDINGS.get(es.kind)(dict(es.params), rt)
        self.head = HEADS.get(hs.kind)(dict(hs.params), rt)

    # -- weights ----------------------------------------------------------------------
    def weight_specs(self) -> List[WeightSpec]:
        specs = list(self.embedding.weight_specs())
        for holder in self._holders:
            specs += holder.full_specs()
        specs += self.final_norm.weight_specs()
        specs += self.head.weight_specs()
        return specs

    def load_notes(self, names) -> List[str]:
        """Extra findings for the weight error that a part can name better than "unexpected
        tensor" (a tied head whose file still has a head tensor)."""
        notes: List[str] = []
        for part in (self.embedding, self.head):
            if hasattr(part, "load_notes"):
                notes += part.load_notes(names)
        return notes

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Gives every part its tensors; ``tensors`` is emptied on the way, so a source that a
        part fused into a copy of its own (q/k/v stacked, gate/up interleaved) is freed as soon
        as that part is loaded."""
        s = self.spec
        self.embedding.load({w.name: tensors.pop(w.name) for w in self.embedding.weight_specs()})
        for holder in self._holders:
            holder.load(tensors)
        self.final_norm.load({s.final_norm_name: tensors.pop(s.final_norm_name)})
        self.head.load({w.name: tensors.pop(w.name) for w in self.head.weight_specs()}, self.embedding)

    # -- cache needs ------------------------------------------------------------------
    def cache_plan(self):
        """Per position of ``run_order``: ``(request, source)``.

        A layer that is run twice shares its weights, not its cache: every occurrence in the
        run order owns a cache of its own (``request`` is a ``PagedKV``/``FixedState``,
        ``source`` is ``None``).  A layer with ``cache_of`` owns none and reads the cache of
        the latest earlier occurrence of that layer (``request`` is ``None``, ``source`` its
        run position)."""
        plan = []
        latest = {}
        for pos, idx in enumerate(self.spec.run_order):
            layer = self.spec.layers[idx]
            if layer.cache_of is None:
                plan.append((self.blocks[idx].mixer.cache_request(), None))
                latest[idx] = pos
            else:
                plan.append((None, latest[layer.cache_of]))
        return plan

    def decode_weight_bytes(self) -> int:
        """Bytes of weights one decode step reads: every layer once per run, the head once
        (the reference's per-step accounting, crates/leone/src/model.rs:306-323)."""
        total = 0
        for idx in self.spec.run_order:
            block = self.blocks[idx]
            for part in (block.mixer, block.feed_forward, *getattr(block, "extra_parts", {}).values()):
                if part is not None and hasattr(part, "weight_bytes"):
                    total += part.weight_bytes()
        total += self.head.weight_bytes()
        return total

    def scratch_bytes(self, max_tokens: int, max_logit_rows: int) -> int:
        """An estimate of the scratch a step of ``max_tokens`` tokens asks the runtime for: the fp32
        residual stream, the normed tokens (twice: a folded norm keeps its own copy), the largest
        layer's buffers (layers share them by name), fp32 logits for ``max_logit_rows`` rows, and what
        the ops keep for themselves."""
        item = self.rt.dtype.itemsize
        total = max_tokens * self.hidden_size * (4 + 3 * item)
        per_layer = [sum(p.scratch_bytes(max_tokens)
                         for p in (b.mixer, b.feed_forward, b.mixer_norm, b.ffn_norm,
                                   *getattr(b, "extra_parts", {}).values()) if p is not None)
                     for b in self.blocks]
        total += max(per_layer, default=0)
        total += max_logit_rows * (self.vocab_size * 4 + self.hidden_size * item)
        ops_scratch = getattr(self.rt.ops, "scratch_bytes", None)
        return total + (ops_scratch() if ops_scratch is not None else 0)

    def load_transient_bytes(self) -> int:
        """The most any one part holds beyond its inputs while it loads."""
        parts = [h.part for h in self._holders] + [self.embedding, self.head, self.final_norm]
        return max((p.load_transient_bytes() for p in parts), default=0)

    # -- forward ----------------------------------------------------------------------
    def forward(self, ctx) -> Optional[torch.Tensor]:
        # every launch of the step goes to the stream that is current now (looked up once)
        pin = getattr(self.rt.ops, "pin_stream", None)
        if pin is None:
            return self._forward(ctx)
        pin(True)
        try:
            return self._forward(ctx)
        finally:
            pin(False)

    def _forward(self, ctx) -> Optional[torch.Tensor]:
        rt = self.rt
        hidden = rt.buffer("hidden", ctx.n_tokens, self.hidden_size, torch.float32)
        self.embedding.forward(ctx, hidden)
        order = self.spec.run_order
        pre = None           # the entry norm of the next block, if the last product before it folded it in
        for pos, idx in enumerate(order):
            block = self.blocks[idx]
            if not getattr(block, "chains_norms", False):
                block.forward(ctx, ctx.cache_view(pos), hidden)
                pre = None
                continue
            after = None
            if pos + 1 < len(order) and getattr(self.blocks[order[pos + 1]], "chains_norms", False):
                after = self.blocks[order[pos + 1]].entry_norm(ctx, hidden)
            pre = block.forward(ctx, ctx.cache_view(pos), hidden, pre=pre, after=after)
        return self.logits(ctx, hidden)

    def logits(self, ctx, hidden) -> Optional[torch.Tensor]:
        m = ctx.n_logit_rows
        if m == 0:
            return None
        x = self.final_norm.forward(ctx, hidden, rows=ctx.logit_rows, out_name="final_normed")
        out = ctx.logits_out if ctx.logits_out is not None else torch.empty(
            (m, self.vocab_size), dtype=torch.float32, device=self.rt.device)
        self.head.forward(ctx, x, out)
        return out


def weight_specs_for_config(config) -> List[WeightSpec]:
    spec = spec_from_config(config)
    return Model(spec, Runtime("cpu", torch.float32, None, 0)).weight_specs()

"""Output head: ``logits = W x`` in fp32 for the wanted rows, optionally scaled and soft-capped.

A head without a tensor of its own (``name`` is ``None``) is tied: it reads the embedding's
token table (crates/leone/src/model.rs:452-471, crates/leone/src/runtime.rs:7442-7452).  The
reference has no logit scale, soft cap or bias; ``logit_scale`` and ``soft_cap`` are this
part's own parameters (``l * scale``, then ``cap * tanh(l / cap)``), off by default.
"""
from __future__ import annotations

from ..registry import HEADS
from .base import Head, WeightSpec


@HEADS.register("linear_head")
class LinearHead(Head):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = params.get("name")              # None: tied to the embedding table
        self.logit_scale = float(params.get("logit_scale", 1.0))
        cap = params.get("soft_cap")
        self.soft_cap = float(cap) if cap else None
        # the name an untied head's tensor would have: present in a tied model's file, it is a conflict
        self.tied_name = params.get("tied_name")
        self.weight = None

    def load_notes(self, names):
        if self.name is None and self.tied_name and self.tied_name in names:
            return [f"{self.tied_name} is present although the configuration ties the head to "
                    "the embedding table"]
        return []

    def weight_specs(self):
        return [] if self.name is None else [WeightSpec(self.name, (self.vocab, self.hidden))]

    def load(self, tensors, embedding=None):
        if self.name is not None:
            w = tensors[self.name]
        else:
            w = embedding.table() if embedding is not None else None
            if w is None:
                raise ValueError("a tied output head needs an embedding that offers its token table")
        self.weight = self.rt.ops.prepare_matrix(w)

    def weight_bytes(self):
        return self.vocab * self.hidden * self.rt.dtype.itemsize

    def forward(self, ctx, x, out):
        self.rt.ops.linear(x, self.weight, out)
        if self.logit_scale != 1.0 or self.soft_cap is not None:
            self.rt.ops.logit_post(out, self.logit_scale, self.soft_cap)

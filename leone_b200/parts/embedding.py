"""Token embedding: ``h[t, :] = scale * E[id_t, :]`` into the fp32 residual stream.

The reference gathers the row without a factor and treats an id outside the table as an error
(crates/leone/src/runtime.rs:7380-7386, 6686-6692; crates/leone/src/cpu.rs:1243-1265); ``scale``
(default 1) is this part's own parameter for models that multiply their embeddings.
"""
from __future__ import annotations

from ..registry import EMBEDDINGS
from .base import Embedding, WeightSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = params["name"]
        self.scale = float(params.get("scale", 1.0))
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.vocab, self.hidden), role="embedding")]

    def load(self, tensors):
        self.weight = tensors[self.name]

    def table(self):
        return self.weight

    def forward(self, ctx, hidden):
        if self.scale == 1.0:
            self.rt.ops.embedding(self.weight, ctx.token_ids, hidden, ctx.status)
        else:
            self.rt.ops.embedding(self.weight, ctx.token_ids, hidden, ctx.status, self.scale)

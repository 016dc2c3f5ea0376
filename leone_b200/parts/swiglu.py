"""Dense SwiGLU feed-forward: ``hidden += W_down (silu(W_gate x) * W_up x)``.

``silu(g) = g / (1 + exp(-g))`` in fp32 (crates/leone/src/cpu.rs:903-905);
order of operations crates/leone/src/runtime.rs:9298-9317.  Gate and up
matrices are stacked row-wise at load time so one product feeds both
(the reference pairs them in one launch too, ie_cuda.cu:1896-1931).
"""
from __future__ import annotations

import torch

from ..registry import FEED_FORWARDS
from .base import FeedForward, WeightSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.gate_name = params.get("gate_name", "gate_proj.weight")
        self.up_name = params.get("up_name", "up_proj.weight")
        self.down_name = params.get("down_name", "down_proj.weight")
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self):
        return [WeightSpec(self.gate_name, (self.inter, self.hidden)),
                WeightSpec(self.up_name, (self.inter, self.hidden)),
                WeightSpec(self.down_name, (self.hidden, self.inter))]

    def load(self, tensors):
        self.w_gate_up = self.rt.ops.prepare_gate_up(tensors[self.gate_name], tensors[self.up_name])
        self.w_down = self.rt.ops.prepare_matrix(tensors[self.down_name])

    def weight_bytes(self):
        return (2 * self.inter * self.hidden + self.hidden * self.inter) * self.rt.dtype.itemsize

    def forward(self, ctx, x, hidden):
        n = x.shape[0]
        act = self.rt.buffer("ffn_act", n, self.inter, self.rt.dtype)
        self.rt.ops.linear_swiglu(x, self.w_gate_up, act)
        self.rt.ops.linear(act, self.w_down, hidden, residual=hidden)

"""Dense SwiGLU feed-forward: ``hidden += W_down (silu(W_gate x) * W_up x)``.

``silu(g) = g / (1 + exp(-g))`` in fp32 (crates/leone/src/cpu.rs:903-905);
order of operations crates/leone/src/runtime.rs:9298-9317.  Gate and up
matrices are stacked row-wise at load time so one product feeds both
(the reference pairs them in one launch too, ie_cuda.cu:1896-1931).
"""
from __future__ import annotations

from ..registry import FEED_FORWARDS
from .base import DeferredNorm, FeedForward, WeightSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    accepts_deferred_norm = True
    fuses_following_norm = True

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

    def scratch_bytes(self, max_tokens):
        # the activation; a path without the fused epilogue also holds gate and up side by side
        return max_tokens * 3 * self.inter * self.rt.dtype.itemsize

    def load_transient_bytes(self):
        return 2 * self.inter * self.hidden * self.rt.dtype.itemsize       # gate and up beside their interleaved copy

    def forward(self, ctx, x, hidden, then=None):
        n = hidden.shape[0]
        ops = self.rt.ops
        act = self.rt.buffer("ffn_act", n, self.inter, self.rt.dtype)
        if isinstance(x, DeferredNorm):
            if x.ready and ops.linear_fuses_norm(n, self.w_gate_up):
                ops.linear_swiglu(x.xn, self.w_gate_up, act, norm_in=x)      # the norm's factor in the epilogue
            else:
                ops.linear_swiglu(x.materialize(), self.w_gate_up, act)
        else:
            ops.linear_swiglu(x, self.w_gate_up, act)
        if then is not None and hasattr(ops, "linear_fuses_norm") and ops.linear_fuses_norm(n, self.w_down):
            then.prepare(self.rt, ops.norm_parts(n, self.hidden))
            ops.linear(act, self.w_down, hidden, residual=hidden, norm_out=then)
            then.ready = True
        else:
            ops.linear(act, self.w_down, hidden, residual=hidden)

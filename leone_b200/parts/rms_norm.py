"""RMSNorm over the residual stream.

``y_c = x_c * w_c / sqrt(mean_c(x_c^2) + eps)`` with the sum of squares in
fp32; the weight multiplies directly, not as ``1 + w``
(crates/leone/src/cpu.rs:1642-1663; CUDA counterpart
crates/leone-cuda/cuda/ie_cuda.cu:2357-2380).
"""
from __future__ import annotations

from ..registry import NORMS
from .base import DeferredNorm, Norm, WeightSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = params.get("name", "weight")
        self.weight = self.weight_f32 = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.size,), role="norm", std=0.1)]

    def load(self, tensors):
        self.weight = tensors[self.name]
        self.weight_f32 = self.weight.float().contiguous()    # for a product that applies the norm itself

    def defer(self, ctx, hidden, tag="a"):
        return DeferredNorm(self, ctx, hidden, self.weight_f32, self.eps, tag)

    def forward(self, ctx, hidden, rows=None, out_name="normed"):
        n = hidden.shape[0] if rows is None else rows.shape[0]
        out = self.rt.buffer(out_name, n, self.size, self.rt.dtype)
        self.rt.ops.rms_norm(hidden, self.weight, out, self.eps, rows)
        return out

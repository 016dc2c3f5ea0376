"""Causal grouped-query attention over a paged cache.

One step of the reference's layer (crates/leone/src/runtime.rs:9111-9157):
``q, k, v = W_qkv x``; per-head RMSNorm of q and k with one weight ``[head_dim]``
shared by all heads and the layer's eps, v untouched
(crates/leone/src/model.rs:601-631, crates/leone/src/cpu.rs:802-820); rotary
on q and k; k and v written at their positions; for a query at absolute
position ``p`` the keys ``max(0, p-window+1) .. p`` are read with
``kv_head = q_head // (n_q / n_kv)``, ``score = (q.k) / sqrt(head_dim)``,
softmax and weighted sum in fp32 (crates/leone/src/cpu.rs:2299-2421); then
``hidden += W_o attn``.  The window is this part's own parameter (``None`` =
all keys); the reference has no windowed layer.

Every size is a parameter: number of heads, groups, head size (independent of
the hidden size), presence of the q/k norm, the position encoding and the
window.
"""
from __future__ import annotations

import math

import torch

from ..registry import MIXERS
from .base import DeferredNorm, Mixer, PagedKV, WeightSpec


@MIXERS.register("attention")
class Attention(Mixer):
    accepts_deferred_norm = True
    fuses_following_norm = True

    def __init__(self, params, rt, position_encodings=None):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.n_q = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        if self.n_q % self.n_kv:
            raise ValueError(f"num_heads {self.n_q} is not a multiple of num_kv_heads {self.n_kv}")
        self.qk_norm = bool(params.get("qk_norm", False))
        self.eps = float(params.get("qk_norm_eps", 1e-6))
        self.window = params.get("window")
        self.scale = float(params.get("scale", 1.0 / math.sqrt(self.d)))
        pe_name = params.get("position_encoding")
        self.pos = (position_encodings or {}).get(pe_name) if pe_name else None
        if pe_name and self.pos is None:
            raise ValueError(f"attention names position encoding '{pe_name}' that the model lacks")
        self.names = {k: params.get(f"{k}_name", f"{k}_proj.weight") for k in ("q", "k", "v", "o")}
        self.q_norm_name = params.get("q_norm_name", "q_norm.weight")
        self.k_norm_name = params.get("k_norm_name", "k_norm.weight")
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        self.qkv_cols = (self.n_q + 2 * self.n_kv) * self.d

    def weight_specs(self):
        specs = [WeightSpec(self.names["q"], (self.n_q * self.d, self.hidden)),
                 WeightSpec(self.names["k"], (self.n_kv * self.d, self.hidden)),
                 WeightSpec(self.names["v"], (self.n_kv * self.d, self.hidden)),
                 WeightSpec(self.names["o"], (self.hidden, self.n_q * self.d))]
        if self.qk_norm:
            specs += [WeightSpec(self.q_norm_name, (self.d,), role="norm", std=0.1),
                      WeightSpec(self.k_norm_name, (self.d,), role="norm", std=0.1)]
        return specs

    def load(self, tensors):
        stacked = torch.cat([tensors[self.names["q"]], tensors[self.names["k"]],
                             tensors[self.names["v"]]], dim=0).contiguous()
        self.w_qkv = self.rt.ops.prepare_matrix(stacked)
        self.w_o = self.rt.ops.prepare_matrix(tensors[self.names["o"]])
        self.q_norm_f32 = self.k_norm_f32 = None
        if self.qk_norm:
            self.q_norm_w = tensors[self.q_norm_name]
            self.k_norm_w = tensors[self.k_norm_name]
            # fp32 copies for the decode kernel that does the norm itself
            self.q_norm_f32 = self.q_norm_w.float().contiguous()
            self.k_norm_f32 = self.k_norm_w.float().contiguous()

    def weight_bytes(self):
        return (self.qkv_cols * self.hidden + self.hidden * self.n_q * self.d) * self.rt.dtype.itemsize

    def scratch_bytes(self, max_tokens):
        return max_tokens * (self.qkv_cols + self.n_q * self.d) * self.rt.dtype.itemsize

    def load_transient_bytes(self):
        return self.qkv_cols * self.hidden * self.rt.dtype.itemsize       # q, k, v beside their stacked copy

    def cache_request(self):
        return PagedKV(self.n_kv, self.d, self.window)

    def _out_proj(self, attn, hidden, then):
        """``hidden += W_o attn``; folds the norm that follows (``then``) into the product if it can."""
        ops = self.rt.ops
        n = hidden.shape[0]
        if then is not None and hasattr(ops, "linear_fuses_norm") and ops.linear_fuses_norm(n, self.w_o):
            then.prepare(self.rt, ops.norm_parts(n, self.hidden))
            ops.linear(attn, self.w_o, hidden, residual=hidden, norm_out=then)
            then.ready = True
        else:
            ops.linear(attn, self.w_o, hidden, residual=hidden)

    def forward(self, ctx, cache, x, hidden, then=None):
        rt = self.rt
        n = hidden.shape[0]
        qkv = rt.buffer("qkv", n, self.qkv_cols, rt.dtype)
        if isinstance(x, DeferredNorm):
            if x.ready and rt.ops.linear_fuses_norm(n, self.w_qkv):
                rt.ops.linear(x.xn, self.w_qkv, qkv, norm_in=x)          # the norm's factor in the epilogue
            else:
                rt.ops.linear(x.materialize(), self.w_qkv, qkv)
        else:
            rt.ops.linear(x, self.w_qkv, qkv)
        table, rotary_dim, pairing = None, 0, None
        if self.pos is not None:
            table = self.pos.rotary_table()
            if table is not None:
                rotary_dim, pairing = table.shape[1] * 2, self.pos.pairing
                if pairing not in ("half_split", "adjacent"):
                    raise ValueError(f"attention kernels rotate half-split or adjacent pairs, not '{pairing}'")
        attn = rt.buffer("attn_out", n, self.n_q * self.d, rt.dtype)
        # A decode step whose new key goes to this layer's own cache: the attention kernel may norm
        # and rotate q and the new k and write the cache itself.  (A layer that reads another
        # layer's cache takes every key from there, the newest too, so it is not fused.)
        fusable = cache.writes and (self.pos is None or (table is not None and rotary_dim == self.d))
        if fusable and hasattr(rt.ops, "can_fuse_decode") and \
                rt.ops.can_fuse_decode(ctx, qkv, self.n_q, self.n_kv, self.d):
            rt.ops.attention(ctx, qkv, attn, self.n_q, self.n_kv, self.d, self.scale, self.window, cache,
                             fuse=dict(q_w=self.q_norm_f32, k_w=self.k_norm_f32, eps=self.eps, rope=table,
                                       write_cache=True, pairing=pairing or "half_split"))
            self._out_proj(attn, hidden, then)
            return
        # q/k norm, rotation and the cache write are one kernel; an encoding without a
        # rotary table is applied by the encoding itself between norm and cache write.
        if self.pos is not None and table is None:
            rt.ops.qk_norm_rope_write(ctx, qkv, self.n_q, self.n_kv, self.d, self.q_norm_w,
                                      self.k_norm_w, self.eps, None, 0, None)
            q = qkv[:, :self.n_q * self.d].unflatten(1, (self.n_q, self.d))
            k = qkv[:, self.n_q * self.d:(self.n_q + self.n_kv) * self.d].unflatten(1, (self.n_kv, self.d))
            self.pos.apply(ctx, q, k)
            rt.ops.qk_norm_rope_write(ctx, qkv, self.n_q, self.n_kv, self.d, None, None,
                                      self.eps, None, 0, cache if cache.writes else None)
        else:
            extra = {} if pairing in (None, "half_split") else dict(pairing=pairing)
            rt.ops.qk_norm_rope_write(ctx, qkv, self.n_q, self.n_kv, self.d, self.q_norm_w,
                                      self.k_norm_w, self.eps, table, rotary_dim,
                                      cache if cache.writes else None, **extra)
        rt.ops.attention(ctx, qkv, attn, self.n_q, self.n_kv, self.d, self.scale,
                         self.window, cache)
        self._out_proj(attn, hidden, then)

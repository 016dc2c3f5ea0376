"""A stand-in for the CUDA kernel table, for tests that run without a GPU.

It implements the same calls as ``leone_b200.ops.cuda.CudaOps`` with plain
torch on the CPU, reading and writing the same paged pools through the same
block tables.  It lets the ``-m "not gpu"`` tests exercise the step function,
the cache manager and the scheduler end to end.  It is a test fixture only:
the engine never falls back to it.
"""
from __future__ import annotations

import math

import numpy as np
import torch


class EmulatedOps:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype
        self.calls = []

    # -- weights ------------------------------------------------------------------------
    def prepare_matrix(self, w):
        return w

    def prepare_gate_up(self, gate, up):
        return torch.cat([gate, up], dim=0).contiguous()

    def describe_status(self, word):
        return f"emulated status {word}"

    # -- kernels ------------------------------------------------------------------------
    def embedding(self, table, ids, out, status, scale=1.0):
        out.copy_(table[ids.long()].float() * scale)

    def logit_post(self, logits, scale=1.0, soft_cap=None):
        logits.mul_(scale)
        if soft_cap:
            logits.copy_(soft_cap * torch.tanh(logits / soft_cap))

    def rms_norm(self, x, weight, out, eps, rows=None):
        src = x if rows is None else x[rows.long()]
        src = src.float()
        ms = (src * src).mean(dim=-1, keepdim=True)
        out.copy_((src * weight.float() * torch.rsqrt(ms + eps)).to(out.dtype))

    def linear(self, x, w, out, residual=None):
        y = x.float() @ w.float().t()
        if residual is not None:
            y = y + residual
        out.copy_(y.to(out.dtype))

    def linear_swiglu(self, x, w_gate_up, out):
        y = x.float() @ w_gate_up.float().t()
        inter = y.shape[1] // 2
        if self.dtype != torch.float32:
            y = y.to(self.dtype).float()
        g, u = y[:, :inter], y[:, inter:]
        out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))

    def qk_norm_rope_write(self, ctx, qkv, n_q, n_kv, d, q_norm_w, k_norm_w, eps, table,
                           rotary_dim, cache, pairing="half_split"):
        n = qkv.shape[0]
        x = qkv.float().view(n, n_q + 2 * n_kv, d)
        q, k, v = x[:, :n_q], x[:, n_q:n_q + n_kv], x[:, n_q + n_kv:]

        def norm(t, w):
            if w is None:
                return t
            ms = (t * t).mean(dim=-1, keepdim=True)
            return t * w.float() * torch.rsqrt(ms + eps)

        def rope(t):
            if table is None:
                return t
            half = rotary_dim // 2
            cs = table[ctx.positions.long()]          # [n, half, 2]
            cos, sin = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
            out = t.clone()
            if pairing == "adjacent":
                a, b = t[..., 0:rotary_dim:2], t[..., 1:rotary_dim:2]
                out[..., 0:rotary_dim:2] = a * cos - b * sin
                out[..., 1:rotary_dim:2] = a * sin + b * cos
                return out
            a, b = t[..., :half], t[..., half:rotary_dim]
            out[..., :half] = a * cos - b * sin
            out[..., half:rotary_dim] = a * sin + b * cos
            return out

        q = rope(norm(q, q_norm_w))
        k = rope(norm(k, k_norm_w))
        new = torch.cat([q, k, v], dim=1).reshape(n, -1).to(qkv.dtype)
        qkv.copy_(new)
        if cache is None:
            return
        kk = new.view(n, n_q + 2 * n_kv, d)[:, n_q:n_q + n_kv]
        vv = new.view(n, n_q + 2 * n_kv, d)[:, n_q + n_kv:]
        pt = cache.page_tokens
        pos = ctx.positions.long()
        seq = ctx.seq_of_token.long()
        page = cache.block_table[seq, pos // pt].long()
        assert (page >= 0).all(), "write into a block without a page"
        cache.k_pool[page, :, pos % pt, :] = kk
        cache.v_pool[page, :, pos % pt, :] = vv

    def attention(self, ctx, qkv, out, n_q, n_kv, d, scale, window, cache):
        n = qkv.shape[0]
        q = qkv.float().view(n, n_q + 2 * n_kv, d)[:, :n_q]
        g = n_q // n_kv
        pt = cache.page_tokens
        res = torch.zeros(n, n_q, d)
        positions = ctx.positions.tolist()
        seqs = ctx.seq_of_token.tolist()
        for t in range(n):
            p, s = positions[t], seqs[t]
            lo = 0 if not window else max(0, p - window + 1)
            idx = torch.arange(lo, p + 1)
            pages = cache.block_table[s, idx // pt].long()
            assert (pages >= 0).all(), "read from a block without a page"
            keys = cache.k_pool[pages, :, idx % pt, :].float()      # [ctx, n_kv, d]
            vals = cache.v_pool[pages, :, idx % pt, :].float()
            for h in range(n_q):
                sc = (keys[:, h // g, :] @ q[t, h]) * scale
                w = torch.softmax(sc, dim=0)
                res[t, h] = (w[:, None] * vals[:, h // g, :]).sum(0)
        out.copy_(res.reshape(n, n_q * d).to(out.dtype))

    def sample(self, logits, temperature, seeds, positions, out):
        from tests.plain.model import sample
        for i in range(logits.shape[0]):
            out[i] = sample(logits[i].tolist(), float(temperature[i]), int(seeds[i]), int(positions[i]))

    def penalize(self, logits, entries, penalties):
        for row, token, count, dry in entries:
            p = penalties[row]
            value = logits[row, token].item()
            if count > 0 and (p.repetition != 1.0 or p.presence != 0.0 or p.frequency != 0.0):
                v = float(value)
                v = v / p.repetition if v > 0.0 else v * p.repetition
                v = v - p.presence - p.frequency * count
                value = float(np.float32(v))
            if dry > 0.0:
                value = float(np.float32(float(value) - dry))
            logits[row, token] = value

    def sample_truncated(self, logits, temperatures, seeds, positions, stages, want_probs=False,
                         maximum_surprise=None, rows=None, out=None):
        from leone_b200.sampling.sampler import TRUNCATION_STAGES
        from tests.plain.model import mirostat_select, select, truncated_probs, uniform
        import math
        names = {v: k for k, v in TRUNCATION_STAGES.items()}
        named = [(names[t], v) for t, v in stages]
        members = list(range(logits.shape[0])) if rows is None else list(rows)
        if out is None:
            out = torch.zeros(logits.shape[0], dtype=torch.int32)
        dists = [truncated_probs(logits[r].tolist(), temperatures[i], named) for i, r in enumerate(members)]
        if maximum_surprise is not None:
            drawn = [mirostat_select(p, maximum_surprise[i], uniform(seeds[i], positions[i])) for i, p in enumerate(dists)]
            for r, (t, _) in zip(members, drawn):
                out[r] = t
            return out, torch.tensor([math.exp(-s_) for _, s_ in drawn], dtype=torch.float64)
        for i, (r, p) in enumerate(zip(members, dists)):
            out[r] = select(p, uniform(seeds[i], positions[i]))
        return (out, torch.tensor(np.stack(dists))) if want_probs else out

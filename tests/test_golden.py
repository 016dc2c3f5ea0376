"""The plain attention (and, on a GPU, the kernels) against outputs of the reference's own
float64 attention oracle, stored by tests/golden/make_attention_golden.py."""
import json
import math
import os
import types

import numpy as np
import pytest
import torch

from tests.plain import model as pm

HERE = os.path.dirname(os.path.abspath(__file__))


def _cases():
    with open(os.path.join(HERE, "golden", "attention_oracle.json")) as fh:
        raw = json.load(fh)
    for item in raw:
        c = item["case"]
        rows, n_q, n_kv, d, t = c["query_rows"], c["query_heads"], c["kv_heads"], c["head_dim"], c["tokens"]
        q = torch.tensor(item["queries"], dtype=torch.float64).view(rows, n_q, d)
        kv_rows = 1 if c["shared_prefix"] else rows
        k = torch.from_numpy(np.array(item["keys_f16_bits"], dtype=np.uint16).view(np.float16).astype(np.float64))
        v = torch.from_numpy(np.array(item["values_f16_bits"], dtype=np.uint16).view(np.float16).astype(np.float64))
        k = k.view(kv_rows, n_kv, t, d).permute(0, 2, 1, 3)      # [row, token, kv head, d]
        v = v.view(kv_rows, n_kv, t, d).permute(0, 2, 1, 3)
        want = torch.tensor(item["outputs"], dtype=torch.float64).view(rows, n_q, d)
        yield c, q, k, v, want


def test_plain_attention_matches_the_reference_oracle():
    for c, q, k, v, want in _cases():
        t = c["tokens"]
        for row in range(c["query_rows"]):
            kr = k[0 if c["shared_prefix"] else row]
            vr = v[0 if c["shared_prefix"] else row]
            # a decode step: the query sits at the last position and reads every key
            qq = torch.zeros(t, c["query_heads"], c["head_dim"], dtype=torch.float64)
            qq[t - 1] = q[row]
            got = pm.attention(qq, kr, vr, list(range(t)))[t - 1]
            assert torch.allclose(got, want[row], rtol=1e-12, atol=1e-13), c


@pytest.mark.gpu
def test_gpu_attention_kernels_match_the_reference_oracle():
    from leone_b200.ops.cuda import CudaOps
    dev = "cuda:0"
    for dtype, tol in ((torch.float32, dict(rtol=3e-4, atol=3e-5)), (torch.bfloat16, dict(rtol=2e-2, atol=4e-3))):
        ops = CudaOps(dev, dtype)
        for c, q, k, v, want in _cases():
            t, n_q, n_kv, d, rows = c["tokens"], c["query_heads"], c["kv_heads"], c["head_dim"], c["query_rows"]
            pt = 4
            blocks = -(-t // pt)
            k_pool = torch.zeros((rows * blocks + 2, n_kv, pt, d), device=dev, dtype=dtype)
            v_pool = torch.zeros_like(k_pool)
            table = torch.zeros((rows, blocks), dtype=torch.int32)
            perm = torch.randperm(rows * blocks + 2, generator=torch.Generator().manual_seed(1))
            for r in range(rows):
                kr = k[0 if c["shared_prefix"] else r]
                vr = v[0 if c["shared_prefix"] else r]
                for b in range(blocks):
                    page = int(perm[r * blocks + b])
                    table[r, b] = page
                    n = min(pt, t - b * pt)
                    k_pool[page, :, :n] = kr[b * pt:b * pt + n].permute(1, 0, 2).to(dtype)
                    v_pool[page, :, :n] = vr[b * pt:b * pt + n].permute(1, 0, 2).to(dtype)
            qkv = torch.zeros((rows, (n_q + 2 * n_kv) * d), device=dev, dtype=dtype)
            qkv[:, :n_q * d] = q.reshape(rows, -1).to(dtype)
            out = torch.empty((rows, n_q * d), device=dev, dtype=dtype)
            ctx = types.SimpleNamespace(
                positions=torch.full((rows,), t - 1, device=dev, dtype=torch.int32),
                seq_of_token=torch.arange(rows, device=dev, dtype=torch.int32),
                q_start=torch.arange(rows + 1, device=dev, dtype=torch.int32),
                ctx_len=torch.full((rows,), t, device=dev, dtype=torch.int32),
                status=torch.zeros(4, device=dev, dtype=torch.int32), n_seqs=rows, max_q_len=1,
                max_ctx_len=t, decode_only=True)
            cache = types.SimpleNamespace(k_pool=k_pool, v_pool=v_pool, block_table=table.to(dev), page_tokens=pt)
            ops.attention(ctx, qkv, out, n_q, n_kv, d, 1 / math.sqrt(d), None, cache)
            assert ctx.status[0].item() == 0
            if dtype == torch.bfloat16:
                # the oracle's inputs are not bf16 values: compare with the plain result on rounded inputs
                qr = q.float().to(dtype).double()
                ref = []
                for r in range(rows):
                    kr = k[0 if c["shared_prefix"] else r].float().to(dtype).double()
                    vr = v[0 if c["shared_prefix"] else r].float().to(dtype).double()
                    qq = torch.zeros(t, n_q, d, dtype=torch.float64)
                    qq[t - 1] = qr[r]
                    ref.append(pm.attention(qq, kr, vr, list(range(t)))[t - 1])
                target = torch.stack(ref)
            else:
                target = want
            assert torch.allclose(out.double().cpu().view(rows, n_q, d), target, **tol), (c, dtype)

"""Cases that the reference's own unit tests state with literal numbers, replayed through the
plain implementation (and, on the GPU, through the engine's kernels).  The reference's model
code is Rust and cannot be compiled or imported here; its tests are read as text.  These few
cases pin, against numbers the reference wrote down: that the norm weight multiplies directly
(not ``1 + w``), that argmax takes the flat index of the largest value, that attention is causal
by position with scores scaled by 1/sqrt(head_dim), and that one KV head serves its group.

For the rotary pairing, the q/k norm before the rotation and SwiGLU the reference's tests hold
no literal outputs but a second statement of each formula, written apart from the product
code and compared with it there: ``rope_oracle`` (crates/leone-cuda/tests/gpu.rs:4563-4581: pair
``i`` is elements ``(i, i + half)``, angle ``position * theta^(-2 i / head_dim)``, ``first * cos -
second * sin`` and ``first * sin + second * cos``), ``rms_rope_oracle`` (norm with the weight,
then that rotation: crates/leone-cuda/tests/gpu.rs:1604) and ``swiglu_expected``
(crates/leone-cuda/tests/gpu.rs:1851-1857).  ``tests/plain/model.py`` agrees with both statements."""
import math

import pytest
import torch

from tests.plain import model as pm


def test_rms_norm_and_argmax_case():
    """crates/leone/src/cpu.rs:2781-2806: rows [1, 2] and [3, 4], weight [1, 0.5], eps 1e-6; the
    largest normalised value is element 2.  (With ``1 + w`` as the factor it would be element 1.)"""
    x = torch.tensor([[1.0, 2.0], [3.0, 4.0]], dtype=torch.float64)
    y = pm.rms_norm(x, torch.tensor([1.0, 0.5], dtype=torch.float64), 1e-6)
    assert pm.argmax(y.flatten().tolist()) == 2
    wrong = x * (1 + torch.tensor([1.0, 0.5])) / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6)
    assert int(wrong.flatten().argmax()) == 1


def _causal_case():
    # crates/leone/src/cpu.rs:2850-2898: 2 query heads on 1 KV head, head_dim 2, two tokens
    k = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]], dtype=torch.float64)
    v = torch.tensor([[[2.0, 4.0]], [[6.0, 8.0]]], dtype=torch.float64)
    q = torch.tensor([[[1.0, 0.0], [0.0, 1.0]], [[1.0, 0.0], [0.0, 1.0]]], dtype=torch.float64)
    high = math.exp(1.0 / math.sqrt(2.0))
    den = high + 1.0
    expected = torch.tensor([[2.0, 4.0, 2.0, 4.0],
                             [(high * 2 + 6) / den, (high * 4 + 8) / den, (2 + high * 6) / den, (4 + high * 8) / den]],
                            dtype=torch.float64)
    return q, k, v, expected


def test_prefill_attention_is_causal_within_the_position_block_case():
    q, k, v, expected = _causal_case()
    out = pm.attention(q, k, v, [0, 1]).reshape(2, 4)
    assert (out - expected).abs().max().item() < 1e-12


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32])
def test_the_same_case_through_the_paged_attention_kernel(dtype):
    """The same numbers through the engine's own attention over a paged cache (head size 2 is
    below what the tiled kernels take: this is the any-size kernel of the 32-bit path)."""
    from leone_b200.engine.batch import StepContext
    from leone_b200.ops.cuda import CudaOps
    from leone_b200.parts.base import PagedCacheView
    q, k, v, expected = _causal_case()
    dev = "cuda:0"
    ops = CudaOps(dev, dtype)
    qkv = torch.cat([q.reshape(2, 4), k.reshape(2, 2), v.reshape(2, 2)], dim=1).to(dtype).to(dev).contiguous()
    k_pool = torch.zeros((3, 1, 4, 2), dtype=dtype, device=dev)
    v_pool = torch.zeros_like(k_pool)
    ctx = StepContext()
    ctx.n_tokens, ctx.n_seqs = 2, 1
    ctx.positions = torch.tensor([0, 1], dtype=torch.int32, device=dev)
    ctx.seq_of_token = torch.zeros(2, dtype=torch.int32, device=dev)
    ctx.q_start = torch.tensor([0, 2], dtype=torch.int32, device=dev)
    ctx.ctx_len = torch.tensor([2], dtype=torch.int32, device=dev)
    ctx.status = torch.zeros(4, dtype=torch.int32, device=dev)
    ctx.max_q_len, ctx.max_ctx_len, ctx.decode_only = 2, 2, False
    cache = PagedCacheView(k_pool, v_pool, torch.tensor([[2]], dtype=torch.int32, device=dev), 4)
    ops.qk_norm_rope_write(ctx, qkv, 2, 1, 2, None, None, 1e-6, None, 0, cache)
    out = torch.empty((2, 4), dtype=dtype, device=dev)
    ops.attention(ctx, qkv, out, 2, 1, 2, 1.0 / math.sqrt(2.0), None, cache)
    assert int(ctx.status[0]) == 0
    assert (out.double().cpu() - expected).abs().max().item() < 1e-6

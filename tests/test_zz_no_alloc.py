"""The allocation-free decode attention entry point (csrc/leone_static.h).

It exists for programs that embed the library but may not allocate device memory once they
are running: hosts that fixed their memory budget at start-up and gave the rest to a pool of
their own, and latency-bound loops that cannot afford an allocator call between launches.
The split-KV scratch therefore sits in a static device array inside the library.

The test calls the exported C symbol directly, twice in a row with different inputs (the
second call finds the first call's leftovers in the shared scratch), and checks each output
against the ordinary entry point, which takes its scratch from the caller.  It also checks
that a call too large for the static array is refused with a message and launches nothing.
This file sorts last so that a run stopping at the first failure has run everything else.
"""
import ctypes
import math
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _case(seed, seq_lens, n_q, n_kv, d, pt):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    blocks = [-(-l // pt) for l in seq_lens]
    pages = sum(blocks) + 2
    k_pool = torch.randn((pages, n_kv, pt, d), device=DEV, generator=g).to(torch.bfloat16)
    v_pool = torch.randn((pages, n_kv, pt, d), device=DEV, generator=g).to(torch.bfloat16)
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((len(seq_lens), max(blocks)), -1, dtype=torch.int32)
    for s, nb in enumerate(blocks):
        for b in range(nb):
            table[s, b] = perm.pop()
    n = len(seq_lens)
    qkv = torch.randn((n, (n_q + 2 * n_kv) * d), device=DEV, generator=g).to(torch.bfloat16)
    return dict(qkv=qkv, k_pool=k_pool, v_pool=v_pool, table=table.to(DEV),
                q_start=torch.arange(n + 1, device=DEV, dtype=torch.int32),
                ctx_len=torch.tensor(seq_lens, device=DEV, dtype=torch.int32), n=n)


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from leone_b200.csrc.build import ensure_built
    ordinary = ctypes.CDLL(ensure_built("bf16"))
    static = ctypes.CDLL(ensure_built("static"))
    ordinary.leone_attention_decode_scratch.restype = ctypes.c_longlong
    n_q, n_kv, d, pt, splits = 8, 2, 64, 16, 5
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    err = ctypes.create_string_buffer(256)
    for seed, seq_lens in ((1, [700, 33, 1, 260]), (2, [90, 1500, 64, 65])):
        c = _case(seed, seq_lens, n_q, n_kv, d, pt)
        args = (_ptr(c["k_pool"]), _ptr(c["v_pool"]), _ptr(c["table"]), c["table"].shape[1],
                _ptr(c["q_start"]), _ptr(c["ctx_len"]), c["n"], n_q, n_kv, d, c_float(1 / math.sqrt(d)),
                0, pt, c["k_pool"].shape[0], splits)
        want = torch.full((c["n"], n_q * d), 3.0, device=DEV, dtype=torch.bfloat16)
        need = ordinary.leone_attention_decode_scratch(c["n"], n_q, d, splits)
        scratch = torch.empty(need, dtype=torch.float32, device=DEV)
        rc = ordinary.leone_attention_decode(_ptr(c["qkv"]), c["qkv"].stride(0), _ptr(want), want.stride(0),
                                             *args, _ptr(scratch), _ptr(status), stream)
        assert rc == 0
        got = torch.full_like(want, -3.0)
        rc = static.leone_attention_decode_static(_ptr(c["qkv"]), c["qkv"].stride(0), _ptr(got), got.stride(0),
                                                  *args, _ptr(status), err, 256, stream)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        assert status[0].item() == 0
        assert torch.isfinite(got.float()).all()
        # the same kernels in the same order: the tests' bf16 attention tolerance, and in fact equal
        assert torch.allclose(got.float(), want.float(), rtol=2 ** -6, atol=4e-3)
        assert torch.equal(got, want)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from leone_b200.csrc.build import ensure_built
    static = ctypes.CDLL(ensure_built("static"))
    err = ctypes.create_string_buffer(256)
    out = torch.full((4, 8), 5.0, device=DEV, dtype=torch.bfloat16)
    # 4096 sequences x 64 heads x 64 splits x 130 floats is far beyond the 4 MiB array
    rc = static.leone_attention_decode_static(c_void_p(0), 0, _ptr(out), 0, c_void_p(0), c_void_p(0),
                                              c_void_p(0), 1, c_void_p(0), c_void_p(0), 4096, 64, 8, 128,
                                              c_float(1.0), 0, 16, 1, 64, c_void_p(0), err, 256, c_void_p(0))
    assert rc == -4
    assert b"static array holds" in err.value
    torch.cuda.synchronize()
    assert bool((out == 5.0).all())

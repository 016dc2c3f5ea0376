"""Each CUDA kernel alone against a plain torch reference, at sizes other than the engine's."""
import math
import types

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops32():
    from leone_b200.ops.cuda import CudaOps
    return CudaOps(DEV, torch.float32)


@pytest.fixture(scope="module")
def ops16():
    from leone_b200.ops.cuda import CudaOps
    ops = CudaOps(DEV, torch.bfloat16)
    status = torch.zeros(4, device=DEV, dtype=torch.int32)
    ops.bind_status(status)                 # a wait that runs out inside a kernel shows here
    yield ops
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0], f"a kernel reported {ops.describe_status(int(status[0]))}: {status.tolist()}"


def _gen(seed):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    return g


def _randn(shape, seed, dtype=torch.float32, scale=1.0):
    return (torch.randn(shape, generator=_gen(seed), device=DEV) * scale).to(dtype)


def _close(got, want, rtol, atol, what=""):
    got, want = got.double(), want.double()
    err = (got - want).abs()
    bound = atol + rtol * want.abs()
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.numel()} outside tolerance; worst "
                           f"err {err.max().item():.3e} at {int(err.argmax())}, "
                           f"|want| there {want.flatten()[err.argmax()].abs().item():.3e}")


# -- embedding -----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab,hidden,n", [(331, 80, 7), (1000, 1536, 33)])
def test_embedding(ops32, dtype, vocab, hidden, n):
    table = _randn((vocab, hidden), 1, dtype)
    ids = torch.randint(0, vocab, (n,), generator=_gen(2), device=DEV, dtype=torch.int32)
    out = torch.empty((n, hidden), device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops32.embedding(table, ids, out, status)
    assert torch.equal(out, table[ids.long()].float())
    assert status[0].item() == 0


def test_embedding_bad_id_sets_status(ops32):
    table = _randn((50, 32), 1)
    ids = torch.tensor([3, 50, 7], device=DEV, dtype=torch.int32)
    out = torch.full((3, 32), 9.0, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops32.embedding(table, ids, out, status)
    assert status.tolist()[:3] == [1, 1, 50]
    assert torch.equal(out[1], torch.zeros(32, device=DEV))
    assert torch.equal(out[0], table[3])


# -- rms norm ------------------------------------------------------------------------------
@pytest.mark.parametrize("hidden,eps", [(80, 3e-6), (96, 1e-5), (4096, 1e-6), (5120, 1e-6), (1000, 1e-5)])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("odtype", [torch.float32, torch.bfloat16])
def test_rms_norm(ops32, hidden, eps, wdtype, odtype):
    x = _randn((13, hidden), 3, scale=2.5)
    w = (1 + 0.1 * _randn((hidden,), 4)).to(wdtype)
    out = torch.empty((13, hidden), device=DEV, dtype=odtype)
    ops32.rms_norm(x, w, out, eps)
    xd = x.double()
    want = xd * w.double() / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps)
    if odtype == torch.float32:
        _close(out, want, 2e-5, 3e-6, "rms_norm")
    else:
        _close(out, want, 2 ** -8, 1e-6, "rms_norm bf16")


def test_rms_norm_gathers_rows(ops32):
    x = _randn((20, 96), 5)
    w = _randn((96,), 6)
    rows = torch.tensor([19, 0, 7, 7], device=DEV, dtype=torch.int32)
    out = torch.empty((4, 96), device=DEV)
    ops32.rms_norm(x, w, out, 1e-5, rows)
    xd = x[rows.long()].double()
    want = xd * w.double() / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-5)
    _close(out, want, 2e-5, 3e-6, "rms_norm rows")


# -- CUDA-core matrix product ----------------------------------------------------------------
@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (3, 100, 33), (65, 129, 64), (130, 64, 200), (17, 331, 80)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt(ops32, m, n, k, dtype):
    x = _randn((m, k), 7, dtype)
    w = _randn((n, k), 8, dtype, scale=0.1)
    want = x.double() @ w.double().t()
    out = torch.empty((m, n), device=DEV, dtype=dtype)
    ops32._gemm_simt(x, w, out, 0, None)
    if dtype == torch.float32:
        _close(out, want, 1e-5, 1e-5 * math.sqrt(k), "simt f32")
    else:
        _close(out, want, 2 ** -8, 1e-4, "simt bf16")
    res = _randn((m, n), 9)
    out32 = res.clone()
    ops32._gemm_simt(x, w, out32, 2, out32)
    _close(out32, want + res.double(), 1e-5, 1e-5 * math.sqrt(k), "simt residual in place")
    if dtype == torch.bfloat16:
        out32 = torch.empty((m, n), device=DEV)
        ops32._gemm_simt(x, w, out32, 1, None)
        _close(out32, want, 1e-5, 1e-5 * math.sqrt(k), "simt fp32 out")


def test_gemm_simt_true_fp32(ops32):
    """Values that a reduced-precision matrix mode would round away must survive."""
    k = 64
    x = torch.ones((4, k), device=DEV)
    x[:, 0] = 1.0 + 2.0 ** -20
    w = torch.ones((8, k), device=DEV)
    out = torch.empty((4, 8), device=DEV)
    ops32._gemm_simt(x, w, out, 0, None)
    assert torch.equal(out, torch.full((4, 8), k + 2.0 ** -20, device=DEV))


# -- tensor-core matrix product ----------------------------------------------------------------
TC_SHAPES = [(1, 128, 64), (5, 100, 72), (16, 256, 128), (17, 384, 200), (64, 1000, 4096),
             (100, 128, 640), (200, 520, 512), (300, 264, 1024), (2048, 512, 256), (8, 4096, 12288)]


@pytest.mark.parametrize("m,n,k", TC_SHAPES)
@pytest.mark.parametrize("splits", [1, 3])
def test_gemm_tc(ops16, m, n, k, splits):
    fast = ops16.fast
    x = _randn((m, k), 11, torch.bfloat16)
    w = _randn((n, k), 12, torch.bfloat16, scale=0.05)
    want = x.double() @ w.double().t()
    atol32 = 2e-6 * math.sqrt(k) * 4
    out = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    fast._gemm(x, w, out, 0, None, n, splits=splits)
    _close(out, want, 2 ** -8, atol32, f"tc bf16 out m{m} n{n} k{k} s{splits}")
    out32 = torch.empty((m, n), device=DEV)
    fast._gemm(x, w, out32, 1, None, n, splits=splits)
    _close(out32, want, 1e-5, atol32, "tc fp32 out")
    res = _randn((m, n), 13)
    hidden = res.clone()
    fast._gemm(x, w, hidden, 2, hidden, n, splits=splits)
    _close(hidden, want + res.double(), 1e-5, atol32, "tc residual in place")
    torch.cuda.synchronize()
    if fast._counters is not None:
        assert int(fast._counters.abs().sum()) == 0, "split-K counters were not reset"


@pytest.mark.parametrize("m,inter,k", [(1, 64, 64), (7, 176, 80), (33, 224, 96), (260, 1024, 512)])
def test_gemm_tc_swiglu(ops16, m, inter, k):
    gate = _randn((inter, k), 14, torch.bfloat16, scale=0.2)
    up = _randn((inter, k), 15, torch.bfloat16, scale=0.2)
    x = _randn((m, k), 16, torch.bfloat16)
    w = ops16.prepare_gate_up(gate, up)
    assert w.gate_up_layout == "interleaved16"
    out = torch.empty((m, inter), device=DEV, dtype=torch.bfloat16)
    ops16.linear_swiglu(x, w, out)
    g = x.double() @ gate.double().t()
    u = x.double() @ up.double().t()
    _close(out, g / (1 + torch.exp(-g)) * u, 2 ** -7, 1e-4, "tc swiglu")


@pytest.mark.parametrize("m,n,k", [(1, 264, 64), (65, 520, 200), (100, 1000, 4096), (129, 256, 1024),
                                   (200, 24576 // 8, 512), (256, 300, 72)])
def test_gemm_tc_token_major_below_the_prompt_sizes(ops16, m, n, k):
    """The token-major form (128 tokens x 256 weight rows per tile) forced for 256 tokens or
    fewer: every epilogue against float64, and the refusal of a folded norm."""
    fast = ops16.fast
    x = _randn((m, k), 51, torch.bfloat16)
    w = _randn((n, k), 52, torch.bfloat16, scale=0.05)
    want = x.double() @ w.double().t()
    atol32 = 2e-6 * math.sqrt(k) * 4
    out = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    fast._gemm(x, w, out, 0, None, n, token_major=True)
    _close(out, want, 2 ** -8, atol32, f"token-major bf16 out m{m} n{n} k{k}")
    out32 = torch.empty((m, n), device=DEV)
    fast._gemm(x, w, out32, 1, None, n, token_major=True)
    _close(out32, want, 1e-5, atol32, "token-major fp32 out")
    res = _randn((m, n), 53)
    hidden = res.clone()
    fast._gemm(x, w, hidden, 2, hidden, n, token_major=True)
    _close(hidden, want + res.double(), 1e-5, atol32, "token-major residual in place")
    inter = (n // 32) * 16
    gate, up = w[:inter].contiguous(), w[inter:2 * inter].contiguous()
    gu = ops16.prepare_gate_up(gate, up)
    act = torch.empty((m, inter), device=DEV, dtype=torch.bfloat16)
    fast._gemm(x, gu.weight, act, 3, None, 2 * inter, token_major=True)
    g = x.double() @ gate.double().t()
    u = x.double() @ up.double().t()
    _close(act, g / (1 + torch.exp(-g)) * u, 2 ** -7, 1e-4, "token-major swiglu")
    xn = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    ss = torch.empty((fast.norm_parts(m, n, pairs=False), m), device=DEV)
    with pytest.raises(RuntimeError, match="refused"):
        fast._gemm(x, w, hidden, 2, hidden, n, token_major=True, norm_out=(xn, torch.ones(n, device=DEV), ss))


@pytest.mark.parametrize("m,n,k,splits", [(100, 520, 2048, 3), (300, 264, 1024, 2), (129, 256, 4096, 8),
                                          (512, 1000, 640, 5), (65, 4096, 512, 4), (1, 300, 1032, 2),
                                          (600, 768, 12288, 7)])
def test_gemm_tc_token_major_cluster_split(ops16, m, n, k, splits):
    """The token-major form with the splits of a tile as a thread-block cluster: every epilogue
    against float64, the same bits on every run, and the refusal of a folded norm."""
    fast = ops16.fast
    assert fast._token_major_capacity(splits) > 0
    x = _randn((m, k), 61, torch.bfloat16)
    w = _randn((n, k), 62, torch.bfloat16, scale=0.05)
    want = x.double() @ w.double().t()
    atol32 = 2e-6 * math.sqrt(k) * 4
    kw = dict(splits=splits, cluster=True, token_major=True)
    out = torch.full((m, n), 9.0, device=DEV, dtype=torch.bfloat16)
    fast._gemm(x, w, out, 0, None, n, **kw)
    _close(out, want, 2 ** -8, atol32, f"token-major cluster bf16 out m{m} n{n} k{k} s{splits}")
    out32 = torch.full((m, n), 9.0, device=DEV)
    fast._gemm(x, w, out32, 1, None, n, **kw)
    _close(out32, want, 1e-5, atol32, "token-major cluster fp32 out")
    res = _randn((m, n), 63)
    hidden = res.clone()
    fast._gemm(x, w, hidden, 2, hidden, n, **kw)
    _close(hidden, want + res.double(), 1e-5, atol32, "token-major cluster residual in place")
    again = res.clone()
    fast._gemm(x, w, again, 2, again, n, **kw)
    assert torch.equal(hidden, again)
    inter = (n // 32) * 16
    gate, up = w[:inter].contiguous(), w[inter:2 * inter].contiguous()
    gu = ops16.prepare_gate_up(gate, up)
    act = torch.full((m, inter), 9.0, device=DEV, dtype=torch.bfloat16)
    fast._gemm(x, gu.weight, act, 3, None, 2 * inter, **kw)
    g = x.double() @ gate.double().t()
    u = x.double() @ up.double().t()
    _close(act, g / (1 + torch.exp(-g)) * u, 2 ** -7, 1e-4, "token-major cluster swiglu")
    xn = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    ss = torch.empty((fast.norm_parts(m, n, pairs=False), m), device=DEV)
    with pytest.raises(RuntimeError, match="refused"):
        fast._gemm(x, w, hidden, 2, hidden, n, norm_out=(xn, torch.ones(n, device=DEV), ss), **kw)
    torch.cuda.synchronize()


def test_the_dispatcher_splits_narrow_products_in_the_token_major_form(ops16, monkeypatch):
    """(In single blocks: the splits on pairs of SMs, which take some of these, are switched off.)"""
    fast = ops16.fast
    monkeypatch.setattr(fast, "use_pair_splits", False)
    sms = fast.sm_count
    assert fast.plan_product(8, 4096, 4096)[0] is False                     # decode-sized: swapped
    tm, s, full, cluster = fast.plan_product(300, 4096, 4096)                # 3 x 16 tiles
    assert tm and cluster and full == 0 and 2 <= s <= 8 and 48 * s <= sms
    assert fast.plan_product(2048, 4096, 4096) == (True, 1, 0, False)        # fills the SMs unsplit
    assert not fast.fuses_norm(300, 4096, 4096) and fast.fuses_norm(2048, 4096, 4096)
    assert fast.plan_product(300, 4096, 256)[:2] == (True, 1)                # too few k-blocks to split


def test_gemm_tc_prompt_sized_tiles_of_240_weight_rows(ops16, monkeypatch):
    """The single-block kernel above 256 tokens: the tile's width is 256 or 240, whichever costs
    fewer rounds: a size where 240 wins, with the folded norm on both sides (its parts follow the
    width) and a ragged edge."""
    fast = ops16.fast
    monkeypatch.setattr(fast, "use_pairs", False)
    sms = fast.sm_count
    m, k = 128 * 8, 256
    n = 240 * (2 * sms // 8)                                # 2 rounds of 240-wide tiles; 256-wide ones need 3
    assert fast.lib.leone_gemm_tc_token_major_width(m, n, 0) == 240
    assert fast.lib.leone_gemm_tc_token_major_width(m, n, 1) == 256
    assert fast.norm_parts(m, n) == n // 240
    n -= 40                                                 # the last tile is ragged
    x = _randn((m, k), 71, torch.bfloat16)
    w = _randn((n, k), 72, torch.bfloat16, scale=0.05)
    want = x.double() @ w.double().t()
    res = _randn((m, n), 73)
    g = 1 + 0.2 * _randn((n,), 74)
    hidden = res.clone()
    parts = fast.norm_parts(m, n)
    xn = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    ss = torch.full((parts, m), -1.0, device=DEV)
    fast._gemm(x, w, hidden, 2, hidden, n, norm_out=(xn, g, ss))
    h64 = want + res.double()
    _close(hidden, h64, 1e-5, 2e-6 * math.sqrt(k) * 4, "240-wide tiles, residual")
    _close(ss.sum(0), (hidden.double() ** 2).sum(1), 1e-5, 1e-6, "240-wide tiles, sums of squares")
    _close(xn, hidden.double() * g.double(), 2 ** -8, 1e-6, "240-wide tiles, bf16(out * weight)")
    out = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    fast._gemm(x, w, out, 0, None, n)
    _close(out, want, 2 ** -8, 2e-6 * math.sqrt(k) * 4, "240-wide tiles, bf16 out")
    w2 = _randn((264, n), 75, torch.bfloat16, scale=0.05)
    rs = torch.rsqrt((hidden.double() ** 2).mean(dim=1, keepdim=True) + 1e-5)
    out2 = torch.empty((m, 264), device=DEV, dtype=torch.bfloat16)
    fast._gemm(xn, w2, out2, 0, None, 264, norm_in=(ss, parts, 1e-5))
    _close(out2, (xn.double() @ w2.double().t()) * rs, 2 ** -8, 1e-3, "the product after, parts of 240")


@pytest.mark.parametrize("m,n,k,width", [(129, 264, 64, 0), (200, 4096, 1024, 0), (257, 264, 64, 48), (300, 520, 512, 0),
                                         (513, 1000, 200, 112), (768, 4096, 1024, 0), (1000, 1024, 264, 176),
                                         (256, 1200, 4096, 32), (2048, 240 * 5 - 24, 4096, 0), (384, 777 * 16, 136, 208)])
def test_gemm_pair_on_two_sms(ops16, m, n, k, width):
    """Products on pairs of SMs (one MMA of 256 tokens over both blocks' shared memory), at the
    dispatcher's tile width (0) and at forced ones from 32 to 256: ragged last pairs (a second
    block with no token at all), ragged weight tiles, K that is no multiple of the k-block; every
    epilogue and the folded norm on both sides against float64, the same bits on every run and
    the same as the single-block kernel's."""
    fast = ops16.fast
    if not fast.use_pairs:
        pytest.skip("LEONE_NO_PAIRS is set")
    try:
        fast.pair_width_override = width
        fast.pair_padding = 0.0                               # pairs also where their last tile is half empty
        fast.token_major_split_from = 1 << 30                 # ... and where the dispatcher would split along K
        assert fast.in_pairs(m, n, k)
        x = _randn((m, k), 81, torch.bfloat16)
        w = _randn((n, k), 82, torch.bfloat16, scale=0.05)
        want = x.double() @ w.double().t()
        atol32 = 2e-6 * math.sqrt(k) * 4
        out = torch.full((m, n), 9.0, device=DEV, dtype=torch.bfloat16)
        fast._gemm(x, w, out, 0, None, n)
        _close(out, want, 2 ** -8, atol32, f"pair bf16 out m{m} n{n} k{k}")
        out32 = torch.full((m, n), 9.0, device=DEV)
        fast._gemm(x, w, out32, 1, None, n)
        _close(out32, want, 1e-5, atol32, "pair fp32 out")
        res = _randn((m, n), 83)
        g = 1 + 0.2 * _randn((n,), 84)
        hidden = res.clone()
        parts = fast.norm_parts(m, n)
        assert parts == -(-n // (width or fast.pair_width(m, n, False)))
        xn = torch.full((m, n), 7.0, device=DEV, dtype=torch.bfloat16)
        ss = torch.full((parts, m), -1.0, device=DEV)
        fast._gemm(x, w, hidden, 2, hidden, n, norm_out=(xn, g, ss))
        _close(hidden, want + res.double(), 1e-5, atol32, "pair residual in place")
        h64 = hidden.double()
        _close(xn, h64 * g.double(), 2 ** -8, 1e-6, "pair bf16(out * weight)")
        _close(ss.sum(0), (h64 * h64).sum(1), 1e-5, 1e-6, "pair sums of squares")
        again, xn2, ss2 = res.clone(), torch.empty_like(xn), torch.empty_like(ss)
        fast._gemm(x, w, again, 2, again, n, norm_out=(xn2, g, ss2))
        assert torch.equal(hidden, again) and torch.equal(xn, xn2) and torch.equal(ss, ss2)
        plain = res.clone()                                   # the residual epilogue without the norm
        fast._gemm(x, w, plain, 2, plain, n)
        assert torch.equal(plain, hidden)
        n2, inter = 328, 160
        w2 = _randn((n2, n), 85, torch.bfloat16, scale=0.05)
        rs = torch.rsqrt((h64 * h64).mean(dim=1, keepdim=True) + 1e-5)
        out2 = torch.empty((m, n2), device=DEV, dtype=torch.bfloat16)
        fast._gemm(xn, w2, out2, 0, None, n2, norm_in=(ss, parts, 1e-5))
        _close(out2, (xn.double() @ w2.double().t()) * rs, 2 ** -8, 1e-3, "pair, the product after the norm")
        gate, up = w2[:inter].contiguous(), w2[inter:2 * inter].contiguous()
        gu = ops16.prepare_gate_up(gate, up)
        act = torch.full((m, inter), 9.0, device=DEV, dtype=torch.bfloat16)
        fast.pair_width_override = max(32, width // 32 * 32) if width else 0      # whole groups of gate and up rows
        fast._gemm(xn, gu.weight, act, 3, None, 2 * inter, norm_in=(ss, parts, 1e-5))
        gg = (xn.double() @ gate.double().t()) * rs
        uu = (xn.double() @ up.double().t()) * rs
        _close(act, gg / (1 + torch.exp(-gg)) * uu, 2 ** -7, 1e-3, "pair swiglu after the norm")
        # the single-block kernel on the same inputs: the same sums in the same order
        fast.use_pairs = False
        single = torch.empty_like(out32)
        fast._gemm(x, w, single, 1, None, n, token_major=True)
        assert torch.equal(single, out32)
        torch.cuda.synchronize()
        assert int(fast.status.abs().sum()) == 0
    finally:
        fast.pair_width_override, fast.use_pairs, fast.pair_padding, fast.token_major_split_from = 0, True, 0.8, 128


@pytest.mark.parametrize("m,n,k,splits", [(129, 264, 1024, 2), (200, 520, 2048, 4), (256, 2048, 4096, 4),
                                          (300, 1000, 4096, 2), (512, 1000, 2048, 4), (600, 768, 640, 2)])
def test_gemm_pair_split_along_k(ops16, m, n, k, splits):
    """Two or four pairs of SMs share the k-blocks of a tile (clusters of four or eight blocks, the
    partial sums through the workspace): every epilogue against float64, the same bits on every
    run, and the refusals."""
    fast = ops16.fast
    if not fast.use_pairs:
        pytest.skip("LEONE_NO_PAIRS is set")
    assert fast._pair_capacity(splits) > 0
    try:
        fast.pair_padding, fast.pair_split_override = 0.0, splits
        x = _randn((m, k), 91, torch.bfloat16)
        w = _randn((n, k), 92, torch.bfloat16, scale=0.05)
        want = x.double() @ w.double().t()
        atol32 = 2e-6 * math.sqrt(k) * 4
        out = torch.full((m, n), 9.0, device=DEV, dtype=torch.bfloat16)
        fast._gemm(x, w, out, 0, None, n)
        _close(out, want, 2 ** -8, atol32, f"pair split bf16 out m{m} n{n} k{k} s{splits}")
        out32 = torch.full((m, n), 9.0, device=DEV)
        fast._gemm(x, w, out32, 1, None, n)
        _close(out32, want, 1e-5, atol32, "pair split fp32 out")
        res = _randn((m, n), 93)
        hidden = res.clone()
        fast._gemm(x, w, hidden, 2, hidden, n)
        _close(hidden, want + res.double(), 1e-5, atol32, "pair split residual in place")
        again = res.clone()
        fast._gemm(x, w, again, 2, again, n)
        assert torch.equal(hidden, again)
        inter = (n // 32) * 16
        gate, up = w[:inter].contiguous(), w[inter:2 * inter].contiguous()
        gu = ops16.prepare_gate_up(gate, up)
        act = torch.full((m, inter), 9.0, device=DEV, dtype=torch.bfloat16)
        fast._gemm(x, gu.weight, act, 3, None, 2 * inter)
        g = x.double() @ gate.double().t()
        u = x.double() @ up.double().t()
        _close(act, g / (1 + torch.exp(-g)) * u, 2 ** -7, 1e-4, "pair split swiglu")
        torch.cuda.synchronize()
        assert int(fast.status.abs().sum()) == 0
        # fewer than four k-blocks a pair, or a width that is not 128 or 256
        short = _randn((m, 64 * 3 * splits), 94, torch.bfloat16)
        with pytest.raises(RuntimeError, match="refused"):
            fast._gemm(short, w[:, :short.shape[1]].contiguous(), out, 0, None, n)
    finally:
        fast.pair_padding, fast.pair_split_override = 0.8, 0


def test_gemm_pair_refusals(ops16):
    fast = ops16.fast
    if not fast.use_pairs:
        pytest.skip("LEONE_NO_PAIRS is set")
    x = _randn((400, 64), 86, torch.bfloat16)
    w = _randn((512, 64), 87, torch.bfloat16)
    out = torch.empty((400, 512), device=DEV, dtype=torch.bfloat16)
    try:
        for width in (16, 40, 272):                           # not a multiple of 16 between 32 and 256
            fast.pair_width_override = width
            with pytest.raises(RuntimeError, match="refused"):
                fast._gemm(x, w, out, 0, None, 512)
        fast.pair_width_override = 48                         # SwiGLU needs whole groups of 32 rows
        act = torch.empty((400, 256), device=DEV, dtype=torch.bfloat16)
        with pytest.raises(RuntimeError, match="refused"):
            fast._gemm(x, w, act, 3, None, 512)
    finally:
        fast.pair_width_override = 0


def test_the_dispatcher_takes_pairs_for_unsplit_products_at_widths_that_fill_their_rounds(ops16):
    fast = ops16.fast
    if not fast.use_pairs:
        pytest.skip("LEONE_NO_PAIRS is set")
    assert fast.pair_padding == 0.8 and fast.token_major_split_from == 128
    assert [m for m in (128, 129, 256, 257, 384, 385, 512, 513, 640, 641, 2048, 8193) if fast.in_pairs(m)] == \
        [129, 256, 385, 512, 513, 640, 641, 2048, 8193]
    if fast.sm_count == 148:
        assert fast.pair_width(256, 24576, True) == 192         # 128 tiles: two rounds of narrower tiles
        assert fast.pair_width(2048, 4096, False) == 240        # 144 tiles: two rounds
        assert fast.pair_width(2048, 24576, True) == 256 and fast.pair_width(2048, 151936, False) == 256
        # the narrow products of a layer stay split along K up to about 600 tokens
        assert not fast.in_pairs(256, 4096, 4096) and not fast.in_pairs(256, 4096, 12288)
        assert fast.in_pairs(256, 24576, 4096) and fast.in_pairs(200, 151936, 4096) and fast.in_pairs(1024, 4096, 4096)
        assert fast.plan_product(300, 6144, 4096)[1] > 1 and fast.plan_product(2048, 4096, 4096) == (True, 1, 0, False)
        # ... unless pairs can split as many ways: two pairs a tile, clusters of four blocks
        assert fast.pair_split(256, 6144, 4096) == 2 and fast.in_pairs(256, 6144, 4096)
        assert fast.pair_split(512, 4096, 12288) == 2 and fast.pair_split(256, 4096, 12288) == 1
        assert fast.pair_split(2048, 4096, 4096) == 1 and fast.pair_split(300, 4096, 4096) == 2
    for m, n, swiglu in ((300, 1000, False), (129, 24576, True), (5000, 151936, False)):
        w = fast.pair_width(m, n, swiglu)
        assert 32 <= w <= 256 and w % (32 if swiglu else 16) == 0


def test_the_dispatcher_picks_the_token_major_form_only_where_its_tiles_fill_the_device(ops16):
    fast = ops16.fast
    sms = fast.sm_count
    assert fast.token_major(257, 64) and fast.token_major(2048, 4096)
    assert not fast.token_major(64, 256 * sms)                       # decode-sized: always swapped
    assert fast.token_major(128, 256 * sms) and fast.token_major(200, 128 * sms)
    assert not fast.token_major(128, 256 * (sms // 2))               # too few tiles: swapped, split along K
    assert not fast.token_major(128, 256 * 3 * sms)                  # many tiles (an output head): swapped


@pytest.mark.parametrize("m,n,k,splits,full", [(8, 128 * 7, 1024, 3, 4), (40, 128 * 5 + 17, 2048, 4, 2),
                                               (1, 128 * 3, 4096, 8, 1), (64, 1000, 512, 2, 7)])
def test_gemm_tc_splits_only_the_last_tiles(ops16, m, n, k, splits, full):
    fast = ops16.fast
    x = _randn((m, k), 21, torch.bfloat16)
    w = _randn((n, k), 22, torch.bfloat16, scale=0.05)
    want = x.double() @ w.double().t()
    res = _randn((m, n), 23)
    hidden = res.clone()
    fast._gemm(x, w, hidden, 2, hidden, n, splits=splits, full_tiles=full)
    _close(hidden, want + res.double(), 1e-5, 2e-6 * math.sqrt(k) * 4, "tail split")
    out = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    fast._gemm(x, w, out, 0, None, n)                    # the heuristic's own choice
    _close(out, want, 2 ** -8, 2e-6 * math.sqrt(k) * 4, "heuristic split")
    torch.cuda.synchronize()
    assert int(fast._counters.abs().sum()) == 0


@pytest.mark.parametrize("m,n,k,splits", [(1, 384, 4096, 8), (5, 1000, 1024, 3), (16, 128 * 9, 520, 2),
                                          (40, 520, 2048, 5), (64, 4096, 1024, 4), (100, 300, 640, 7),
                                          (200, 1000, 2048, 6), (8, 4096, 4096, 8)])
def test_gemm_tc_cluster_split(ops16, m, n, k, splits):
    """The splits of a tile as a thread-block cluster: same sums, in the same order, as through
    the workspace, for every epilogue."""
    fast = ops16.fast
    assert fast.cluster_capacity(m, splits) > 0
    x = _randn((m, k), 31, torch.bfloat16)
    w = _randn((n, k), 32, torch.bfloat16, scale=0.05)
    want = x.double() @ w.double().t()
    atol32 = 2e-6 * math.sqrt(k) * 4
    out = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    fast._gemm(x, w, out, 0, None, n, splits=splits, cluster=True)
    _close(out, want, 2 ** -8, atol32, f"cluster bf16 out m{m} n{n} k{k} s{splits}")
    via_workspace = torch.empty_like(out)
    fast._gemm(x, w, via_workspace, 0, None, n, splits=splits)
    assert torch.equal(out, via_workspace)
    res = _randn((m, n), 33)
    hidden = res.clone()
    fast._gemm(x, w, hidden, 2, hidden, n, splits=splits, cluster=True)
    _close(hidden, want + res.double(), 1e-5, atol32, "cluster residual in place")
    again = res.clone()
    fast._gemm(x, w, again, 2, again, n, splits=splits, cluster=True)
    assert torch.equal(hidden, again)
    # SwiGLU epilogue on interleaved gate/up rows
    inter = (n // 32) * 16
    if inter:
        gate, up = w[:inter].contiguous(), w[inter:2 * inter].contiguous()
        gu = ops16.prepare_gate_up(gate, up)
        act = torch.empty((m, inter), device=DEV, dtype=torch.bfloat16)
        fast._gemm(x, gu.weight, act, 3, None, 2 * inter, splits=splits, cluster=True)
        g = x.double() @ gate.double().t()
        u = x.double() @ up.double().t()
        _close(act, g / (1 + torch.exp(-g)) * u, 2 ** -7, 1e-4, "cluster swiglu")


@pytest.mark.parametrize("m,n,k,splits,cluster", [(1, 384, 4096, 1, False), (8, 1000, 1032, 1, False),
                                                  (5, 640, 520, 3, True), (16, 4096, 4096, 4, True),
                                                  (17, 256, 2048, 2, True), (33, 1024, 1024, 5, True),
                                                  (64, 520, 4096, 3, False), (200, 384, 768, 6, True),
                                                  (300, 520, 512, 1, False), (1000, 1024, 264, 1, False)])
def test_gemm_tc_norm_between_products(ops16, m, n, k, splits, cluster):
    """An RMSNorm folded into the product before it (which leaves bf16(out * weight) and the sums
    of out^2) and the product after it (which scales its rows): against float64."""
    fast = ops16.fast
    x = _randn((m, k), 41, torch.bfloat16)
    w1 = _randn((n, k), 42, torch.bfloat16, scale=0.05)
    res = _randn((m, n), 43) * 2.0
    res[0, 5] = 40.0                                       # one large element dominates a row's scale
    g = 1 + 0.2 * _randn((n,), 44)
    eps = 1e-5
    hidden = res.clone()
    parts = fast.norm_parts(m, n, pairs=None if splits == 1 else False)    # a forced split: the single-block kernel
    xn = torch.full((m, n), 7.0, device=DEV, dtype=torch.bfloat16)
    ss = torch.full((parts, m), -1.0, device=DEV)
    fast._gemm(x, w1, hidden, 2, hidden, n, splits=splits, cluster=cluster, norm_out=(xn, g, ss))
    want_hidden = x.double() @ w1.double().t() + res.double()
    _close(hidden, want_hidden, 1e-5, 2e-6 * math.sqrt(k) * 4, "the product before the norm")
    h64 = hidden.double()
    _close(xn, h64 * g.double(), 2 ** -8, 1e-6, "bf16(out * weight)")
    _close(ss.sum(0), (h64 * h64).sum(1), 1e-5, 1e-6, "sums of squares")
    # the product after the norm
    n2 = 328
    w2 = _randn((n2, n), 45, torch.bfloat16, scale=0.05)
    rs = torch.rsqrt((h64 * h64).mean(dim=1, keepdim=True) + eps)
    want = (xn.double() @ w2.double().t()) * rs
    exact = (h64 * g.double() * rs) @ w2.double().t()
    out = torch.empty((m, n2), device=DEV, dtype=torch.bfloat16)
    for s2, cl in ((1, False), (2, m <= 256), (3, False)):      # a prompt-sized product with a norm is never split
        fast._gemm(xn, w2, out, 0, None, n2, splits=s2, cluster=cl, norm_in=(ss, parts, eps))
        _close(out, want, 2 ** -8, 1e-3, f"the product after the norm, splits {s2}")
        _close(out, exact, 2 ** -5, 5e-2, "against the exact norm")
    inter = 160
    gate, up = w2[:inter].contiguous(), w2[inter:2 * inter].contiguous()
    gu = ops16.prepare_gate_up(gate, up)
    act = torch.empty((m, inter), device=DEV, dtype=torch.bfloat16)
    fast._gemm(xn, gu.weight, act, 3, None, 2 * inter, norm_in=(ss, parts, eps))
    gg = (xn.double() @ gate.double().t()) * rs
    uu = (xn.double() @ up.double().t()) * rs
    _close(act, gg / (1 + torch.exp(-gg)) * uu, 2 ** -7, 1e-3, "swiglu after the norm")
    torch.cuda.synchronize()
    assert int(fast.status.abs().sum()) == 0


def test_linear_with_norm_through_the_ops_table(ops16):
    from leone_b200.parts.base import DeferredNorm, Runtime
    m, k, n = 8, 512, 640
    rt = Runtime(DEV, torch.bfloat16, ops16, 16)
    x = _randn((m, k), 50, torch.bfloat16)
    hidden = _randn((m, n), 51)
    g = 1 + 0.1 * _randn((n,), 52)
    w1 = ops16.prepare_matrix(_randn((n, k), 53, torch.bfloat16, scale=0.05))
    w2 = ops16.prepare_matrix(_randn((384, n), 54, torch.bfloat16, scale=0.05))
    assert ops16.linear_fuses_norm(m, w1) and ops16.linear_fuses_norm(m, w2)
    assert not ops16.linear_fuses_norm(100, w1)           # between 33 and 256 tokens the norm kernel stays
    assert ops16.linear_fuses_norm(300, w1)
    d = DeferredNorm(None, None, hidden, g, 1e-6, "t")
    d.prepare(rt, ops16.norm_parts(m, n))
    ops16.linear(x, w1, hidden, residual=hidden, norm_out=d)
    out = torch.empty((m, 384), device=DEV, dtype=torch.bfloat16)
    ops16.linear(d.xn, w2, out, norm_in=d)
    normed = torch.empty((m, n), device=DEV, dtype=torch.bfloat16)
    ops16.rms_norm(hidden, g, normed, 1e-6)
    two = torch.empty_like(out)
    ops16.linear(normed, w2, two)
    _close(out, two.double(), 2 ** -6, 2e-2, "folded norm against the norm kernel")


def test_gemm_tc_cluster_refusals(ops16):
    fast = ops16.fast
    x = _randn((8, 512), 1, torch.bfloat16)
    w = _randn((256, 512), 2, torch.bfloat16)
    out = torch.empty((8, 256), device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="refused"):
        fast._gemm(x, w, out, 0, None, 256, splits=2, full_tiles=1, cluster=True)   # tail-only split
    big = _randn((4096 * 4, 512), 3, torch.bfloat16)
    out_big = torch.empty((8, 4096 * 4), device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="refused"):
        fast._gemm(x, big, out_big, 0, None, 4096 * 4, splits=8, cluster=True)      # more than one round


def test_gemm_tc_refuses_unaligned_k(ops16):
    x = _randn((4, 60), 1, torch.bfloat16)
    w = ops16.prepare_matrix(_randn((32, 60), 2, torch.bfloat16))
    out = torch.empty((4, 32), device=DEV, dtype=torch.bfloat16)
    ops16.linear(x, w, out)          # falls to the any-size kernel
    _close(out, x.double() @ w.weight.double().t(), 2 ** -8, 1e-4, "k=60")


# -- q/k norm + rotary + cache write, and attention ------------------------------------------
def _paged_setup(seq_lens, page_tokens, n_kv, d, dtype, seed, extra_pages=3):
    """Random block tables over a shuffled pool."""
    blocks = [-(-l // page_tokens) for l in seq_lens]
    num_pages = sum(blocks) + extra_pages
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max(blocks) + 1
    table = torch.full((len(seq_lens), width), -1, dtype=torch.int32)
    for s, nb in enumerate(blocks):
        for b in range(nb):
            table[s, b] = perm.pop()
    k_pool = torch.zeros((num_pages, n_kv, page_tokens, d), device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    return table.to(DEV), k_pool, v_pool


def _ctx(positions, seq_of_token):
    c = types.SimpleNamespace()
    c.positions = torch.tensor(positions, device=DEV, dtype=torch.int32)
    c.seq_of_token = torch.tensor(seq_of_token, device=DEV, dtype=torch.int32)
    c.status = torch.zeros(4, dtype=torch.int32, device=DEV)
    return c


def _rope_table(max_pos, rd, theta):
    from leone_b200.parts.rotary import build_rotary_table
    return build_rotary_table(max_pos, rd, theta).to(DEV)


def _ref_norm_rope(x, w, eps, positions, theta, rd, adjacent=False):
    """x [n, heads, d] float64.  Pair i: elements (i, i + rd/2), or (2i, 2i + 1) if adjacent."""
    if w is not None:
        x = x * w.double() / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    half = rd // 2
    inv = torch.tensor([theta ** (-2.0 * i / rd) for i in range(half)], dtype=torch.float64, device=x.device)
    ang = torch.tensor(positions, dtype=torch.float64, device=x.device)[:, None] * inv[None]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if adjacent:
        a, b = x[..., 0:rd:2], x[..., 1:rd:2]
        out[..., 0:rd:2] = a * cos - b * sin
        out[..., 1:rd:2] = a * sin + b * cos
        return out
    a, b = x[..., :half], x[..., half:rd]
    out[..., :half] = a * cos - b * sin
    out[..., half:rd] = a * sin + b * cos
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,pt,theta,eps", [(5, 1, 48, 16, 5e4, 3e-6), (6, 3, 32, 8, 1e6, 1e-5),
                                                     (8, 2, 128, 16, 1e6, 1e-6), (3, 3, 80, 4, 1e4, 1e-6),
                                                     (4, 2, 64, 16, 1e4, 1e-6), (2, 1, 256, 8, 1e6, 1e-5)])
@pytest.mark.parametrize("pairing", ["half_split", "adjacent"])
def test_qk_norm_rope_write(ops32, dtype, n_q, n_kv, d, pt, theta, eps, pairing):
    seq_lens = [11, 3, 25]
    starts = [4, 0, 20]                      # tokens of this step: positions start..len-1
    positions, seqs = [], []
    for s, (l, st) in enumerate(zip(seq_lens, starts)):
        positions += list(range(st, l))
        seqs += [s] * (l - st)
    n = len(positions)
    table, k_pool, v_pool = _paged_setup(seq_lens, pt, n_kv, d, dtype, 5)
    qkv = _randn((n, (n_q + 2 * n_kv) * d), 21, dtype)
    qw = (1 + 0.1 * _randn((d,), 22))
    kw = (1 + 0.1 * _randn((d,), 23))
    rope = _rope_table(64, d, theta)
    orig = qkv.clone()
    cache = types.SimpleNamespace(k_pool=k_pool, v_pool=v_pool, block_table=table, page_tokens=pt)
    ctx = _ctx(positions, seqs)
    ops32.qk_norm_rope_write(ctx, qkv, n_q, n_kv, d, qw, kw, eps, rope, d, cache, pairing=pairing)
    assert ctx.status[0].item() == 0
    x = orig.double().view(n, n_q + 2 * n_kv, d)
    q_ref = _ref_norm_rope(x[:, :n_q], qw, eps, positions, theta, d, pairing == "adjacent")
    k_ref = _ref_norm_rope(x[:, n_q:n_q + n_kv], kw, eps, positions, theta, d, pairing == "adjacent")
    got = qkv.view(n, n_q + 2 * n_kv, d)
    rt, at = (5e-6, 5e-6) if dtype == torch.float32 else (2 ** -7, 1e-5)
    _close(got[:, :n_q], q_ref, rt * 4, at, "q")
    _close(got[:, n_q:n_q + n_kv], k_ref, rt * 4, at, "k")
    assert torch.equal(got[:, n_q + n_kv:], orig.view(n, -1, d)[:, n_q + n_kv:])
    for i, (p, s) in enumerate(zip(positions, seqs)):
        page = int(table[s, p // pt])
        assert torch.equal(k_pool[page, :, p % pt, :], got[i, n_q:n_q + n_kv])
        assert torch.equal(v_pool[page, :, p % pt, :], got[i, n_q + n_kv:])


def test_qk_write_missing_page_sets_status(ops32):
    table = torch.full((1, 2), -1, dtype=torch.int32, device=DEV)
    k_pool = torch.zeros((2, 1, 4, 16), device=DEV)
    cache = types.SimpleNamespace(k_pool=k_pool, v_pool=k_pool.clone(), block_table=table, page_tokens=4)
    ctx = _ctx([0], [0])
    qkv = _randn((1, 3 * 16), 1)
    ops32.qk_norm_rope_write(ctx, qkv, 1, 1, 16, None, None, 1e-6, None, 0, cache)
    assert ctx.status[0].item() == 2
    assert float(k_pool.abs().sum()) == 0.0


def _ref_attention(q, keys, vals, n_q, n_kv, scale, lo):
    """q [n_q, d]; keys/vals [ctx, n_kv, d] float64 → [n_q, d]."""
    g = n_q // n_kv
    out = torch.zeros_like(q)
    for h in range(n_q):
        s = (keys[lo:, h // g] @ q[h]) * scale
        w = torch.softmax(s, 0)
        out[h] = (w[:, None] * vals[lo:, h // g]).sum(0)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,pt,window", [(5, 1, 48, 16, None), (6, 3, 32, 8, None),
                                                  (8, 2, 128, 16, None), (4, 4, 80, 4, 7), (2, 1, 256, 16, 130)])
def test_attention_generic(ops32, dtype, n_q, n_kv, d, pt, window):
    seq_lens = [300, 3, 131]
    starts = [290, 0, 100]
    positions, seqs = [], []
    for s, (l, st) in enumerate(zip(seq_lens, starts)):
        positions += list(range(st, l))
        seqs += [s] * (l - st)
    n = len(positions)
    table, k_pool, v_pool = _paged_setup(seq_lens, pt, n_kv, d, dtype, 9)
    keys = [_randn((l, n_kv, d), 30 + s, dtype) for s, l in enumerate(seq_lens)]
    vals = [_randn((l, n_kv, d), 40 + s, dtype) for s, l in enumerate(seq_lens)]
    for s, l in enumerate(seq_lens):
        for p in range(l):
            page = int(table[s, p // pt])
            k_pool[page, :, p % pt] = keys[s][p]
            v_pool[page, :, p % pt] = vals[s][p]
    if window:
        for s, st in enumerate(starts):
            table[s, :max(0, st - window + 1) // pt] = -1      # pages the window has passed are gone
    qkv = _randn((n, (n_q + 2 * n_kv) * d), 50, dtype)
    # make one far key dominate for one row: a single wrong page would show
    qkv.view(n, -1, d)[0, 0] = (keys[0][5, 0].float() * 4).to(dtype)
    out = torch.empty((n, n_q * d), device=DEV, dtype=dtype)
    cache = types.SimpleNamespace(k_pool=k_pool, v_pool=v_pool, block_table=table, page_tokens=pt)
    ctx = _ctx(positions, seqs)
    scale = 1 / math.sqrt(d)
    ops32.attention(ctx, qkv, out, n_q, n_kv, d, scale, window, cache)
    assert ctx.status[0].item() == 0
    for i, (p, s) in enumerate(zip(positions, seqs)):
        lo = 0 if not window else max(0, p - window + 1)
        want = _ref_attention(qkv[i].double().view(-1, d)[:n_q], keys[s][:p + 1].double(),
                              vals[s][:p + 1].double(), n_q, n_kv, scale, lo)
        rt, at = (3e-4, 3e-5) if dtype == torch.float32 else (2 ** -7, 2e-3)
        _close(out[i].view(n_q, d), want, rt, at, f"attention row {i}")


# -- sampling ------------------------------------------------------------------------------------
def test_sample_greedy_ties_and_nonfinite(ops32):
    logits = torch.zeros((3, 1000), device=DEV)
    logits[0, 17] = 5.0
    logits[0, 900] = 5.0                 # tie → lowest id
    logits[1, :] = float("-inf")
    logits[1, 333] = -7.0
    logits[2, 0] = float("nan")
    logits[2, 999] = 1.0
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    z = torch.zeros(3, device=DEV)
    zi = torch.zeros(3, dtype=torch.int64, device=DEV)
    ops32.sample(logits, z, zi, zi, out)
    assert out.tolist() == [17, 333, 999]


@pytest.mark.parametrize("vocab", [331, 151936])
def test_sample_temperature_matches_host(ops32, vocab):
    from tests.plain.model import temperature_probs, uniform
    import numpy as np
    rows = 6
    logits = _randn((rows, vocab), 60, scale=3.0)
    logits[0, 5] = float("-inf")
    temps = torch.tensor([0.8, 1.0, 0.3, 2.0, 0.0, 0.7], device=DEV)
    seeds = torch.tensor([0, 1, 2, 3, 4, 12345678901], dtype=torch.int64, device=DEV)
    pos = torch.tensor([0, 5, 17, 100, 3, 2047], dtype=torch.int64, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops32.sample(logits, temps, seeds, pos, out)
    host = logits.cpu().numpy()
    for r in range(rows):
        t = float(temps[r])
        if t == 0.0:
            assert out[r].item() == int(np.argmax(host[r]))
            continue
        probs = temperature_probs(host[r], t)
        cdf = np.cumsum(probs)
        u = uniform(int(seeds[r]), int(pos[r]))
        got = out[r].item()
        lo = cdf[got - 1] if got > 0 else 0.0
        # the drawn value lies in the chosen token's interval, up to summation rounding
        assert lo - 1e-9 <= u < cdf[got] + 1e-9 and probs[got] > 0


# -- tiled bf16 attention: prompt portions / mixed batches, and split-KV decode ------------------
def _tiled_case(ops16, n_q, n_kv, d, pt, window, seq_lens, starts, seed, leading_decode_rows=None):
    positions, seqs, q_start = [], [], [0]
    for s, (l, st) in enumerate(zip(seq_lens, starts)):
        positions += list(range(st, l))
        seqs += [s] * (l - st)
        q_start.append(len(positions))
    n = len(positions)
    dtype = torch.bfloat16
    table, k_pool, v_pool = _paged_setup(seq_lens, pt, n_kv, d, dtype, seed)
    keys = [_randn((l, n_kv, d), seed * 100 + s, dtype) for s, l in enumerate(seq_lens)]
    vals = [_randn((l, n_kv, d), seed * 100 + 50 + s, dtype) for s, l in enumerate(seq_lens)]
    for s, l in enumerate(seq_lens):
        pos = torch.arange(l)
        pages = table[s, (pos // pt).to(DEV)].long()
        k_pool[pages, :, (pos % pt).to(DEV)] = keys[s]
        v_pool[pages, :, (pos % pt).to(DEV)] = vals[s]
    if window:
        # pages that the window has passed are given back before the step: the kernel must not read them
        for s, st in enumerate(starts):
            passed = max(0, st - window + 1) // pt
            table[s, :passed] = -1
    qkv = _randn((n, (n_q + 2 * n_kv) * d), seed + 7, dtype)
    # one far key dominates for the first row of every sequence: a wrong page or a lost
    # tile changes the output by far more than the tolerance
    for s in range(len(seq_lens)):
        row = q_start[s]
        far = min(3, positions[row])
        qkv.view(n, -1, d)[row, 0] = (keys[s][far, 0].float() * 3).to(dtype)
    out = torch.full((n, n_q * d), 7.0, device=DEV, dtype=dtype)
    cache = types.SimpleNamespace(k_pool=k_pool, v_pool=v_pool, block_table=table, page_tokens=pt)
    ctx = _ctx(positions, seqs)
    ctx.q_start = torch.tensor(q_start, device=DEV, dtype=torch.int32)
    ctx.ctx_len = torch.tensor(seq_lens, device=DEV, dtype=torch.int32)
    ctx.n_seqs = len(seq_lens)
    ctx.max_q_len = max(l - st for l, st in zip(seq_lens, starts))
    ctx.max_ctx_len = max(seq_lens)
    ctx.decode_only = ctx.max_q_len == 1
    ctx.fixed_shapes = False
    ctx.q_lens = np.array([l - st for l, st in zip(seq_lens, starts)])
    ctx.ctx_lens = np.array(seq_lens)
    if leading_decode_rows is not None:
        assert ops16.fast.leading_decode_rows(ctx) == leading_decode_rows
    scale = 1 / math.sqrt(d)
    assert ops16.fast.attention(ctx, qkv, out, n_q, n_kv, d, scale, window, cache)
    assert ctx.status[0].item() == 0
    for i, (p, s) in enumerate(zip(positions, seqs)):
        lo = 0 if not window else max(0, p - window + 1)
        want = _ref_attention(qkv[i].double().view(-1, d)[:n_q], keys[s][:p + 1].double(),
                              vals[s][:p + 1].double(), n_q, n_kv, scale, lo)
        _close(out[i].view(n_q, d), want, 2 ** -6, 4e-3, f"tiled attention row {i} (seq {s}, pos {p})")


@pytest.mark.parametrize("n_q,n_kv,d,pt,window", [(5, 1, 48, 16, None), (6, 3, 32, 8, None),
                                                  (8, 2, 128, 16, None), (4, 4, 80, 4, 37),
                                                  (32, 8, 128, 16, None), (16, 1, 64, 64, 100), (40, 2, 16, 16, None)])
def test_attention_prefill_tiled(ops16, n_q, n_kv, d, pt, window):
    # whole prompts, a continued portion, a 1-token row and a 2-token portion in one batch
    _tiled_case(ops16, n_q, n_kv, d, pt, window, seq_lens=[150, 3, 131, 70, 64], starts=[0, 0, 100, 69, 62],
                seed=3)


@pytest.mark.parametrize("n_q,n_kv,d,pt,window", [(8, 2, 128, 16, None), (6, 3, 32, 8, None), (10, 2, 64, 16, 90),
                                                  (32, 8, 128, 16, None)])
def test_attention_mixed_step_divided_between_the_decode_and_the_prompt_kernel(ops16, n_q, n_kv, d, pt, window):
    """A mixed step whose first sequences bring one token each: those rows run on the decode
    kernel and the rest on the prompt kernel, each over its own slice of the step's tables; and
    the same batch through the prompt kernel alone."""
    kw = dict(seq_lens=[300, 65, 1000, 150, 131, 40], starts=[299, 64, 999, 0, 100, 39], seed=9)
    _tiled_case(ops16, n_q, n_kv, d, pt, window, leading_decode_rows=3, **kw)
    ops16.fast.divide_mixed_steps = False
    try:
        _tiled_case(ops16, n_q, n_kv, d, pt, window, leading_decode_rows=0, **kw)
    finally:
        ops16.fast.divide_mixed_steps = True


@pytest.mark.parametrize("n_q,n_kv,d,pt,window", [(10, 2, 64, 16, None), (28, 4, 128, 8, 200), (3, 1, 128, 32, None),
                                                  (8, 2, 128, 16, 129), (64, 1, 64, 16, None)])
def test_attention_prefill_tensor_memory_kernel_long(ops16, n_q, n_kv, d, pt, window):
    """The tcgen05 prompt kernel over many key tiles: a long first portion, a continued portion
    that starts in the middle of a tile, head groups that do not divide the 128 rows of a block,
    windows that end inside a tile; and the mma.sync kernel on the same batch."""
    assert ops16.fast.use_tc_attention
    kw = dict(seq_lens=[700, 517, 130], starts=[0, 300, 127], seed=8)
    _tiled_case(ops16, n_q, n_kv, d, pt, window, **kw)        # tcgen05: two query tiles per block, P in tensor memory
    ops16.fast.use_tc_attention = False
    try:
        _tiled_case(ops16, n_q, n_kv, d, pt, window, **kw)    # mma.sync
    finally:
        ops16.fast.use_tc_attention = True


@pytest.mark.parametrize("n_q,n_kv,d,pt,window", [(32, 8, 128, 16, None), (6, 2, 64, 8, 70), (5, 1, 128, 16, None)])
def test_attention_prefill_pingpong_short_and_uneven_portions(ops16, n_q, n_kv, d, pt, window):
    """The kernel with two query tiles per block on portions that fill less than one query tile,
    exactly one, one and a bit (the second tile nearly empty), and on a portion whose two query
    tiles read different numbers of key tiles."""
    assert ops16.fast.use_tc_attention
    g = n_q // n_kv
    tq = 128 // g
    _tiled_case(ops16, n_q, n_kv, d, pt, window, seq_lens=[2, tq, tq + 1, 2 * tq, 3 * tq + 5, 128 + tq + 3],
                starts=[0, 0, 0, 0, 0, 128 - tq + 1], seed=11)
    _tiled_case(ops16, n_q, n_kv, d, pt, window, seq_lens=[1500], starts=[0], seed=12)


@pytest.mark.parametrize("n_q,n_kv,d,pt,window", [(5, 1, 48, 16, None), (6, 3, 32, 8, None),
                                                  (8, 2, 128, 16, None), (4, 4, 80, 4, 37),
                                                  (32, 8, 128, 16, None), (40, 2, 16, 16, None)])
@pytest.mark.parametrize("seq_lens", [[1], [300, 2, 64, 65, 1000], [2100]])
@pytest.mark.parametrize("clusters", [True, False])
def test_attention_decode_tiled(ops16, n_q, n_kv, d, pt, window, seq_lens, clusters, monkeypatch):
    """Split-KV decode, the splits merged inside a thread-block cluster or through scratch and a
    merge kernel."""
    monkeypatch.setattr(ops16.fast, "use_clusters", clusters)
    _tiled_case(ops16, n_q, n_kv, d, pt, window, seq_lens=seq_lens, starts=[l - 1 for l in seq_lens], seed=4)


@pytest.mark.parametrize("seq_lens", [[9000, 130], [33000], [17000, 16999, 5, 4097]])
def test_attention_decode_long_contexts(ops16, seq_lens):
    """Contexts of tens of thousands of tokens (more splits than a cluster holds, the merge
    kernel, block tables thousands of entries wide), at the 8B head shape; a far key dominates
    the first head of every sequence, so a lost split shows."""
    _tiled_case(ops16, 32, 8, 128, 16, None, seq_lens=seq_lens, starts=[l - 1 for l in seq_lens], seed=21)
    _tiled_case(ops16, 6, 2, 64, 16, 4500, seq_lens=seq_lens, starts=[l - 1 for l in seq_lens], seed=22)


@pytest.mark.parametrize("n_q,n_kv,d,pt,window,qk_norm,rotary", [
    (8, 2, 128, 16, None, True, True), (6, 3, 64, 8, None, True, True), (5, 1, 64, 16, 40, False, True),
    (40, 2, 128, 16, None, True, False), (4, 4, 128, 4, 300, True, True)])
@pytest.mark.parametrize("seq_lens,pairing", [([300, 1, 64, 65, 17], "half_split"), ([2100], "half_split"),
                                              ([1, 2], "half_split"), ([300, 1, 64, 65, 17], "adjacent"),
                                              ([2100], "adjacent")])
def test_attention_decode_fused_norm_rope_write(ops16, n_q, n_kv, d, pt, window, qk_norm, rotary, seq_lens, pairing):
    """The decode kernel doing q/k norm, rotation and cache write itself against the two-kernel
    path on the same raw projections: the same cache bit for bit, the same outputs."""
    dtype = torch.bfloat16
    n = len(seq_lens)
    table, k_pool, v_pool = _paged_setup(seq_lens, pt, n_kv, d, dtype, 6)
    k_pool.copy_(_randn(tuple(k_pool.shape), 300, dtype))      # what older tokens (and freed pages) left
    v_pool.copy_(_randn(tuple(v_pool.shape), 400, dtype))
    raw = _randn((n, (n_q + 2 * n_kv) * d), 77, dtype)
    qw = (1 + 0.1 * _randn((d,), 78)) if qk_norm else None
    kw = (1 + 0.1 * _randn((d,), 79)) if qk_norm else None
    rope = _rope_table(4096, d, 1e4) if rotary else None
    ctx = _ctx([l - 1 for l in seq_lens], list(range(n)))
    ctx.q_start = torch.arange(n + 1, device=DEV, dtype=torch.int32)
    ctx.ctx_len = torch.tensor(seq_lens, device=DEV, dtype=torch.int32)
    ctx.n_seqs, ctx.max_q_len, ctx.max_ctx_len, ctx.decode_only = n, 1, max(seq_lens), True
    scale = 1 / math.sqrt(d)
    # two kernels
    qkv_a, k_a, v_a = raw.clone(), k_pool.clone(), v_pool.clone()
    cache_a = types.SimpleNamespace(k_pool=k_a, v_pool=v_a, block_table=table, page_tokens=pt)
    ops16.qk_norm_rope_write(ctx, qkv_a, n_q, n_kv, d, qw, kw, 1e-6, rope, d if rotary else 0, cache_a,
                             pairing=pairing)
    out_a = torch.empty((n, n_q * d), device=DEV, dtype=dtype)
    ops16.attention(ctx, qkv_a, out_a, n_q, n_kv, d, scale, window, cache_a)
    # one kernel
    qkv_b, k_b, v_b = raw.clone(), k_pool.clone(), v_pool.clone()
    cache_b = types.SimpleNamespace(k_pool=k_b, v_pool=v_b, block_table=table, page_tokens=pt)
    out_b = torch.full_like(out_a, 7.0)
    assert ops16.can_fuse_decode(ctx, qkv_b, n_q, n_kv, d)
    ops16.attention(ctx, qkv_b, out_b, n_q, n_kv, d, scale, window, cache_b,
                    fuse=dict(q_w=qw, k_w=kw, eps=1e-6, rope=rope, write_cache=True, pairing=pairing))
    torch.cuda.synchronize()
    assert ctx.status[0].item() == 0
    assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b), "the cache differs"
    assert torch.equal(out_a, out_b), "the outputs differ"
    # without the cache write the pools stay as they were and the outputs are the same
    k_c, v_c = k_pool.clone(), v_pool.clone()
    cache_c = types.SimpleNamespace(k_pool=k_c, v_pool=v_c, block_table=table, page_tokens=pt)
    out_c = torch.empty_like(out_a)
    ops16.attention(ctx, raw.clone(), out_c, n_q, n_kv, d, scale, window, cache_c,
                    fuse=dict(q_w=qw, k_w=kw, eps=1e-6, rope=rope, write_cache=False, pairing=pairing))
    torch.cuda.synchronize()
    assert torch.equal(k_c, k_pool) and torch.equal(v_c, v_pool)
    assert torch.equal(out_c, out_a)


def test_attention_decode_cluster_refuses_what_it_cannot_do(ops16):
    from ctypes import c_float, c_void_p
    lib = ops16.fast.lib
    z = c_void_p(0)
    args = lambda d, splits, fuse: (z, 1024, z, 1024, z, z, z, 4, z, z, 2, 8, 2, d, c_float(1.0), 0, 16, 8,
                                    splits, fuse, z, z, c_float(1e-6), z, 0, 0, 0, z, z)
    assert lib.leone_attention_decode_cluster(*args(128, 9, 0)) != 0        # more splits than a cluster holds
    assert lib.leone_attention_decode_cluster(*args(96, 2, 1)) != 0         # fused preparation needs d 64 or 128


# -- the sampler's truncation stages (fp64 pipeline) ---------------------------------------------
PIPELINES = [
    [("top_k", 40)], [("top_p", 0.9)], [("min_p", 0.05)], [("top_a", 0.2)], [("tfs", 0.95)], [("typical", 0.7)],
    [("epsilon", 3e-4)], [("eta", 2e-3)], [("min_k", 3.0)], [("top_n_sigma", 1.0)],
    [("top_k", 50), ("top_p", 0.9), ("min_p", 0.05)],
    [("top_n_sigma", 2.0), ("typical", 0.8), ("tfs", 0.9), ("top_k", 7)],
    [("min_k", 1.0), ("eta", 0.01), ("typical", 0.9), ("typical", 0.5), ("epsilon", 1e-3), ("top_a", 0.1)],
    [("top_p", 1.0), ("top_k", 1)], [("epsilon", 1.0), ("tfs", 1e-9)],
]


@pytest.mark.parametrize("vocab", [7, 331, 5000])
@pytest.mark.parametrize("stages", PIPELINES, ids=lambda s: "+".join(n for n, _ in s))
def test_sample_truncated_matches_the_plain_sampler(ops32, vocab, stages):
    """Every stage and several pipelines: the distribution against the plain float64 sampler
    entry by entry, and the drawn ids; rows with ties, excluded entries and different
    temperatures."""
    from leone_b200.sampling.sampler import TRUNCATION_STAGES
    from tests.plain.model import select, truncated_probs, uniform
    rows = 4
    logits = _randn((rows, vocab), 70 + vocab, scale=3.0)
    logits[0, 3] = float("-inf")
    logits[1, 1] = float("nan")
    logits[2] = torch.round(logits[2] * 2) / 2                 # many equal logits: ties go to the lower id
    logits[3, :vocab // 2] = float("-inf")
    temps = [0.7, 1.0, 1.3, 0.25]
    seeds = [1, 2, 12345678901, 4]
    positions = [0, 17, 300, 2047]
    numbered = [(TRUNCATION_STAGES[n], v) for n, v in stages]
    out, probs = ops32.sample_truncated(logits, temps, seeds, positions, numbered, want_probs=True)
    host = logits.cpu().numpy()
    for r in range(rows):
        want = truncated_probs(host[r], temps[r], stages)
        got = probs[r].cpu().numpy()
        assert (got > 0).tolist() == (want > 0).tolist(), f"row {r}: the surviving sets differ"
        assert np.abs(got - want).max() < 1e-13, f"row {r}: {np.abs(got - want).max()}"
        assert int(out[r]) == select(want, uniform(seeds[r], positions[r]))


def test_sample_truncated_on_some_rows_in_place(ops32):
    """A subset of a step's rows goes through the stages where it lies: the ids land at the rows'
    own places, the other places keep what they held, and a row of non-finite logits gets -1."""
    from leone_b200.sampling.sampler import TRUNCATION_STAGES
    from tests.plain.model import select, truncated_probs, uniform
    rows, vocab = 5, 777
    logits = _randn((rows, vocab), 5150, scale=3.0)
    logits[3] = float("nan")
    stages = [("top_k", 50), ("top_p", 0.9)]
    numbered = [(TRUNCATION_STAGES[n], v) for n, v in stages]
    out = torch.full((rows,), 1234, dtype=torch.int32, device=DEV)
    members, temps, seeds, positions = [4, 1, 3], [0.9, 1.2, 0.8], [5, 6, 7], [40, 41, 42]
    got, probs = ops32.sample_truncated(logits, temps, seeds, positions, numbered, want_probs=True, rows=members, out=out)
    assert got.data_ptr() == out.data_ptr() and probs.shape == (3, vocab)
    host = logits.cpu().numpy()
    want = out.tolist()
    assert want[0] == 1234 and want[2] == 1234 and want[3] == -1
    for i, r in enumerate(members[:2]):
        dist = truncated_probs(host[r], temps[i], stages)
        assert want[r] == select(dist, uniform(seeds[i], positions[i]))
        assert np.abs(probs[i].cpu().numpy() - dist).max() < 1e-13


def test_sample_truncated_full_vocabulary(ops32):
    """A row of 151,936 logits (the sort's global passes, the scans over long rows)."""
    from leone_b200.sampling.sampler import TRUNCATION_STAGES
    from tests.plain.model import select, truncated_probs, uniform
    vocab = 151936
    logits = _randn((2, vocab), 99, scale=2.5)
    logits[0, 5] = float("-inf")
    for stages in ([("top_p", 0.95), ("min_p", 0.01)], [("typical", 0.9), ("top_k", 100)], [("tfs", 0.97)]):
        numbered = [(TRUNCATION_STAGES[n], v) for n, v in stages]
        out, probs = ops32.sample_truncated(logits, [0.8, 1.1], [7, 8], [11, 12], numbered, want_probs=True)
        host = logits.cpu().numpy()
        for r in range(2):
            want = truncated_probs(host[r], [0.8, 1.1][r], stages)
            got = probs[r].cpu().numpy()
            assert (got > 0).tolist() == (want > 0).tolist()
            assert np.abs(got - want).max() < 1e-13
            assert int(out[r]) == select(want, uniform([7, 8][r], [11, 12][r]))


def test_sampler_routes_rows_with_stages_through_the_pipeline(ops32):
    from leone_b200.sampling.sampler import Sampler, SamplingParams
    from tests.plain.model import sample as plain_sample
    vocab = 500
    logits = _randn((5, vocab), 123, scale=3.0)
    params = [SamplingParams(), SamplingParams(0.9, 3), SamplingParams(0.9, 3, (("top_k", 5),)),
              SamplingParams(0.0, 1, (("top_k", 5),)), SamplingParams(1.2, 9, (("min_p", 0.1), ("top_p", 0.8)))]
    positions = [4, 5, 6, 7, 8]
    got = Sampler(ops32, DEV).sample(logits, params, positions).tolist()
    host = logits.cpu().numpy()
    want = [plain_sample(host[i].tolist(), p.temperature, p.seed, positions[i], p.truncations)
            for i, p in enumerate(params)]
    assert got == want
    with pytest.raises(ValueError, match="valid range"):
        SamplingParams(1.0, 0, (("top_p", 1.5),))
    with pytest.raises(ValueError, match="unknown"):
        SamplingParams(1.0, 0, (("top_q", 0.5),))


def test_penalize_matches_the_plain_penalties(ops32):
    """The penalty kernel on rows with different settings and histories (ids past the vocabulary,
    repeated suffixes, a row without penalties) against the plain implementation, bit for bit."""
    from leone_b200.sampling.sampler import Penalties, Sampler, SamplingParams
    from tests.plain.model import apply_penalties, sample as plain_sample
    vocab = 300
    rng = np.random.default_rng(11)
    settings = [dict(repetition=1.3, presence=0.2, frequency=0.05, window=20),
                dict(repetition=0.7, window=None, dry_multiplier=0.9, dry_allowed_length=1, dry_breakers=(7,)),
                dict(), dict(frequency=-0.3, window=64, dry_multiplier=0.5, dry_base=2.0, dry_window=16)]
    histories = []
    for i in range(len(settings)):
        h = rng.integers(0, 40, 50).tolist()
        h = h + h[10:18] + [vocab + 5] + h[10:14]              # a repeated stretch, an id past the vocabulary
        histories.append(h)
    logits = _randn((len(settings), vocab), 200, scale=3.0)
    host = logits.cpu().numpy().copy()
    params = [SamplingParams(0.0 if i % 2 else 0.8, i, (), Penalties(**kw)) for i, kw in enumerate(settings)]
    got = Sampler(ops32, DEV).sample(logits, params, [len(h) - 1 for h in histories], histories).tolist()
    for i, kw in enumerate(settings):
        want = apply_penalties(host[i], histories[i], **kw)
        assert logits[i].cpu().numpy().tolist() == want.tolist(), f"row {i}"
        if kw:
            assert want.tolist() != host[i].tolist()
        assert got[i] == plain_sample(want.tolist(), params[i].temperature, params[i].seed, len(histories[i]) - 1)
    with pytest.raises(ValueError, match="history"):
        Sampler(ops32, DEV).sample(logits, params, [0] * len(settings))


@pytest.mark.parametrize("vocab", [50, 5000])
def test_mirostat_filter_matches_the_plain_sampler(ops32, vocab):
    """Mirostat v2's surprise filter after the stages: the drawn ids and the drawn tokens'
    probabilities before the filter, with maxima that keep everything, a part, and nothing
    (the most probable token is then the only one left)."""
    import math
    from leone_b200.sampling.sampler import TRUNCATION_STAGES
    from tests.plain.model import mirostat_select, truncated_probs, uniform
    rows = 4
    logits = _randn((rows, vocab), 300 + vocab, scale=2.0)
    temps = [1.0, 0.8, 1.2, 1.0]
    seeds, positions = [3, 4, 5, 6], [9, 10, 11, 12]
    maxima = [50.0, 3.0, 1.0, 1e-9]
    for stages in ([], [("top_k", 30), ("min_p", 0.01)]):
        numbered = [(TRUNCATION_STAGES[n], v) for n, v in stages]
        out, chosen = ops32.sample_truncated(logits, temps, seeds, positions, numbered, maximum_surprise=maxima)
        host = logits.cpu().numpy()
        for r in range(rows):
            target = truncated_probs(host[r], temps[r], stages)
            token, observed = mirostat_select(target, maxima[r], uniform(seeds[r], positions[r]))
            assert int(out[r]) == token
            assert abs(-math.log(float(chosen[r])) - observed) < 1e-12
    assert int(out[3]) == int(torch.argmax(logits[3]))


@pytest.mark.parametrize("vocab", [5000, 151936])
def test_sample_truncated_small_top_k_first(ops32, vocab):
    """A pipeline that starts with a small top-k orders only the heads of the row's tiles: equal
    logits across tiles (ties go to the lower id), a row with fewer finite logits than k, the
    largest k the short way takes and the first it does not."""
    from leone_b200.sampling.sampler import TRUNCATION_STAGES
    from tests.plain.model import select, truncated_probs, uniform
    rows = 4
    logits = _randn((rows, vocab), 400 + vocab, scale=2.0)
    logits[1] = torch.round(logits[1])                         # thousands of equal logits
    logits[2, 7:] = float("-inf")                              # seven finite logits
    logits[3, ::3] = float("nan")
    temps, seeds, positions = [0.9, 1.0, 1.1, 0.7], [5, 6, 7, 8], [1, 2, 3, 4]
    tiles = (1 << (vocab - 1).bit_length()) // 2048
    edge = 8192 // tiles
    for stages in ([("top_k", 40), ("top_p", 0.9)], [("top_k", 1)], [("top_k", edge), ("min_p", 0.001)],
                   [("top_k", edge + 1), ("tfs", 0.99)], [("top_k", 12), ("typical", 0.8), ("top_k", 3)]):
        numbered = [(TRUNCATION_STAGES[n], v) for n, v in stages]
        out, probs = ops32.sample_truncated(logits, temps, seeds, positions, numbered, want_probs=True)
        host = logits.cpu().numpy()
        for r in range(rows):
            want = truncated_probs(host[r], temps[r], stages)
            got = probs[r].cpu().numpy()
            assert (got > 0).tolist() == (want > 0).tolist(), (stages, r)
            assert np.abs(got - want).max() < 1e-13
            assert int(out[r]) == select(want, uniform(seeds[r], positions[r]))

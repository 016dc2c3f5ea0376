"""The dispatchers' rules (which form a product takes, how the decode attention splits its keys)
on the CPU, against a stand-in for the library's size queries: what the rules promise for any size,
and the choices at the sizes they were measured at."""
import pytest

from leone_b200.ops.fast import FastKernels


class _Sizes:
    """Stand-in for the library's host-side size queries on a B200 (148 SMs)."""

    @staticmethod
    def leone_gemm_tc_tiles_token_major(m, n):
        return -(-m // 128) * -(-n // 256)

    @staticmethod
    def leone_gemm_tc_cluster_capacity_token_major(splits):
        # clusters of one block per SM that are resident at once: fewer than 148 / splits, since a
        # cluster lies inside one GPC (22 of six and 33 of four were what the occupancy query gave)
        return {2: 74, 3: 44, 4: 33, 5: 26, 6: 22, 7: 18, 8: 15}.get(splits, 0)

    @staticmethod
    def leone_gemm_pair_capacity(width, splits):
        return {2: 33, 4: 15}.get(splits, 0)


@pytest.fixture()
def fast():
    f = FastKernels.__new__(FastKernels)
    f.sm_count = 148
    f.lib = _Sizes()
    f._configure()
    for name in ("use_clusters", "use_token_major", "use_pairs", "use_pair_splits"):   # whatever the environment says
        setattr(f, name, True)
    return f


def test_pairs_take_unsplit_products_from_129_tokens(fast):
    assert [m for m in (1, 128, 129, 256, 257, 384, 385, 512, 513, 640, 641, 2048, 8193) if fast.in_pairs(m)] == \
        [129, 256, 385, 512, 513, 640, 641, 2048, 8193]
    # the narrow products of the 8B layer stay split along K in single blocks up to 256 tokens ...
    assert not fast.in_pairs(256, 4096, 4096) and not fast.in_pairs(256, 4096, 12288)
    # ... the wide ones and the prompt-sized ones run on pairs
    assert fast.in_pairs(256, 24576, 4096) and fast.in_pairs(200, 151936, 4096) and fast.in_pairs(2048, 4096, 4096)
    fast.use_pairs = False
    assert not fast.in_pairs(2048) and fast.pair_split(512, 4096, 12288) == 1


def test_pair_widths_fill_whole_rounds(fast):
    assert fast.pair_width(256, 24576, True) == 192            # 128 tiles: two rounds of narrower tiles
    assert fast.pair_width(2048, 4096, False) == 240           # 144 tiles: two rounds
    assert fast.pair_width(2048, 24576, True) == 256 and fast.pair_width(2048, 151936, False) == 256
    for m in (129, 300, 700, 5000):
        for n in (256, 1000, 4096, 6144, 24576, 151936):
            for swiglu in (False, True):
                w = fast.pair_width(m, n, swiglu)
                assert 32 <= w <= 256 and w % (32 if swiglu else 16) == 0
                rounds = -(-(-(-n // w) * -(-m // 256)) // 74)
                widest = -(-(-(-n // 256) * -(-m // 256)) // 74)
                assert rounds * w <= widest * 256               # never more work per pair than the widest tile's
    fast.pair_width_override = 64
    assert fast.pair_width(2048, 4096, False) == 64


def test_pair_splits_only_where_they_match_the_single_block_split(fast):
    assert fast.token_major_split(256, 6144, 4096) == 2 and fast.pair_split(256, 6144, 4096) == 2
    assert fast.token_major_split(512, 4096, 12288) == 2 and fast.pair_split(512, 4096, 12288) == 2
    assert fast.token_major_split(256, 4096, 12288) == 4 and fast.pair_split(256, 4096, 12288) == 1
    assert fast.pair_split(2048, 4096, 4096) == 1              # not split at all
    # 257 to 384 tokens: unsplit products stay in single blocks, split ones take pairs
    assert fast.pair_split(300, 4096, 4096) == 2 and fast.in_pairs(300, 4096, 4096) and not fast.in_pairs(300)
    assert not fast.in_pairs(300, 24576, 4096) and fast.pair_split(300, 24576, 4096) == 1
    assert fast.plan_product(512, 4096, 12288) == (True, 1, 0, False) and fast.in_pairs(512, 4096, 12288)
    fast.use_pair_splits = False
    assert fast.pair_split(512, 4096, 12288) == 1 and not fast.in_pairs(512, 4096, 12288)
    assert fast.plan_product(512, 4096, 12288)[:2] == (True, 2)


def test_a_changed_switch_forgets_the_remembered_plans(fast):
    fast._plans[("k",)] = "plan"
    fast._pair_widths[(1, 2, False)] = 240
    fast.pair_padding = 0.5
    assert not fast._plans and not fast._pair_widths
    fast._plans[("k",)] = "plan"
    fast.pin_stream(None)                                       # not a switch
    assert fast._plans


def test_decode_attention_split_rule(fast):
    g, n_kv = 4, 8
    assert fast.decode_splits(8, n_kv, g, 2048) == 4 and fast.decode_in_clusters(8, n_kv, g, 2048)
    assert 6 <= fast.decode_splits(1, n_kv, g, 2048) <= 8
    assert fast.decode_splits(64, n_kv, g, 2048) == 1 and fast.decode_splits(192, n_kv, g, 2048) == 1
    assert fast.decode_splits(1, n_kv, g, 32768) >= 16          # long contexts at small batches: many splits
    for batch in (1, 2, 5, 8, 12, 20, 48, 64, 160, 256):
        for ctx in (1, 100, 128, 1000, 2048, 8192, 40960):
            s = fast.decode_splits(batch, n_kv, g, ctx)
            assert 1 <= s <= 32 and (s == 1 or ctx // s >= 128)   # a split keeps at least 128 keys
    fast.force_decode_splits = 3
    assert fast.decode_splits(64, n_kv, g, 2048) == 3

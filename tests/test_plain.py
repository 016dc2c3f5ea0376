"""The plain implementation itself: each part against hand-checked values or identities."""
import math

import numpy as np
import torch

from tests.plain import model as pm


def test_rms_norm_weight_multiplies_directly():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = pm.rms_norm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    assert torch.allclose(y, torch.tensor([[6.0, 2.0]], dtype=torch.float64) / math.sqrt(12.5))


def test_rope_is_a_rotation_and_identity_at_position_zero():
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    y = pm.rope_half_split(x, [0, 5, 9], 10000.0)
    assert torch.allclose(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # pair (i, i+half): element 0 pairs with element 4 at frequency 1
    one = torch.zeros(1, 1, 8, dtype=torch.float64)
    one[0, 0, 0] = 1.0
    r = pm.rope_half_split(one, [1], 10000.0)[0, 0]
    assert abs(r[0] - math.cos(1.0)) < 1e-12 and abs(r[4] - math.sin(1.0)) < 1e-12


def test_rope_scores_depend_on_distance_only():
    q, k = torch.randn(1, 1, 16, dtype=torch.float64), torch.randn(1, 1, 16, dtype=torch.float64)
    a = (pm.rope_half_split(q, [7], 1e6) * pm.rope_half_split(k, [3], 1e6)).sum()
    b = (pm.rope_half_split(q, [104], 1e6) * pm.rope_half_split(k, [100], 1e6)).sum()
    assert abs(a - b) < 1e-9


def test_attention_is_causal_grouped_and_windowed():
    t, n_q, n_kv, d = 6, 4, 2, 8
    q, k, v = (torch.randn(t, h, d, dtype=torch.float64) for h in (n_q, n_kv, n_kv))
    out = pm.attention(q, k, v, list(range(t)))
    assert torch.allclose(out[0, 1], v[0, 0])                 # first token sees only itself; head 1 -> kv 0
    assert torch.allclose(out[0, 2], v[0, 1])                 # head 2 -> kv head 1
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 0, 0
    assert torch.allclose(pm.attention(q, k2, v2, list(range(t)))[:4], out[:4])   # the future does not matter
    w1 = pm.attention(q, k, v, list(range(t)), window=1)
    assert torch.allclose(w1, v[:, [0, 0, 1, 1]])             # a window of one key is that key's value
    s = (k[:3, 0] @ q[2, 0]) / math.sqrt(d)
    want = (torch.softmax(s, 0)[:, None] * v[:3, 0]).sum(0)
    assert torch.allclose(out[2, 0], want)


def test_swiglu():
    g, u = torch.tensor([0.0, 2.0]).double(), torch.tensor([3.0, 5.0]).double()
    assert torch.allclose(pm.swiglu(g, u), torch.tensor([0.0, 2.0 / (1 + math.exp(-2.0)) * 5.0]).double())


def test_sampling_rules():
    assert pm.argmax([1.0, 3.0, 3.0, float("nan"), float("inf")]) == 1       # lowest id on a tie; non-finite skipped
    assert pm.argmax([float("nan")]) is None
    p = pm.temperature_probs([0.0, math.log(3.0), float("-inf")], 1.0)
    assert np.allclose(p, [0.25, 0.75, 0.0])
    assert pm.select(p, 0.2499) == 0 and pm.select(p, 0.25) == 1 and pm.select(p, 0.9999999) == 1
    assert pm.select([0.5, 0.5 - 1e-17, 0.0], 1.0 - 1e-18) == 1             # falls back to the last eligible
    u = [pm.uniform(0, i) for i in range(2000)]
    assert 0.0 <= min(u) and max(u) < 1.0 and abs(np.mean(u) - 0.5) < 0.03
    assert pm.uniform(1, 5) != pm.uniform(2, 5) and pm.uniform(1, 5) == pm.uniform(1, 5)
    assert pm.splitmix64(0) == 0xE220A8397B1DCDAF                           # the published first output of splitmix64


def test_whole_model_prefix_property(tmp_path):
    """Logits at a position do not depend on later tokens."""
    from tests.tiny import make_folder
    m = pm.PlainModel(make_folder(tmp_path, "B"))
    a = m.logits([5, 9, 200, 31, 7])
    b = m.logits([5, 9, 200, 1, 1])
    assert torch.allclose(a[:3], b[:3]) and not torch.allclose(a[3], b[3])
    assert a.shape == (5, 384)


def test_truncation_stages_of_the_plain_sampler():
    """Each stage on a small row, against what its definition gives by hand
    (crates/leone/src/sampler.rs:184-234)."""
    import math
    import numpy as np
    from tests.plain.model import truncated_probs
    logits = [2.0, 1.0, 0.0, -1.0, float("-inf"), 1.0]
    base = truncated_probs(logits, 1.0, [])
    w = np.array([math.exp(x - 2.0) if math.isfinite(x) else 0.0 for x in logits])
    assert np.allclose(base, w / w.sum(), atol=1e-15) and base[4] == 0.0
    # top-k 2: the highest, and of the two tied at 1.0 the lower id
    p = truncated_probs(logits, 1.0, [("top_k", 2)])
    assert (p > 0).tolist() == [True, True, False, False, False, False] and abs(p.sum() - 1) < 1e-15
    # top-p: the shortest prefix whose mass reaches p
    order = [0, 1, 5, 2, 3]
    cum = np.cumsum([base[i] for i in order])
    for mass in (0.3, 0.6, 0.8, 0.99):
        p = truncated_probs(logits, 1.0, [("top_p", mass)])
        assert int((p > 0).sum()) == int(np.searchsorted(cum, mass) + 1)
    # min-p: at least a fraction of the highest
    p = truncated_probs(logits, 1.0, [("min_p", 0.3)])
    assert (p > 0).tolist() == [bool(b >= 0.3 * base[0]) for b in base]
    # stages see the renormalised survivors of the stage before
    two = truncated_probs(logits, 1.0, [("top_k", 3), ("epsilon", 0.25)])
    three = truncated_probs(logits, 1.0, [("top_k", 3)])
    assert (two > 0).tolist() == [bool(b >= 0.25) for b in three]
    # typical can drop the most probable token when it is atypically certain
    peaked = [6.0] + [0.0] * 600           # 0.4 on one token, 0.001 on each of 600: entropy 4.5 nats
    p = truncated_probs(peaked, 1.0, [("typical", 0.2)])
    assert p[0] == 0.0 and 195 < (p > 0).sum() < 210 and abs(p.sum() - 1) < 1e-12
    # the raw-logit stages do not depend on the temperature
    rng = np.random.default_rng(3)
    row = (rng.normal(size=200) * 2).tolist()
    for stage in (("top_n_sigma", 1.5), ("min_k", 3.0)):
        a = truncated_probs(row, 0.5, [stage]) > 0
        b = truncated_probs(row, 2.0, [stage]) > 0
        assert a.tolist() == b.tolist() and 1 <= a.sum() < 200
    # no stage empties the set
    assert (truncated_probs(row, 1.0, [("epsilon", 1.0), ("top_a", 1.0), ("tfs", 1e-9)]) > 0).sum() == 1


def test_penalties_of_the_plain_sampler_and_the_products_history_walk():
    """The plain penalties on a hand-made case, and the product's list of touched tokens
    (computed from the history on the host) against it on random histories."""
    import numpy as np
    from leone_b200.sampling.sampler import Penalties
    from tests.plain.model import apply_penalties
    logits = np.array([2.0, -1.0, 0.5, 3.0, -2.0, 1.0], dtype=np.float32)
    out = apply_penalties(logits, [0, 1, 1, 5], repetition=2.0, presence=0.25, frequency=0.5)
    assert out.tolist() == [2.0 / 2 - 0.25 - 0.5, -1.0 * 2 - 0.25 - 1.0, 0.5, 3.0, -2.0, 1.0 / 2 - 0.25 - 0.5]
    assert apply_penalties(logits, [0, 1, 1, 5], repetition=2.0, window=0).tolist() == logits.tolist()
    assert apply_penalties(logits, [0, 1, 1, 5], repetition=2.0, window=1).tolist() == [2.0, -1.0, 0.5, 3.0, -2.0, 0.5]
    # DRY: "1 2 3 4 | 2 3 9 | 1 2 3": 4 would extend a match of three, 9 a match of two
    out = apply_penalties(logits * 0, [1, 2, 3, 4, 2, 3, 5, 1, 2, 3], dry_multiplier=0.8)
    assert np.allclose(out, [0, 0, 0, 0, -0.8 * 1.75, -0.8]) and out[1] == 0
    out = apply_penalties(logits * 0, [1, 2, 3, 4, 2, 3, 5, 1, 2, 3], dry_multiplier=0.8, dry_breakers=(2,))
    assert out.tolist() == [0.0] * 6               # the match cannot cross the breaker, one token is allowed free
    rng = np.random.default_rng(5)
    for trial in range(40):
        vocab = 12
        context = rng.integers(0, vocab + 3, int(rng.integers(0, 60))).tolist()     # some ids past the vocabulary
        kw = dict(repetition=float(rng.choice([1.0, 1.3, 0.8])), presence=float(rng.choice([0.0, 0.4, -0.2])),
                  frequency=float(rng.choice([0.0, 0.1])), window=rng.choice([None, 0, 5, 64]),
                  dry_multiplier=float(rng.choice([0.0, 0.7])), dry_base=1.5, dry_allowed_length=int(rng.integers(1, 4)),
                  dry_window=int(rng.choice([0, 8, 64])), dry_breakers=tuple(rng.integers(0, vocab, 2).tolist()))
        kw["window"] = None if kw["window"] is None else int(kw["window"])
        row = rng.normal(size=vocab).astype(np.float32)
        want = apply_penalties(row, context, **kw)
        p = Penalties(**kw)
        got = row.copy()
        for token, (count, dry) in (p.touched(context).items() if p.active else ()):
            if token >= vocab:
                continue
            v = float(got[token])
            if count > 0 and p.counting:
                v = v / p.repetition if v > 0 else v * p.repetition
                v = float(np.float32(v - p.presence - p.frequency * count))
            if dry > 0:
                v = float(np.float32(v - dry))
            got[token] = v
        assert got.tolist() == want.tolist(), (trial, kw)

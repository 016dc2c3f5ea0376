"""A plain, slow implementation of the Qwen3 dense decoder for the tests.

Whole sequences, no cache, one function per part, float64 by default.  It
shares no code with ``leone_b200``: it reads ``config.json`` keys and
safetensors names itself.  It rests on the reference's formulas (each
function cites the file and line it restates); the reference's model code is
Rust and cannot be compiled or imported here, so nothing but the attention
oracle under ``tests/golden`` is checked against running reference code.
"""
from __future__ import annotations

import json
import math
import sys
import os
import struct

import numpy as np
import torch

DT = torch.float64


# ---------------------------------------------------------------------------------------
# reading a model folder (independent of the engine's loader)
# ---------------------------------------------------------------------------------------
def read_folder(folder):
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    path = os.path.join(folder, "model.safetensors")
    with open(path, "rb") as fh:
        (hlen,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(hlen))
        data = fh.read()
    np_types = {"F32": np.float32, "F16": np.float16, "I32": np.int32}
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        raw = data[b:e]
        if meta["dtype"] == "BF16":
            u16 = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32)
        else:
            arr = np.frombuffer(raw, dtype=np_types[meta["dtype"]])
        tensors[name] = torch.from_numpy(arr.astype(np.float64).reshape(meta["shape"]))
    return cfg, tensors


def round_bf16(t):
    """Round to bfloat16 and back: what a bfloat16 run keeps of a matrix."""
    return t.to(torch.float32).to(torch.bfloat16).to(t.dtype)


# ---------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------
def embedding(table, ids):
    """h[t,:] = E[id_t,:], no scale (crates/leone/src/cpu.rs:1243-1265)."""
    return table[torch.as_tensor(ids, dtype=torch.long, device=table.device)]


def rms_norm(x, weight, eps):
    """y = x * w / sqrt(mean(x^2) + eps); weight multiplies directly
    (crates/leone/src/cpu.rs:1642-1663)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * weight / torch.sqrt(ms + eps)


def linear(x, w):
    """y[r] = sum_c W[r,c] x[c], no bias (crates/leone/src/cpu.rs:1622-1640)."""
    return x @ w.t()


def rope_half_split(x, positions, theta, rotary_dim=None):
    """Half-split rotary: pair i = (i, i+half); inv_i = theta^(-2i/d), angle = pos*inv_i in
    float64 (crates/leone/src/cpu.rs:1735-1745, 1747-1779).  ``x``: [T, heads, d]."""
    d = x.shape[-1]
    rd = d if rotary_dim is None else rotary_dim
    half = rd // 2
    inv = torch.tensor([float(theta) ** (-2.0 * i / rd) for i in range(half)], dtype=torch.float64,
                       device=x.device)
    ang = torch.as_tensor(positions, dtype=torch.float64, device=x.device)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
    out = x.clone()
    a, b = x[..., :half], x[..., half:rd]
    out[..., :half] = a * cos - b * sin
    out[..., half:rd] = a * sin + b * cos
    return out


def rope_adjacent(x, positions, theta, rotary_dim=None):
    """Adjacent-pair rotary: pair i = (2i, 2i+1), the same angles as the half-split form
    (crates/leone/src/backend.rs:1216-1222, crates/leone/src/cpu.rs:1767-1770).  ``x``: [T, heads, d]."""
    d = x.shape[-1]
    rd = d if rotary_dim is None else rotary_dim
    out = x.clone()
    for t, p in enumerate(positions):
        for i in range(rd // 2):
            ang = float(p) * float(theta) ** (-2.0 * i / rd)
            c, s_ = math.cos(ang), math.sin(ang)
            a, b = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = a * c - b * s_
            out[t, :, 2 * i + 1] = a * s_ + b * c
    return out


def attention(q, k, v, positions, scale=None, window=None):
    """Causal grouped-query attention, one query row at a time.

    kv_head = q_head // (n_q/n_kv); score = (q.k) * 1/sqrt(d); the query at absolute
    position p reads keys 0..p (crates/leone/src/cpu.rs:2299-2421; mask by loop bound,
    :2372).  ``window`` (not in the reference) limits keys to p-window+1..p.
    q: [T, n_q, d], k/v: [T, n_kv, d] for the whole sequence from position 0;
    ``positions[t]`` is row t's absolute position and equals its row index in k/v.
    """
    t_len, n_q, d = q.shape
    n_kv = k.shape[1]
    g = n_q // n_kv
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out = torch.zeros_like(q)
    for t in range(t_len):
        p = int(positions[t])
        lo = 0 if window is None else max(0, p - window + 1)
        for h in range(n_q):
            kh = h // g
            s = (k[lo:p + 1, kh, :] @ q[t, h, :]) * scale
            w = torch.exp(s - s.max())
            out[t, h, :] = (w[:, None] * v[lo:p + 1, kh, :]).sum(0) / w.sum()
    return out


def swiglu(gate, up):
    """a = g / (1 + exp(-g)) * u (crates/leone/src/cpu.rs:903-905)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def attention_layer(x, w, prefix, cfg, positions, window=None):
    """q/k/v projection, per-head q/k RMSNorm with the layer eps before rotary, attention,
    output projection (crates/leone/src/runtime.rs:9111-9157; crates/leone/src/model.rs:601-631)."""
    n_q, n_kv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    d = cfg.get("head_dim", cfg["hidden_size"] // n_q)
    t_len = x.shape[0]
    q = linear(x, w[prefix + "self_attn.q_proj.weight"]).reshape(t_len, n_q, d)
    k = linear(x, w[prefix + "self_attn.k_proj.weight"]).reshape(t_len, n_kv, d)
    v = linear(x, w[prefix + "self_attn.v_proj.weight"]).reshape(t_len, n_kv, d)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], cfg["rms_norm_eps"])
    # "rope_pairing" is no key of the architecture's config.json: tests of the adjacent-pair
    # position encoding put it into the dictionary they hand to this implementation
    rope = rope_adjacent if cfg.get("rope_pairing", "half_split") == "adjacent" else rope_half_split
    q = rope(q, positions, cfg["rope_theta"])
    k = rope(k, positions, cfg["rope_theta"])
    a = attention(q, k, v, positions, window=window)
    return linear(a.reshape(t_len, n_q * d), w[prefix + "self_attn.o_proj.weight"])


def mlp_layer(x, w, prefix):
    """SwiGLU feed-forward (crates/leone/src/runtime.rs:9298-9317)."""
    g = linear(x, w[prefix + "mlp.gate_proj.weight"])
    u = linear(x, w[prefix + "mlp.up_proj.weight"])
    return linear(swiglu(g, u), w[prefix + "mlp.down_proj.weight"])


def block(h, w, i, cfg, positions):
    """Pre-norm residual block (crates/leone/src/runtime.rs:9103-9317)."""
    p = f"model.layers.{i}."
    h = h + attention_layer(rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"]),
                            w, p, cfg, positions)
    h = h + mlp_layer(rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]), w, p)
    return h


def forward_logits(cfg, w, tokens):
    """Logits [T, V] for a whole sequence from position 0
    (final norm + head: crates/leone/src/runtime.rs:7428-7452; tied head model.rs:452-471)."""
    positions = list(range(len(tokens)))
    h = embedding(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        h = block(h, w, i, cfg, positions)
    h = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(h, head)


def tensor_list(cfg):
    """(name, shape, role) of every tensor of the architecture, by the checkpoint's names
    (the reference's eleven tensors per layer, crates/leone/src/model.rs:513-560)."""
    h, i, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    out = [("model.embed_tokens.weight", (cfg["vocab_size"], h), "matrix")]
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        out += [(f"{p}.self_attn.q_proj.weight", (nq * d, h), "matrix"),
                (f"{p}.self_attn.k_proj.weight", (nkv * d, h), "matrix"),
                (f"{p}.self_attn.v_proj.weight", (nkv * d, h), "matrix"),
                (f"{p}.self_attn.o_proj.weight", (h, nq * d), "matrix"),
                (f"{p}.self_attn.q_norm.weight", (d,), "norm"),
                (f"{p}.self_attn.k_norm.weight", (d,), "norm"),
                (f"{p}.mlp.gate_proj.weight", (i, h), "matrix"),
                (f"{p}.mlp.up_proj.weight", (i, h), "matrix"),
                (f"{p}.mlp.down_proj.weight", (h, i), "matrix"),
                (f"{p}.input_layernorm.weight", (h,), "norm"),
                (f"{p}.post_attention_layernorm.weight", (h,), "norm")]
    out.append(("model.norm.weight", (h,), "norm"))
    if not cfg.get("tie_word_embeddings", False):
        out.append(("lm_head.weight", (cfg["vocab_size"], h), "matrix"))
    return out


class PlainModel:
    """A model folder read once; ``logits(tokens)`` runs the whole sequence."""

    @classmethod
    def from_seed(cls, cfg, seed, matrices_as_bf16=False):
        """No file: the seeded random weights as tests/plain/random_draw.py restates them
        (matrices N(0, 0.02), norm weights 1 + N(0, 0.1))."""
        from tests.plain import random_draw
        self = cls.__new__(cls)
        self.cfg = dict(cfg)
        self.w = {}
        for name, shape, role in tensor_list(cfg):
            t = torch.from_numpy(random_draw.draw(seed, name, shape, role, 0.1 if role == "norm" else 0.02)).double()
            self.w[name] = round_bf16(t) if (matrices_as_bf16 and t.dim() == 2) else t
        self._memo = {}
        return self

    def __init__(self, folder, matrices_as_bf16=False):
        self.cfg, self.w = read_folder(folder)
        if matrices_as_bf16:
            for name, t in self.w.items():
                if t.dim() == 2:
                    self.w[name] = round_bf16(t)
        self._memo = {}

    def logits(self, tokens):
        key = tuple(int(t) for t in tokens)
        if key not in self._memo:
            self._memo[key] = forward_logits(self.cfg, self.w, list(key))
        return self._memo[key]


# ---------------------------------------------------------------------------------------
# sampling (host, float64)
# ---------------------------------------------------------------------------------------
MASK = (1 << 64) - 1


def splitmix64(v):
    """crates/leone/src/sampler.rs:166-171."""
    z = (v + 0x9E3779B97F4A7C15) & MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def uniform(seed, position):
    """Select-purpose draw in [0,1): crates/leone/src/sampler.rs:84-94."""
    mixed = splitmix64((seed & MASK) ^ splitmix64((position ^ 0xBF58476D1CE4E5B9) & MASK))
    return (mixed >> 11) * (1.0 / (1 << 53))


def argmax(logits):
    """Highest finite logit, lowest index on a tie (crates/leone/src/sampler.rs:787-799)."""
    best, best_v = None, None
    for i, v in enumerate(logits):
        v = float(v)
        if not math.isfinite(v):
            continue
        if best is None or v > best_v:
            best, best_v = i, v
    return best


def temperature_probs(logits, temperature):
    """w_i = exp(l_i/t - max_j l_j/t) over finite logits in float64, normalised
    (crates/leone/src/sampler.rs:502-534)."""
    l = np.asarray(logits, dtype=np.float64)
    finite = np.isfinite(l)
    scaled = np.where(finite, l / temperature, -np.inf)
    w = np.where(finite, np.exp(scaled - scaled[finite].max()), 0.0)
    return w / w.sum()


def select(probs, u):
    """First token in id order whose cumulative probability exceeds u; last eligible otherwise
    (crates/leone/src/sampler.rs:839-858)."""
    c, last = 0.0, None
    for i, p in enumerate(probs):
        if p <= 0.0:
            continue
        last = i
        c += p
        if u < c:
            return i
    return last


def _entropy(kept):
    """Entropy of a normalised distribution in nats (crates/leone/src/sampler.rs:625-630)."""
    return float(sum(-p * math.log(p) for p in kept if p > 0.0))


def _threshold_keep(kept, floor):
    """Leading entries with probability >= floor (crates/leone/src/sampler.rs:635-637)."""
    n = 0
    for p in kept:
        if not p >= floor:
            break
        n += 1
    return n


def truncated_probs(logits, temperature, stages):
    """The distribution a temperature and an ordered list of truncation stages produce from one
    row of logits, float64, in id order (crates/leone/src/sampler.rs:451-469).

    ``stages``: ``(name, value)`` pairs; names top_k, top_p, min_p, top_a, tfs, typical, epsilon,
    eta, min_k, top_n_sigma (crates/leone/src/sampler.rs:184-234).  Finite logits are sorted
    descending, ties by lower id (:512-516), weights exp(l/t - l_max/t) normalised (:517-530).
    min_k and top_n_sigma read the raw logits and run first (:532-553); the others run in the
    order given, each on the renormalised survivors of the one before, always keeping at least
    the most probable token (:555-612)."""
    l = [float(x) for x in logits]
    order = sorted((i for i in range(len(l)) if math.isfinite(l[i])), key=lambda i: (-l[i], i))
    if not order:
        raise ValueError("every logit is non-finite")
    top = l[order[0]] / temperature
    kept = [math.exp(l[i] / temperature - top) for i in order]
    total = sum(kept)
    kept = [w / total for w in kept]

    def renorm(v):
        t = sum(v)
        return [x / t for x in v]

    changed = False
    for name, value in stages:
        if name == "top_n_sigma":            # crates/leone/src/sampler.rs:659-689
            if len(order) >= 2:
                n = len(order)
                mean = sum(l[i] for i in order) / n
                dev = math.sqrt(sum((l[i] - mean) ** 2 for i in order) / n)
                keep = n
                if math.isfinite(dev):
                    cut = l[order[0]] - value * dev
                    keep = max(1, _threshold_keep([l[i] for i in order], cut))
                order, kept = order[:max(keep, 1)], kept[:max(keep, 1)]
            changed = True
        elif name == "min_k":                # crates/leone/src/sampler.rs:733-762
            n = len(order)
            keep = n
            if n >= 2:
                rng = l[order[0]] - l[order[-1]] + 1e-8
                if math.isfinite(rng) and rng > 0.0:
                    cliff, best = 1, -math.inf
                    for rank in range(1, n):
                        weighted = ((l[order[rank - 1]] - l[order[rank]]) / rng) / rank
                        if weighted > best:
                            best, cliff = weighted, rank
                    fb = math.floor(value / rng)
                    fallback = min(int(fb), n) if math.isfinite(fb) and fb >= 0 else n
                    keep = min(max(cliff, fallback, 1), n)
            order, kept = order[:max(keep, 1)], kept[:max(keep, 1)]
            changed = True
    if changed:
        kept = renorm(kept)

    for name, value in stages:
        keep = None
        if name == "top_k":
            keep = min(int(value), len(kept))
        elif name == "top_p":                # shortest prefix whose mass reaches p (:640-649)
            covered, keep = 0.0, len(kept)
            for count, p in enumerate(kept):
                covered += p
                if covered >= value:
                    keep = count + 1
                    break
        elif name == "min_p":
            keep = _threshold_keep(kept, value * kept[0])
        elif name == "top_a":
            keep = _threshold_keep(kept, value * kept[0] * kept[0])
        elif name == "epsilon":
            keep = _threshold_keep(kept, value)
        elif name == "eta":                  # floor = min(eta, sqrt(eta) * exp(-H)) (:601-607)
            keep = _threshold_keep(kept, min(value, math.sqrt(value) * math.exp(-_entropy(kept))))
        elif name == "tfs":                  # crates/leone/src/sampler.rs:697-723
            keep = len(kept)
            if len(kept) >= 3:
                second = [abs(kept[s] - 2.0 * kept[s + 1] + kept[s + 2]) for s in range(len(kept) - 2)]
                tot = sum(second)
                if tot > 0.0 and math.isfinite(tot):
                    covered, keep = 0.0, 1
                    for v in second:
                        covered += v / tot
                        if covered <= value:
                            keep += 1
                        else:
                            break
        elif name == "typical":              # crates/leone/src/sampler.rs:766-790
            h = _entropy(kept)
            scored = sorted(range(len(kept)),
                            key=lambda s_: (abs(-math.log(kept[s_]) - h) if kept[s_] > 0.0 else math.inf, s_))
            covered, chosen = 0.0, []
            for s_ in scored:
                chosen.append(s_)
                covered += kept[s_]
                if covered >= value:
                    break
            chosen.sort()
            order, kept = [order[s_] for s_ in chosen], renorm([kept[s_] for s_ in chosen])
            continue
        else:
            continue                          # the raw-logit stages ran first
        keep = max(keep, 1)
        order, kept = order[:keep], renorm(kept[:keep])
    probs = np.zeros(len(l), dtype=np.float64)
    for i, p in zip(order, kept):
        probs[i] = p
    return probs


def apply_penalties(logits, context, repetition=1.0, presence=0.0, frequency=0.0, window=64,
                    dry_multiplier=0.0, dry_base=1.75, dry_allowed_length=2, dry_window=64, dry_breakers=()):
    """The logit row after the penalties, the slow and obvious way: every token of the vocabulary
    is looked up in the history (crates/leone/src/penalty.rs:163-206).  A token seen in the last
    ``window`` tokens (None: all, 0: none): positive logits are divided by ``repetition``, the
    others multiplied; ``presence`` is subtracted once and ``frequency`` once per occurrence; the
    result is rounded to float32.  DRY (:208-257): every earlier place in the last ``dry_window``
    tokens that holds the last token starts a match backwards against the end of the history
    (stopped by a breaker); from ``dry_allowed_length`` on, the token after that place is charged
    ``multiplier * base ** (length - allowed)``, the largest charge counts, subtracted in float64
    from the float32 logit."""
    out = np.array(logits, dtype=np.float32)
    context = [int(t) for t in context]
    recent = [] if window == 0 else (context if window is None else context[max(0, len(context) - window):])
    if repetition != 1.0 or presence != 0.0 or frequency != 0.0:
        for token in range(len(out)):
            count = sum(1 for t in recent if t == token)
            if count == 0:
                continue
            value = float(out[token])
            value = value / repetition if value > 0.0 else value * repetition
            value -= presence
            value -= frequency * count
            out[token] = np.float32(value)
    if dry_multiplier > 0.0 and dry_window > 0:
        recent = context[max(0, len(context) - dry_window):]
        if len(recent) >= 2:
            last = len(recent) - 1
            best = {}
            for start in range(last):
                if recent[start] != recent[last]:
                    continue
                length = 1
                while (length <= start and recent[start - length] == recent[last - length]
                       and recent[last - length] not in dry_breakers):
                    length += 1
                nxt = recent[start + 1]
                if length < dry_allowed_length or nxt in dry_breakers or nxt >= len(out):
                    continue
                charge = dry_multiplier
                for _ in range(length - dry_allowed_length):
                    charge *= dry_base
                best[nxt] = max(best.get(nxt, 0.0), charge)
            for token, charge in best.items():
                if charge > 0.0:
                    out[token] = np.float32(float(out[token]) - charge)
    return out


def mirostat_select(target, maximum_surprise, u):
    """Mirostat v2's draw (crates/leone/src/sampler.rs:383-420): of the target distribution the
    tokens whose surprise -ln p is at most the maximum are kept (the most probable one if none
    is) and renormalised, the token is drawn in id order, and its surprise under the target is
    returned with it."""
    kept = np.array([p if p > 0.0 and -math.log(p) <= maximum_surprise else 0.0 for p in target])
    if kept.sum() == 0.0:
        best = max(range(len(target)), key=lambda i: (target[i], -i))
        kept[best] = target[best]
    token = select(kept / kept.sum(), u)
    return token, -math.log(target[token])


def sample(logits, temperature, seed, position, truncations=()):
    if truncations and temperature:
        return select(truncated_probs(logits, temperature, truncations), uniform(seed, position))
    if temperature is None or temperature == 0.0:
        return argmax(logits)
    return select(temperature_probs(logits, temperature), uniform(seed, position))


def generate(model: PlainModel, prompt, max_new_tokens, temperature=0.0, seed=0, eos=None, truncations=(),
             penalties=None, mirostat=None):
    """Greedy/temperature generation by re-running the whole sequence each token.  The draw
    for a token uses the position of the token whose logits are sampled
    (crates/leone/src/runtime.rs:4945, 6080)."""
    tokens = list(prompt)
    out = []
    maximum_surprise = 2.0 * mirostat[0] if mirostat else None      # crates/leone/src/sampler.rs:138-144
    for _ in range(max_new_tokens):
        logits = model.logits(tokens)[-1].tolist()
        if penalties:
            logits = apply_penalties(np.array(logits, dtype=np.float32), tokens, **penalties).tolist()
        if mirostat and temperature:
            target = truncated_probs(logits, temperature, truncations)
            tok, observed = mirostat_select(target, maximum_surprise, uniform(seed, len(tokens) - 1))
            maximum_surprise -= mirostat[1] * (observed - mirostat[0])
            maximum_surprise = max(maximum_surprise, sys.float_info.epsilon)
            out.append(tok)
            tokens.append(tok)
            if eos is not None and tok == eos:
                break
            continue
        tok = sample(logits, temperature, seed, len(tokens) - 1, truncations)
        out.append(tok)
        tokens.append(tok)
        if eos is not None and tok == eos:
            break
    return out

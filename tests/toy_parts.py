"""Toy parts defined by the tests, outside the framework: a mixer with a state of its own, a
feed-forward that routes each token to two of several small experts, a position encoding
without a rotary table, and an architecture that mixes them with attention and the dense
feed-forward layer by layer.  Nothing here is a model of anyone's; it shows that parts are pluggable."""
from dataclasses import dataclass

import torch

from leone_b200.config.base import ConfigReader, ModelConfig
from leone_b200.parts.base import (Block, Embedding, FeedForward, FixedState, Mixer, PagedKV, PositionEncoding,
                                   WeightSpec)
from leone_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
from leone_b200.registry import ARCHITECTURES, BLOCKS, EMBEDDINGS, FEED_FORWARDS, MIXERS, POSITION_ENCODINGS


class DecayMixer(Mixer):
    """state <- decay * state + (1 - decay) * x_t;  hidden_t += W state.  The state is a
    fixed-size vector per request, kept in the request's state slot between steps."""

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.size = int(params["hidden_size"])
        self.decay = float(params["decay"])
        self.w = None

    def weight_specs(self):
        return [WeightSpec("mix.weight", (self.size, self.size))]

    def load(self, tensors):
        self.w = tensors["mix.weight"]

    def cache_request(self):
        return FixedState((self.size,))

    def forward(self, ctx, cache, x, hidden):
        if ctx.decode_only:
            # one token per sequence, no host read: this is what a captured decode step replays
            slots = ctx.slot_ids.long()
            state = self.decay * cache.state[slots] + (1.0 - self.decay) * x.float()
            cache.state.index_copy_(0, slots, state)
            hidden += state @ self.w.float().t()
            return
        slots = ctx.slot_ids.tolist()
        bounds = ctx.q_start.tolist()
        for s, slot in enumerate(slots):
            state = cache.state[slot]
            rows = []
            for t in range(bounds[s], bounds[s + 1]):
                state = self.decay * state + (1.0 - self.decay) * x[t].float()
                rows.append(state)
            cache.state[slot] = state
            hidden[bounds[s]:bounds[s + 1]] += torch.stack(rows) @ self.w.float().t()


class RoutedFeedForward(FeedForward):
    """Each token goes to the ``top_k`` experts with the largest router logits (fp32).  An
    expert's share is its logit's lead over the best expert left out, normalised, so that an
    expert enters the chosen set with share zero and the output is continuous in the input
    (rounding cannot flip a near-tie into a different result).  An expert is
    ``W_out relu(W_in x)``; hidden += the mixture."""

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["expert_size"])
        self.experts = int(params["num_experts"])
        self.top_k = int(params["top_k"])
        self.w = None

    def weight_specs(self):
        specs = [WeightSpec("router.weight", (self.experts, self.hidden))]
        for e in range(self.experts):
            specs += [WeightSpec(f"experts.{e}.in.weight", (self.inter, self.hidden)),
                      WeightSpec(f"experts.{e}.out.weight", (self.hidden, self.inter))]
        return specs

    def load(self, tensors):
        self.w = tensors

    def forward(self, ctx, x, hidden):
        xf = x.float()
        logits = xf @ self.w["router.weight"].float().t()
        top, chosen = logits.topk(self.top_k + 1, dim=-1)
        lead = top[:, :self.top_k] - top[:, self.top_k:]
        share = lead / (lead.sum(dim=-1, keepdim=True) + 1e-6)
        chosen = chosen[:, :self.top_k]
        for e in range(self.experts):
            # every row through every expert, weighted by its share there (zero where not chosen):
            # no host read, so a captured decode step can replay it
            weight = (share * (chosen == e)).sum(dim=-1, keepdim=True)
            inner = torch.relu(xf @ self.w[f"experts.{e}.in.weight"].float().t())
            hidden += (inner @ self.w[f"experts.{e}.out.weight"].float().t()) * weight


class AdditivePositions(PositionEncoding):
    """q and k get ``amplitude * sin(position * (dim index + 1) * rate)`` added: an encoding the
    attention kernel cannot fuse, applied through ``apply``."""

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.rate = float(params["rate"])
        self.amplitude = float(params["amplitude"])

    def apply(self, ctx, q, k):
        d = q.shape[-1]
        dims = torch.arange(1, d + 1, device=q.device, dtype=torch.float32)
        enc = self.amplitude * torch.sin(ctx.positions.float()[:, None] * dims[None, :] * self.rate)
        q.copy_((q.float() + enc[:, None, :]).to(q.dtype))
        k.copy_((k.float() + enc[:, None, :]).to(k.dtype))


class LatentMixer(Mixer):
    """Caches one latent vector per token, ``c_t = W_down x_t``, and nothing else: its paged cache
    has a key pool of its own width, no value pool, and is kept in float32 whatever the run
    dtype.  ``hidden_t += W_up sum_j softmax_j(c_t . c_j / sqrt(L)) c_j`` over ``j <= t``."""

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.size = int(params["hidden_size"])
        self.latent = int(params["latent_size"])
        self.w = None

    def weight_specs(self):
        return [WeightSpec("down.weight", (self.latent, self.size)), WeightSpec("up.weight", (self.size, self.latent))]

    def load(self, tensors):
        self.w = tensors

    def cache_request(self):
        return PagedKV(1, self.latent, value_head_dim=0, dtype=torch.float32, tag="latent")

    def forward(self, ctx, cache, x, hidden):
        assert cache.v_pool is None and cache.k_pool.dtype == torch.float32
        page = cache.page_tokens
        c = x.float() @ self.w["down.weight"].float().t()                      # [N, L]
        seq = ctx.seq_of_token.long()
        pos = ctx.positions.long()
        table = cache.block_table.long()                                        # [B, W]
        cache.k_pool.index_put_((table[seq, pos // page], torch.zeros_like(pos), pos % page), c)
        keys = cache.k_pool[table.clamp(min=0)][:, :, 0].flatten(1, 2)          # [B, W * page, L]
        mine = keys[seq]                                                        # [N, W * page, L]
        scores = torch.einsum("nl,nkl->nk", c, mine) / self.latent ** 0.5
        seen = torch.arange(mine.shape[1], device=c.device)[None, :] <= pos[:, None]
        probs = torch.softmax(scores.masked_fill(~seen, float("-inf")), dim=-1)
        mixed = torch.einsum("nk,nkl->nl", probs, torch.where(seen[:, :, None], mine, torch.zeros_like(mine)))
        hidden += mixed @ self.w["up.weight"].float().t()


class ParallelPostNormBlock(Block):
    """``h <- post_norm(h + mixer(norm(h)) + branch(norm(h)))``: one norm feeds the mixer and a
    feed-forward branch beside it, a second norm comes after the sum, and the usual feed-forward
    and its norm are not there at all."""

    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, branch=None, post_norm=None):
        assert feed_forward is None and ffn_norm is None and branch is not None and post_norm is not None
        super().__init__(mixer, None, mixer_norm, None, branch=branch, post_norm=post_norm)

    def forward(self, ctx, cache, hidden):
        x = self.mixer_norm.forward(ctx, hidden)
        self.mixer.forward(ctx, cache, x, hidden)
        self.branch.forward(ctx, x, hidden)
        hidden.copy_(self.post_norm.forward(ctx, hidden).float())


class PositionalEmbedding(Embedding):
    """``h_t = scale * E[id_t] + P[position_t]``: a multiplier and learned absolute positions,
    which the built-in embedding does not have."""

    def __init__(self, params, rt):
        super().__init__(params, rt)
        self.scale = float(params["scale"])
        self.max_positions = int(params["max_positions"])
        self.tokens = self.positions = None

    def weight_specs(self):
        return [WeightSpec("embed.weight", (self.params["vocab_size"], self.params["hidden_size"]), role="embedding"),
                WeightSpec("positions.weight", (self.max_positions, self.params["hidden_size"]), role="embedding")]

    def load(self, tensors):
        self.tokens, self.positions = tensors["embed.weight"], tensors["positions.weight"]

    def table(self):
        return self.tokens

    def forward(self, ctx, hidden):
        hidden.copy_(self.scale * self.tokens[ctx.token_ids.long()].float()
                     + self.positions[ctx.positions.long()].float())


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    hidden_size: int = 0
    vocab_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    max_position_embeddings: int = 0
    window: int = 0
    decay: float = 0.5
    num_experts: int = 0
    expert_size: int = 0

    @classmethod
    def from_dict(cls, raw):
        r = ConfigReader(raw)
        return cls("ToyStateLM", r.positive_int("hidden_size"), r.positive_int("vocab_size"),
                   r.positive_int("num_heads"), r.positive_int("head_dim"),
                   r.positive_int("intermediate_size"), r.positive_int("max_position_embeddings"),
                   r.positive_int("window"), r.positive_float("decay"), r.positive_int("num_experts"),
                   r.positive_int("expert_size"))


def build_toy_spec(cfg: ToyConfig) -> ModelSpec:
    norm = {"size": cfg.hidden_size, "eps": 1e-5}
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})

    routed = PartSpec("toy_routed", {"hidden_size": cfg.hidden_size, "expert_size": cfg.expert_size,
                                     "num_experts": cfg.num_experts, "top_k": 2})

    def layer(i, mixer):
        return LayerSpec(f"blocks.{i}", "pre_norm", mixer, routed if i == 1 else ffn,
                         PartSpec("rms_norm", {**norm, "name": "norm1.weight"}),
                         PartSpec("rms_norm", {**norm, "name": "norm2.weight"}))

    attn = {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads, "num_kv_heads": 1,
            "head_dim": cfg.head_dim, "qk_norm": False}
    layers = (
        layer(0, PartSpec("toy_decay", {"hidden_size": cfg.hidden_size, "decay": cfg.decay})),
        layer(1, PartSpec("attention", {**attn, "position_encoding": "additive", "window": None})),
        layer(2, PartSpec("attention", {**attn, "position_encoding": "rope", "window": cfg.window})),
    )
    return ModelSpec("ToyStateLM", cfg.hidden_size, cfg.vocab_size, cfg.max_position_embeddings,
                     "embed.weight", layers, (0, 1, 2), PartSpec("rms_norm", norm), "final_norm.weight",
                     "head.weight",
                     {"additive": PartSpec("toy_additive", {"rate": 0.01, "amplitude": 0.5}),
                      "rope": PartSpec("rotary_half_split", {"head_dim": cfg.head_dim, "rotary_dim": cfg.head_dim // 2,
                                                             "theta": 100.0, "max_positions": cfg.max_position_embeddings})})


def build_latent_spec(cfg: ToyConfig) -> ModelSpec:
    """A second toy: learned positions and a multiplier at the embedding, a latent-caching mixer,
    the state mixer beside a routed feed-forward, a layer of another arrangement (no feed-forward
    of the usual place, a parallel branch, a post-norm), and a tied head with a logit scale and a
    soft cap."""
    norm = {"size": cfg.hidden_size, "eps": 1e-5}
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    routed = PartSpec("toy_routed", {"hidden_size": cfg.hidden_size, "expert_size": cfg.expert_size,
                                     "num_experts": cfg.num_experts, "top_k": 2})

    def layer(i, mixer, feed_forward):
        return LayerSpec(f"blocks.{i}", "pre_norm", mixer, feed_forward,
                         PartSpec("rms_norm", {**norm, "name": "norm1.weight"}),
                         PartSpec("rms_norm", {**norm, "name": "norm2.weight"}))

    parallel = LayerSpec("blocks.2", "toy_parallel", PartSpec("toy_decay", {"hidden_size": cfg.hidden_size, "decay": 0.4}),
                         None, PartSpec("rms_norm", {**norm, "name": "norm1.weight"}), None,
                         extra={"branch": ("feed_forward", ffn),
                                "post_norm": ("norm", PartSpec("rms_norm", {**norm, "name": "post.weight"}))})
    layers = (layer(0, PartSpec("toy_latent", {"hidden_size": cfg.hidden_size, "latent_size": 20}), ffn),
              layer(1, PartSpec("toy_decay", {"hidden_size": cfg.hidden_size, "decay": cfg.decay}), routed),
              parallel)
    return ModelSpec("ToyLatentLM", cfg.hidden_size, cfg.vocab_size, cfg.max_position_embeddings,
                     "embed.weight", layers, (0, 1, 2), PartSpec("rms_norm", norm), "final_norm.weight", None,
                     embedding=PartSpec("toy_positional", {"scale": 1.5, "max_positions": cfg.max_position_embeddings}),
                     head=PartSpec("linear_head", {"name": None, "logit_scale": 0.5, "soft_cap": 3.0}))


@dataclass(frozen=True)
class ToyLatentConfig(ToyConfig):
    @classmethod
    def from_dict(cls, raw):
        base = ToyConfig.from_dict(raw)
        return cls(**{**base.__dict__, "architecture": "ToyLatentLM"})


def register():
    BLOCKS.register("toy_parallel", ParallelPostNormBlock)
    MIXERS.register("toy_latent", LatentMixer)
    EMBEDDINGS.register("toy_positional", PositionalEmbedding)
    ARCHITECTURES.add("ToyLatentLM", ToyLatentConfig, build_latent_spec)
    MIXERS.register("toy_decay", DecayMixer)
    FEED_FORWARDS.register("toy_routed", RoutedFeedForward)
    POSITION_ENCODINGS.register("toy_additive", AdditivePositions)
    ARCHITECTURES.add("ToyStateLM", ToyConfig, build_toy_spec)


def unregister():
    BLOCKS.unregister("toy_parallel")
    MIXERS.unregister("toy_latent")
    EMBEDDINGS.unregister("toy_positional")
    ARCHITECTURES.unregister("ToyLatentLM")
    MIXERS.unregister("toy_decay")
    FEED_FORWARDS.unregister("toy_routed")
    POSITION_ENCODINGS.unregister("toy_additive")
    ARCHITECTURES.unregister("ToyStateLM")


TOY = dict(architectures=["ToyStateLM"], hidden_size=48, vocab_size=97, num_heads=3, head_dim=32,
           intermediate_size=80, max_position_embeddings=128, window=9, decay=0.7, num_experts=5,
           expert_size=24)


def plain_logits(cfg: ToyConfig, w, tokens):
    """The toy model on a whole sequence in float64, written without the framework."""
    from tests.plain import model as pm
    w = {k: v.double() for k, v in w.items()}
    t_len = len(tokens)
    pos = list(range(t_len))
    h = w["embed.weight"][torch.tensor(tokens)]

    def ffn(x, p):
        return pm.linear(pm.swiglu(pm.linear(x, w[p + "gate_proj.weight"]), pm.linear(x, w[p + "up_proj.weight"])),
                         w[p + "down_proj.weight"])

    def routed(x, p):
        logits = x @ w[p + "router.weight"].t()
        out = torch.zeros_like(x)
        for t in range(t_len):
            top, chosen = logits[t].topk(3)
            lead = top[:2] - top[2]
            share = lead / (lead.sum() + 1e-6)
            for s, e in zip(share, chosen[:2].tolist()):
                inner = torch.relu(w[f"{p}experts.{e}.in.weight"] @ x[t])
                out[t] += s * (w[f"{p}experts.{e}.out.weight"] @ inner)
        return out

    # layer 0: decay mixer
    x = pm.rms_norm(h, w["blocks.0.norm1.weight"], 1e-5)
    state = torch.zeros(cfg.hidden_size, dtype=torch.float64)
    rows = []
    for t in range(t_len):
        state = cfg.decay * state + (1 - cfg.decay) * x[t]
        rows.append(state)
    h = h + torch.stack(rows) @ w["blocks.0.mix.weight"].t()
    h = h + ffn(pm.rms_norm(h, w["blocks.0.norm2.weight"], 1e-5), "blocks.0.")
    # layers 1, 2: attention with one kv head
    for i, window in ((1, None), (2, cfg.window)):
        p = f"blocks.{i}."
        x = pm.rms_norm(h, w[p + "norm1.weight"], 1e-5)
        q = pm.linear(x, w[p + "q_proj.weight"]).reshape(t_len, cfg.num_heads, cfg.head_dim)
        k = pm.linear(x, w[p + "k_proj.weight"]).reshape(t_len, 1, cfg.head_dim)
        v = pm.linear(x, w[p + "v_proj.weight"]).reshape(t_len, 1, cfg.head_dim)
        if i == 1:
            dims = torch.arange(1, cfg.head_dim + 1, dtype=torch.float64)
            enc = 0.5 * torch.sin(torch.tensor(pos, dtype=torch.float64)[:, None] * dims[None, :] * 0.01)
            q, k = q + enc[:, None, :], k + enc[:, None, :]
        else:
            q = pm.rope_half_split(q, pos, 100.0, rotary_dim=cfg.head_dim // 2)
            k = pm.rope_half_split(k, pos, 100.0, rotary_dim=cfg.head_dim // 2)
        a = pm.attention(q, k, v, pos, window=window).reshape(t_len, -1)
        h = h + pm.linear(a, w[p + "o_proj.weight"])
        x = pm.rms_norm(h, w[p + "norm2.weight"], 1e-5)
        h = h + (routed(x, p) if i == 1 else ffn(x, p))
    return pm.linear(pm.rms_norm(h, w["final_norm.weight"], 1e-5), w["head.weight"])


def plain_logits_latent(cfg: ToyConfig, w, tokens):
    """The second toy on a whole sequence in float64, written without the framework."""
    from tests.plain import model as pm
    w = {k: v.double() for k, v in w.items()}
    t_len = len(tokens)
    h = 1.5 * w["embed.weight"][torch.tensor(tokens)] + w["positions.weight"][:t_len]
    # layer 0: the latent mixer
    x = pm.rms_norm(h, w["blocks.0.norm1.weight"], 1e-5)
    c = x @ w["blocks.0.down.weight"].t()
    mixed = []
    for t in range(t_len):
        probs = torch.softmax(c[:t + 1] @ c[t] / 20 ** 0.5, dim=0)
        mixed.append(probs @ c[:t + 1])
    h = h + torch.stack(mixed) @ w["blocks.0.up.weight"].t()
    x = pm.rms_norm(h, w["blocks.0.norm2.weight"], 1e-5)
    h = h + pm.linear(pm.swiglu(pm.linear(x, w["blocks.0.gate_proj.weight"]), pm.linear(x, w["blocks.0.up_proj.weight"])),
                      w["blocks.0.down_proj.weight"])
    # layer 1: the state mixer and the routed feed-forward
    x = pm.rms_norm(h, w["blocks.1.norm1.weight"], 1e-5)
    state = torch.zeros(cfg.hidden_size, dtype=torch.float64)
    rows = []
    for t in range(t_len):
        state = cfg.decay * state + (1 - cfg.decay) * x[t]
        rows.append(state)
    h = h + torch.stack(rows) @ w["blocks.1.mix.weight"].t()
    x = pm.rms_norm(h, w["blocks.1.norm2.weight"], 1e-5)
    logits = x @ w["blocks.1.router.weight"].t()
    out = torch.zeros_like(x)
    for t in range(t_len):
        top, chosen = logits[t].topk(3)
        lead = top[:2] - top[2]
        share = lead / (lead.sum() + 1e-6)
        for sh, e in zip(share, chosen[:2].tolist()):
            out[t] += sh * (w[f"blocks.1.experts.{e}.out.weight"] @ torch.relu(w[f"blocks.1.experts.{e}.in.weight"] @ x[t]))
    h = h + out
    # layer 2: one norm for the state mixer and a feed-forward branch beside it, then a post-norm
    x = pm.rms_norm(h, w["blocks.2.norm1.weight"], 1e-5)
    state = torch.zeros(cfg.hidden_size, dtype=torch.float64)
    rows = []
    for t in range(t_len):
        state = 0.4 * state + 0.6 * x[t]
        rows.append(state)
    branch = pm.linear(pm.swiglu(pm.linear(x, w["blocks.2.gate_proj.weight"]), pm.linear(x, w["blocks.2.up_proj.weight"])),
                       w["blocks.2.down_proj.weight"])
    h = pm.rms_norm(h + torch.stack(rows) @ w["blocks.2.mix.weight"].t() + branch, w["blocks.2.post.weight"], 1e-5)
    raw = pm.linear(pm.rms_norm(h, w["final_norm.weight"], 1e-5), w["embed.weight"]) * 0.5
    return 3.0 * torch.tanh(raw / 3.0)

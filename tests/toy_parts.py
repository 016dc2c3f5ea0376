"""Toy parts defined by the tests, outside the framework: a mixer with a state of its own, a
feed-forward that routes each token to two of several small experts, a position encoding
without a rotary table, and an architecture that mixes them with attention and the dense
feed-forward layer by layer.  Nothing here is a model of anyone's; it shows that parts are pluggable."""
from dataclasses import dataclass

import torch

from leone_b200.config.base import ConfigReader, ModelConfig
from leone_b200.parts.base import FeedForward, FixedState, Mixer, PositionEncoding, WeightSpec
from leone_b200.parts.spec import LayerSpec, ModelSpec, PartSpec
from leone_b200.registry import ARCHITECTURES, FEED_FORWARDS, MIXERS, POSITION_ENCODINGS


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
            rows, which = (chosen == e).nonzero(as_tuple=True)
            if rows.numel() == 0:
                continue
            inner = torch.relu(xf[rows] @ self.w[f"experts.{e}.in.weight"].float().t())
            out = inner @ self.w[f"experts.{e}.out.weight"].float().t()
            hidden.index_add_(0, rows, (out * share[rows, which][:, None]).to(hidden.dtype))


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


def register():
    MIXERS.register("toy_decay", DecayMixer)
    FEED_FORWARDS.register("toy_routed", RoutedFeedForward)
    POSITION_ENCODINGS.register("toy_additive", AdditivePositions)
    ARCHITECTURES.add("ToyStateLM", ToyConfig, build_toy_spec)


def unregister():
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

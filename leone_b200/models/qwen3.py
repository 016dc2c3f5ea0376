"""Qwen3 dense decoder as a :class:`ModelSpec`.

Layer order and tensor roles follow the reference's dense layer
(crates/leone/src/model.rs:513-560 for the eleven tensors per layer,
crates/leone/src/runtime.rs:9019-9319 for the order of operations):
pre-norm → fused q/k/v projection → per-head q/k RMSNorm → half-split rotary →
cache write → causal grouped-query attention → output projection + residual →
pre-norm → SwiGLU feed-forward + residual; then the final norm and the
(optionally tied) output head for the wanted positions only
(crates/leone/src/runtime.rs:7428-7452).  Tensor names are the checkpoint's.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec
from ..registry import ARCHITECTURES


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    rope = PartSpec("rotary_half_split", {
        "head_dim": cfg.head_dim,
        "rotary_dim": cfg.head_dim,
        "theta": cfg.rope_theta,
        "max_positions": cfg.max_position_embeddings,
    })
    norm = PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    mixer = PartSpec("attention", {
        "hidden_size": cfg.hidden_size,
        "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim,
        "qk_norm": True,
        "qk_norm_eps": cfg.rms_norm_eps,   # same eps as the layer norms (model.rs:601-631)
        "position_encoding": "rope",
        "window": None,
        "q_name": "self_attn.q_proj.weight",
        "k_name": "self_attn.k_proj.weight",
        "v_name": "self_attn.v_proj.weight",
        "o_name": "self_attn.o_proj.weight",
        "q_norm_name": "self_attn.q_norm.weight",
        "k_norm_name": "self_attn.k_norm.weight",
    })
    ffn = PartSpec("swiglu", {
        "hidden_size": cfg.hidden_size,
        "intermediate_size": cfg.intermediate_size,
        "gate_name": "mlp.gate_proj.weight",
        "up_name": "mlp.up_proj.weight",
        "down_name": "mlp.down_proj.weight",
    })
    layers = tuple(
        LayerSpec(
            prefix=f"model.layers.{i}",
            block="pre_norm",
            mixer=mixer,
            feed_forward=ffn,
            mixer_norm=PartSpec(norm.kind, {**norm.params, "name": "input_layernorm.weight"}),
            ffn_norm=PartSpec(norm.kind, {**norm.params, "name": "post_attention_layernorm.weight"}),
        )
        for i in range(cfg.num_hidden_layers))
    spec = ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        layers=layers,
        run_order=tuple(range(cfg.num_hidden_layers)),
        final_norm=norm,
        final_norm_name="model.norm.weight",
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        position_encodings={"rope": rope},
        eos_token_id=cfg.eos_token_id,
        eos_token_ids=cfg.eos_token_ids,
        head=PartSpec("linear_head", {"name": None if cfg.tie_word_embeddings else "lm_head.weight",
                                      "tied_name": "lm_head.weight"}),
    )
    spec.validate()
    return spec


ARCHITECTURES.add(Qwen3Config.ARCHITECTURE, Qwen3Config, build_spec)

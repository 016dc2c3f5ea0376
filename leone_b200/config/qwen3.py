"""Typed configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

Keys are those of the architecture's own ``config.json``.  Quantities and
checks follow the reference's ``ModelConfig`` (crates/leone/src/model.rs:54-67,
``from_gguf`` :716-741, ``validate_head_dim`` :773-780) and the metadata reader
(crates/leone-gguf/src/model.rs:83-153).  One deliberate difference: the
reference requires ``head_dim == hidden_size / num_attention_heads``
(crates/leone/src/model.rs:773-780); here ``head_dim`` is independent of
``hidden_size`` because several Qwen3 sizes need that.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigReader, InvalidValue, ModelConfig, UnsupportedField, read_stop_ids


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    num_hidden_layers: int = 0
    hidden_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    rope_theta: float = 0.0
    rms_norm_eps: float = 0.0
    max_position_embeddings: int = 0
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    eos_token_id: Optional[int] = None         # the first stop id
    eos_token_ids: Tuple[int, ...] = ()        # all of them (config.json may list several)

    ARCHITECTURE = "Qwen3ForCausalLM"

    def to_json_dict(self) -> dict:
        out = super().to_json_dict()
        ids = out.pop("eos_token_ids", ())
        if len(ids) > 1:
            out["eos_token_id"] = list(ids)
        return out

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        r = ConfigReader(raw)
        n_q = r.positive_int("num_attention_heads")
        hidden = r.positive_int("hidden_size")
        n_kv = r.positive_int("num_key_value_heads", n_q)
        if n_q % n_kv != 0:
            # crates/leone-gguf/src/model.rs:148-153 (InvalidGqa)
            raise InvalidValue(
                f"config.json: num_attention_heads ({n_q}) must be a multiple of "
                f"num_key_value_heads ({n_kv})")
        if r.has("head_dim"):
            head_dim = r.positive_int("head_dim")
        else:
            if hidden % n_q != 0:
                raise InvalidValue(
                    f"config.json: no 'head_dim' and hidden_size ({hidden}) is not a "
                    f"multiple of num_attention_heads ({n_q})")
            head_dim = hidden // n_q
        if head_dim % 2 != 0:
            raise InvalidValue(f"config.json: head_dim ({head_dim}) must be even for rotary pairs")
        # The reference rejects every kind of rope scaling (crates/leone/src/model.rs:252-256).
        r.must_be_absent_or("rope_scaling", (None,), "rope scaling is not implemented")
        r.must_be_absent_or("use_sliding_window", (None, False),
                            "this architecture is run with full causal attention only")
        r.must_be_absent_or("attention_bias", (None, False), "no bias tensors are read")
        r.must_be_absent_or("mlp_bias", (None, False), "no bias tensors are read")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise UnsupportedField(f"config.json: hidden_act '{act}' is not supported (silu only)")
        vocab = r.positive_int("vocab_size")
        stop_ids = read_stop_ids(raw, vocab)
        eos = stop_ids[0] if stop_ids else None
        return cls(
            architecture=cls.ARCHITECTURE,
            num_hidden_layers=r.positive_int("num_hidden_layers"),
            hidden_size=hidden,
            num_attention_heads=n_q,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            intermediate_size=r.positive_int("intermediate_size"),
            vocab_size=vocab,
            rope_theta=r.positive_float("rope_theta"),
            rms_norm_eps=r.positive_float("rms_norm_eps"),
            max_position_embeddings=r.positive_int("max_position_embeddings"),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            hidden_act=act,
            eos_token_id=eos,
            eos_token_ids=stop_ids,
        )

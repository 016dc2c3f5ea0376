"""Typed reading of a model folder's ``config.json``.

Every architecture has one frozen dataclass derived from :class:`ModelConfig`.
All sizes and constants of a model come from here; no part of the engine
holds a size of its own.  The checks mirror the reference's config errors
(crates/leone-gguf/src/model.rs:60-79 ``Missing``/``WrongType``/``Zero``/
``InvalidFloat``/``InvalidGqa``; crates/leone/src/model.rs:80-87
``UnsupportedField``/``DimensionRelation``).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, fields
from typing import Any, Mapping


class ConfigError(ValueError):
    """A ``config.json`` that cannot describe a model this engine runs."""


class MissingKey(ConfigError):
    pass


class WrongType(ConfigError):
    pass


class InvalidValue(ConfigError):
    pass


class UnsupportedField(ConfigError):
    pass


class UnsupportedArchitecture(ConfigError):
    pass


_ABSENT = object()


class ConfigReader:
    """Checked access to the keys of one ``config.json`` mapping."""

    def __init__(self, raw: Mapping[str, Any]):
        if not isinstance(raw, Mapping):
            raise WrongType("config.json must hold a JSON object")
        self.raw = raw

    def has(self, key: str) -> bool:
        return key in self.raw and self.raw[key] is not None

    def positive_int(self, key: str, default: Any = _ABSENT) -> int:
        if not self.has(key):
            if default is _ABSENT:
                raise MissingKey(f"config.json: missing key '{key}'")
            return default
        value = self.raw[key]
        if isinstance(value, bool) or not isinstance(value, int):
            raise WrongType(f"config.json: '{key}' must be an integer, got {value!r}")
        if value <= 0:
            raise InvalidValue(f"config.json: '{key}' must be > 0, got {value}")
        return value

    def optional_int(self, key: str) -> int | None:
        if not self.has(key):
            return None
        value = self.raw[key]
        if isinstance(value, bool) or not isinstance(value, int):
            raise WrongType(f"config.json: '{key}' must be an integer, got {value!r}")
        return value

    def positive_float(self, key: str, default: Any = _ABSENT) -> float:
        if not self.has(key):
            if default is _ABSENT:
                raise MissingKey(f"config.json: missing key '{key}'")
            return default
        value = self.raw[key]
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise WrongType(f"config.json: '{key}' must be a number, got {value!r}")
        value = float(value)
        if not math.isfinite(value) or value <= 0.0:
            raise InvalidValue(f"config.json: '{key}' must be finite and > 0, got {value}")
        return value

    def boolean(self, key: str, default: bool) -> bool:
        if not self.has(key):
            return default
        value = self.raw[key]
        if not isinstance(value, bool):
            raise WrongType(f"config.json: '{key}' must be true or false, got {value!r}")
        return value

    def string(self, key: str, default: Any = _ABSENT) -> str:
        if not self.has(key):
            if default is _ABSENT:
                raise MissingKey(f"config.json: missing key '{key}'")
            return default
        value = self.raw[key]
        if not isinstance(value, str):
            raise WrongType(f"config.json: '{key}' must be a string, got {value!r}")
        return value

    def must_be_absent_or(self, key: str, allowed: tuple, why: str) -> None:
        if key in self.raw and self.raw[key] not in allowed:
            raise UnsupportedField(
                f"config.json: '{key}' = {self.raw[key]!r} is not supported ({why})")


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration."""

    architecture: str

    def to_json_dict(self) -> dict:
        out = {}
        for f in fields(self):
            if f.name == "architecture":
                continue
            value = getattr(self, f.name)
            if value is not None:
                out[f.name] = value
        out["architectures"] = [self.architecture]
        return out

    def write(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(self.to_json_dict(), fh, indent=1)


def read_stop_ids(raw: Mapping[str, Any], vocab_size: int) -> tuple:
    """``eos_token_id`` as a tuple of ids: the key may hold one id or a list of them (every one
    of which ends a request).  The reference stops on its tokenizer's single end id
    (crates/leone/src/runtime.rs:5383); checkpoints of this architecture may list several."""
    value = raw.get("eos_token_id")
    if value is None:
        return ()
    ids = value if isinstance(value, list) else [value]
    out = []
    for i in ids:
        if isinstance(i, bool) or not isinstance(i, int):
            raise WrongType(f"config.json: 'eos_token_id' must be an integer or a list of integers, got {value!r}")
        if not 0 <= i < vocab_size:
            raise InvalidValue(f"config.json: eos_token_id {i} is outside the vocabulary ({vocab_size})")
        if i not in out:
            out.append(i)
    return tuple(out)


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json")
    with open(path) as fh:
        try:
            raw = json.load(fh)
        except json.JSONDecodeError as err:
            raise ConfigError(f"{path}: not valid JSON ({err})") from None
    if not isinstance(raw, dict):
        raise WrongType(f"{path}: must hold a JSON object")
    # generation_config.json beside it may name the stop ids when config.json does not
    gen_path = os.path.join(folder, "generation_config.json")
    if raw.get("eos_token_id") is None and os.path.isfile(gen_path):
        try:
            with open(gen_path) as fh:
                gen = json.load(fh)
        except json.JSONDecodeError as err:
            raise ConfigError(f"{gen_path}: not valid JSON ({err})") from None
        if isinstance(gen, dict) and gen.get("eos_token_id") is not None:
            raw["eos_token_id"] = gen["eos_token_id"]
    return raw


def architecture_name(raw: Mapping[str, Any]) -> str:
    names = raw.get("architectures")
    if not isinstance(names, list) or len(names) < 1 or not isinstance(names[0], str):
        raise MissingKey("config.json: 'architectures' must be a list with the model class name")
    return names[0]

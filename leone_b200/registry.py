"""Name → factory tables: one for architectures and one per kind of part.

An architecture is registered with its configuration class and a function
that turns a configuration into a :class:`~leone_b200.parts.spec.ModelSpec`
(the reference's counterpart is the architecture support table,
crates/leone-gguf/src/support.rs:39-56, and ``ModelArchitecture::from_gguf``,
crates/leone/src/model.rs:23-31).  Parts (mixer, feed-forward, norm, position
encoding, block arrangement, embedding, output head) are registered by kind name and looked up layer
by layer from the spec, so code outside this package can add one without
touching any file here.
"""
from __future__ import annotations

from typing import Callable, Dict

from .config.base import UnsupportedArchitecture


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._table: Dict[str, object] = {}

    def register(self, name: str, item=None):
        """Use as ``REG.register("name", obj)`` or as a decorator."""
        def put(obj):
            self._table[name] = obj
            return obj
        if item is not None:
            return put(item)
        return put

    def unregister(self, name: str) -> None:
        self._table.pop(name, None)

    def get(self, name: str):
        if name not in self._table:
            known = ", ".join(sorted(self._table)) or "(none)"
            raise KeyError(f"unknown {self.what} '{name}'; registered: {known}")
        return self._table[name]

    def names(self):
        return sorted(self._table)

    def __contains__(self, name: str) -> bool:
        return name in self._table


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")


class ArchitectureEntry:
    def __init__(self, name: str, config_class, build_spec: Callable):
        self.name = name
        self.config_class = config_class
        self.build_spec = build_spec


class ArchitectureRegistry(Registry):
    def __init__(self):
        super().__init__("architecture")

    def add(self, name: str, config_class, build_spec: Callable) -> None:
        self.register(name, ArchitectureEntry(name, config_class, build_spec))

    def get(self, name: str) -> ArchitectureEntry:
        if name not in self._table:
            known = ", ".join(sorted(self._table)) or "(none)"
            raise UnsupportedArchitecture(
                f"architecture '{name}' is not supported; known architectures: {known}")
        return self._table[name]


ARCHITECTURES = ArchitectureRegistry()


def config_from_folder(folder: str):
    """Read ``folder/config.json`` into the typed configuration of its architecture."""
    from .config.base import architecture_name, read_config_json
    raw = read_config_json(folder)
    return config_from_dict(raw)


def config_from_dict(raw: dict):
    from .config.base import architecture_name
    from . import models  # noqa: F401  (registers the built-in architectures)
    entry = ARCHITECTURES.get(architecture_name(raw))
    return entry.config_class.from_dict(raw)


def spec_from_config(config):
    from . import models  # noqa: F401
    return ARCHITECTURES.get(config.architecture).build_spec(config)

"""Registries: from a part's kind to its class, and from an architecture's name (the
first entry of config.json's ``architectures``) to its typed configuration and to the
function that turns that configuration into a ModelSpec.

AIR has no registry: it refuses every architecture but one by name
(src/model/qwen2_contract.cpp:35).  Here that one name is an entry, and a second
architecture is a second entry.
"""
from __future__ import annotations

from typing import Callable, Dict, NamedTuple


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, type] = {}

    def register(self, kind: str, cls=None):
        def put(c):
            self._items[kind] = c
            return c
        return put(cls) if cls is not None else put

    def get(self, kind: str):
        try:
            return self._items[kind]
        except KeyError:
            known = ", ".join(sorted(self._items)) or "none"
            raise KeyError(f"no {self.what} of kind '{kind}' is registered (known: {known})") from None

    def kinds(self):
        return sorted(self._items)


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITION_ENCODINGS = _Registry("position encoding")
BLOCKS = _Registry("block arrangement")


def register_mixer(kind, cls=None):
    return MIXERS.register(kind, cls)


def register_feed_forward(kind, cls=None):
    return FEED_FORWARDS.register(kind, cls)


def register_norm(kind, cls=None):
    return NORMS.register(kind, cls)


def register_position_encoding(kind, cls=None):
    return POSITION_ENCODINGS.register(kind, cls)


def register_block(kind, cls=None):
    return BLOCKS.register(kind, cls)


class Architecture(NamedTuple):
    name: str
    config_class: type       # has from_dict(dict) and to_dict()
    build_spec: Callable     # config -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def architecture(name: str) -> Architecture:
    from ..config.model_config import ConfigError
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "none"
        raise ConfigError("unsupported", f"architecture '{name}' is not registered (known: {known})") from None


def architectures():
    return sorted(_ARCHITECTURES)

"""Registries: architecture name -> model builder, and part kind -> part class.

The reference maps the GGUF architecture string to a model kind and answers an unknown name
with the list of names it knows (src/dense.rs:35-46).  Here the same happens for config.json's
`architectures[0]` / `model_type`, and every family of parts has a registry of its own so that
a new mixer, feed-forward, norm, position encoding or block arrangement is added by
registering a class, without touching the engine.
"""
from __future__ import annotations

from typing import Any, Callable


class RegistryError(KeyError):
    def __str__(self) -> str:  # KeyError would quote the message
        return self.args[0] if self.args else ""


class Registry:
    def __init__(self, family: str):
        self.family = family
        self._items: dict[str, Any] = {}

    def register(self, *names: str, replace: bool = False) -> Callable:
        def deco(obj):
            for n in names:
                if n in self._items and not replace and self._items[n] is not obj:
                    raise RegistryError(f"{self.family} '{n}' is already registered")
                self._items[n] = obj
            return obj
        return deco

    def get(self, name: str):
        try:
            return self._items[name]
        except KeyError:
            raise RegistryError(
                f"unknown {self.family} '{name}'; registered: {', '.join(sorted(self._items)) or '(none)'}"
            ) from None

    def unregister(self, *names: str) -> None:
        for n in names:
            self._items.pop(n, None)

    def names(self) -> list[str]:
        return sorted(self._items)

    def __contains__(self, name: str) -> bool:
        return name in self._items


# architecture name -> function(raw config dict) -> parts.base.ModelPlan
ARCHITECTURES = Registry("architecture")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")


def plan_from_config(raw: dict):
    """config.json (parsed) -> ModelPlan, through the architecture registry."""
    from .config.base import architecture_name
    from . import arch  # noqa: F401  (registers the built-in architecture)

    name = architecture_name(raw)
    return ARCHITECTURES.get(name)(raw)

"""Name -> constructor tables: one for architectures, one for each kind of part.

`architectures[0]` of config.json picks the reader that turns the file into a
ModelSpec; the kind strings inside the spec pick the parts. An unknown name is
refused with the sorted list of known ones; registering an empty name, a missing
constructor or a name twice is a programming error and raises at once
(model/model.go:95-111, :145-173).
"""
from __future__ import annotations

from typing import Callable, Dict


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._table: Dict[str, Callable] = {}

    def register(self, name: str, ctor: Callable, *, replace: bool = False) -> None:
        if not name:
            raise ValueError(f"registry: a {self.what} needs a name")
        if ctor is None:
            raise ValueError(f"registry: {self.what} {name!r} has no constructor")
        if name in self._table and not replace:
            raise ValueError(f"registry: {self.what} {name!r} is registered twice")
        self._table[name] = ctor

    def unregister(self, name: str) -> None:
        self._table.pop(name, None)

    def get(self, name: str) -> Callable:
        try:
            return self._table[name]
        except KeyError:
            known = ", ".join(sorted(self._table)) or "none"
            raise KeyError(f"registry: unknown {self.what} {name!r}; known: {known}") from None

    def names(self):
        return sorted(self._table)

    def __contains__(self, name: str) -> bool:
        return name in self._table


ARCHITECTURES = Registry("architecture")   # name -> (config dict -> ModelSpec)
MIXERS = Registry("mixer")                 # kind -> part class
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block")


def model_spec_from_config(raw: dict):
    """config.json as a dict -> ModelSpec, by architectures[0] (model/model.go:131-192)."""
    archs = raw.get("architectures") if isinstance(raw, dict) else None
    if not archs or not isinstance(archs, list) or not archs[0]:
        raise ValueError("config: architectures[0] is required; it is the registry key")
    return ARCHITECTURES.get(archs[0])(raw)


def _register_builtin() -> None:
    from .config.qwen3 import ARCHITECTURE, qwen3_model_spec
    if ARCHITECTURE not in ARCHITECTURES:
        ARCHITECTURES.register(ARCHITECTURE, qwen3_model_spec)


_register_builtin()

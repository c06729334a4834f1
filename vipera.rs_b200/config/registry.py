"""Registries: architecture name to its configuration and model description, and
part kind to the class that builds it.

The reference has this pattern for samplers (a static table looked up by name,
crates/vipera-traits/src/sampler.rs:99-132, crates/vipera-sampler/src/lib.rs:121)
and specifies one for backends (specs/001-vipera-rs-engine/data-model.md:95-99).
Here one ``Registry`` type serves architectures, mixers, feed-forwards, norms,
position encodings and block arrangements alike.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Any, Callable, Dict, Generic, List, TypeVar

from ..errors import UnsupportedError

T = TypeVar("T")


class Registry(Generic[T]):
    """A table from name to entry; unknown names fail with the list of known ones."""

    def __init__(self, what: str):
        self._what = what
        self._entries: Dict[str, T] = {}

    def register(self, name: str, entry: T, *, replace: bool = False) -> T:
        if name in self._entries and not replace:
            raise ValueError(f"{self._what} {name!r} is already registered")
        self._entries[name] = entry
        return entry

    def unregister(self, name: str) -> None:
        self._entries.pop(name, None)

    def find(self, name: str) -> T:
        try:
            return self._entries[name]
        except KeyError:
            known = ", ".join(sorted(self._entries)) or "none"
            raise UnsupportedError(
                f"unknown {self._what} {name!r}; registered: {known}"
            ) from None

    def names(self) -> List[str]:
        return sorted(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def __len__(self) -> int:
        return len(self._entries)


@dataclass(frozen=True)
class Architecture:
    """What an architecture brings: how to read its config.json and how to
    describe its model in terms of parts."""

    name: str
    config_from_dict: Callable[[Dict[str, Any]], Any]
    model_spec: Callable[[Any], "ModelSpec"]  # noqa: F821
    # Other names a weight file may use: ``tensor_alias(name_in_file)`` returns the name the
    # parts ask for, or None where the name is not an alias.
    tensor_alias: Optional[Callable[[str], Optional[str]]] = None


ARCHITECTURES: Registry[Architecture] = Registry("architecture")
MIXERS: Registry[type] = Registry("mixer")
FEED_FORWARDS: Registry[type] = Registry("feed-forward")
NORMS: Registry[type] = Registry("norm")
POSITION_ENCODINGS: Registry[type] = Registry("position encoding")
BLOCKS: Registry[type] = Registry("block arrangement")


def register_architecture(name, config_from_dict, model_spec, *, tensor_alias=None, replace=False) -> Architecture:
    return ARCHITECTURES.register(
        name, Architecture(name, config_from_dict, model_spec, tensor_alias), replace=replace
    )

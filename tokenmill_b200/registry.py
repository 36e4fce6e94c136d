"""Registries: architecture name -> (config type, spec builder); part kind -> part class.

The reference hard-codes its one model class (src/infer/model/loader.py:18,55) and never reads
``architectures``. Here ``config.json["architectures"][0]`` picks the entry, and every mixer,
feed-forward, norm and position encoding is looked up by the ``kind`` a layer specification names, so a
new part or a whole new architecture is added by registering it — no framework file changes.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable


class RegistryError(KeyError):
    def __str__(self) -> str:  # KeyError quotes its message; keep it readable
        return str(self.args[0]) if self.args else ""


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[dict, dict | None], Any]   # (config.json, generation_config.json) -> typed config
    build_spec: Callable[[Any], Any]                        # typed config -> ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}
_PARTS: dict[str, dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def register_architecture(name: str, config_from_dict, build_spec, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise RegistryError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, build_spec)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise RegistryError(f"unknown architecture {name!r}; registered: {sorted(_ARCHITECTURES)}") from None


def architecture_names() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def register_part(role: str, kind: str, cls: type, *, replace: bool = False) -> None:
    """role: mixer | feed_forward | norm | position | block."""
    if role not in _PARTS:
        raise RegistryError(f"unknown part role {role!r}; roles: {sorted(_PARTS)}")
    if kind in _PARTS[role] and not replace:
        raise RegistryError(f"{role} kind {kind!r} is already registered")
    _PARTS[role][kind] = cls


def get_part(role: str, kind: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[role][kind]
    except KeyError:
        known = sorted(_PARTS.get(role, {}))
        raise RegistryError(f"unknown {role} kind {kind!r}; registered: {known}") from None


def register_mixer(kind: str, cls: type, **kw) -> None:
    register_part("mixer", kind, cls, **kw)


def register_feed_forward(kind: str, cls: type, **kw) -> None:
    register_part("feed_forward", kind, cls, **kw)


def register_norm(kind: str, cls: type, **kw) -> None:
    register_part("norm", kind, cls, **kw)


def register_position_encoding(kind: str, cls: type, **kw) -> None:
    register_part("position", kind, cls, **kw)


def register_block(kind: str, cls: type, **kw) -> None:
    register_part("block", kind, cls, **kw)


_builtin_loaded = False


def _ensure_builtin() -> None:
    """Import the modules whose import registers the built-in parts and the Qwen2 architecture."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    import tokenmill_b200.parts  # noqa: F401  (registers parts)
    import tokenmill_b200.models  # noqa: F401  (registers architectures)

"""Registries of part kinds.

A part is looked up by the ``kind`` string of its spec.  The framework's own
parts register themselves on import; a caller adds another mixer,
feed-forward, norm, position encoding, block arrangement, embedding or head with the matching
``register_*`` function and names it in a plan.  No framework file has to
change for that.
"""
from __future__ import annotations

from typing import Any, Callable, Dict

_KINDS = ("norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head")
_TABLES: Dict[str, Dict[str, Any]] = {k: {} for k in _KINDS}


def _register(table: str, kind: str, cls: Any) -> Any:
    _TABLES[table][kind] = cls
    return cls


def _lookup(table: str, kind: str) -> Any:
    try:
        return _TABLES[table][kind]
    except KeyError:
        raise KeyError(f"no {table} part named {kind!r}; registered: {sorted(_TABLES[table])}") from None


def register_norm(kind: str, cls: Any) -> Any: return _register("norm", kind, cls)
def register_position(kind: str, cls: Any) -> Any: return _register("position", kind, cls)
def register_mixer(kind: str, cls: Any) -> Any: return _register("mixer", kind, cls)
def register_feed_forward(kind: str, cls: Any) -> Any: return _register("feed_forward", kind, cls)
def register_arrangement(kind: str, cls: Any) -> Any: return _register("arrangement", kind, cls)
def register_embedding(kind: str, cls: Any) -> Any: return _register("embedding", kind, cls)
def register_head(kind: str, cls: Any) -> Any: return _register("head", kind, cls)


def norm_class(kind: str) -> Any: return _lookup("norm", kind)
def position_class(kind: str) -> Any: return _lookup("position", kind)
def mixer_class(kind: str) -> Any: return _lookup("mixer", kind)
def feed_forward_class(kind: str) -> Any: return _lookup("feed_forward", kind)
def arrangement_class(kind: str) -> Any: return _lookup("arrangement", kind)
def embedding_class(kind: str) -> Any: return _lookup("embedding", kind)
def head_class(kind: str) -> Any: return _lookup("head", kind)


def unregister(table: str, kind: str) -> None:
    _TABLES[table].pop(kind, None)

"""The one registry from an architecture's name to its model.

An architecture is a configuration class (``from_dict`` / ``to_dict``) and a
plan builder that turns a typed configuration into a ``ModelPlan``.  It is
looked up by ``config.json``'s ``architectures[0]`` and then by its
``model_type``.  The reference has a two-value enum and treats every
``model_type`` that is not GLM as Llama (src/model.h:18, src/model.cpp:86-96);
here an unknown name is an error that lists what is registered.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Sequence

from .fields import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                       # has from_dict(dict) and to_dict()
    build_plan: Callable[[Any], Any]        # typed config -> parts.spec.ModelPlan


_BY_NAME: Dict[str, Architecture] = {}


def register_architecture(names: Sequence[str], config_class: Any,
                          build_plan: Callable[[Any], Any]) -> Architecture:
    """Registers one architecture under every name in ``names`` (class names
    from ``architectures`` and ``model_type`` strings alike)."""
    if not names:
        raise ValueError("register_architecture: no names given")
    arch = Architecture(names[0], config_class, build_plan)
    for n in names:
        _BY_NAME[n] = arch
    return arch


def unregister_architecture(names: Sequence[str]) -> None:
    for n in names:
        _BY_NAME.pop(n, None)


def registered_names() -> List[str]:
    return sorted(_BY_NAME)


def resolve_architecture(config_obj: Dict[str, Any]) -> Architecture:
    """Finds the architecture that a parsed config.json names."""
    tried: List[str] = []
    archs = config_obj.get("architectures")
    if isinstance(archs, list):
        for a in archs:
            if isinstance(a, str):
                tried.append(a)
                if a in _BY_NAME:
                    return _BY_NAME[a]
    mt = config_obj.get("model_type")
    if isinstance(mt, str):
        tried.append(mt)
        if mt in _BY_NAME:
            return _BY_NAME[mt]
    if not tried:
        raise ConfigError("config.json: neither 'architectures' nor 'model_type' names an architecture; "
                          "registered: " + ", ".join(registered_names()))
    raise ConfigError("config.json: unknown architecture " + " / ".join(repr(t) for t in tried)
                      + "; registered: " + ", ".join(registered_names()))

"""Registries: architecture name -> model plan, and part kind -> part class.

One table maps an architecture's name (config.json `architectures[0]`, or its
`model_type`) to the class that reads its configuration and the function that
turns a configuration into a ModelPlan. Five smaller tables map the kind names
a plan uses ("attention", "gated_mlp", "rms_norm", "rope", "pre_norm") to the
classes that implement them. Tests and users add entries with the register_*
functions; nothing below the registry is keyed on a model's name
(the reference keeps numerical policy as data for the same reason,
docs/architecture.md:34-36).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Sequence

from .errors import InvalidError, UnsupportedError


@dataclass(frozen=True)
class Architecture:
    name: str
    model_types: Sequence[str]
    config_class: Any  # has from_dict(dict) and to_dict()
    plan: Callable[[Any], "ModelPlan"]  # noqa: F821  (parts.base.ModelPlan)


ARCHITECTURES: Dict[str, Architecture] = {}
MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}


def register_architecture(name: str, config_class, plan, model_types: Sequence[str] = ()) -> None:
    ARCHITECTURES[name] = Architecture(name, tuple(model_types), config_class, plan)


def _register(table: Dict[str, type], kind: str):
    def wrap(cls):
        table[kind] = cls
        cls.kind = kind
        return cls
    return wrap


def register_mixer(kind: str):
    return _register(MIXERS, kind)


def register_feed_forward(kind: str):
    return _register(FEED_FORWARDS, kind)


def register_norm(kind: str):
    return _register(NORMS, kind)


def register_position_encoding(kind: str):
    return _register(POSITION_ENCODINGS, kind)


def register_block(kind: str):
    return _register(BLOCKS, kind)


def find_architecture(root: Mapping[str, Any]) -> Architecture:
    """The registered architecture a config.json names.

    `architectures[0]` is looked up first; the reference keys on `model_type`
    (crates/model-format/src/mlx/config.rs:28-44), which is the second try.
    """
    _ensure_builtin()
    archs = root.get("architectures")
    if isinstance(archs, list):
        for name in archs:
            if name in ARCHITECTURES:
                return ARCHITECTURES[name]
    kind = root.get("model_type")
    for arch in ARCHITECTURES.values():
        if kind is not None and kind in arch.model_types:
            return arch
    if kind is None and not isinstance(archs, list):
        raise InvalidError("config.model_type")
    raise UnsupportedError(
        f"architecture {archs if isinstance(archs, list) else kind!r} is not registered "
        f"(registered: {', '.join(sorted(ARCHITECTURES))})")


def build_part(table: Dict[str, type], spec, family: str):
    if spec.kind not in table:
        raise UnsupportedError(f"{family} kind {spec.kind!r} is not registered "
                               f"(registered: {', '.join(sorted(table))})")
    return table[spec.kind](**spec.params)


def _ensure_builtin() -> None:
    """Import the built-in parts and models so that their register_* calls have run."""
    from . import parts, models  # noqa: F401

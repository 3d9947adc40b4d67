"""Typed readers for config.json keys.

Same rules as the reference's `number`/`real` helpers
(crates/model-format/src/mlx/config.rs:7-25): a missing required key is an
error that names the key, integers above 1,000,000 are rejected, reals must be
finite.
"""
from __future__ import annotations

import json
import math
import os
from typing import Any, Mapping

from ..errors import InvalidError

INTEGER_LIMIT = 1_000_000
_MISSING = object()


def read_int(table: Mapping[str, Any], key: str, default: Any = _MISSING) -> int:
    value = table.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value < 0:
        if default is _MISSING:
            raise InvalidError(f"missing config.{key}")
        value = default
    if value is not None and value > INTEGER_LIMIT:
        raise InvalidError(f"config.{key} exceeds supported limit")
    return value


def read_real(table: Mapping[str, Any], key: str, default: float) -> float:
    value = table.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        value = default
    value = float(value)
    if not math.isfinite(value):
        raise InvalidError(f"nonfinite config.{key}")
    return value


def read_bool(table: Mapping[str, Any], key: str, default: bool) -> bool:
    value = table.get(key)
    return value if isinstance(value, bool) else default


def read_config_json(model_dir: str) -> dict:
    """config.json of a model folder as a dict; a clear error if absent or not an object."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            root = json.load(handle)
    except FileNotFoundError:
        raise InvalidError(f"{model_dir}: no config.json") from None
    except json.JSONDecodeError as exc:
        raise InvalidError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(root, dict):
        raise InvalidError(f"{path}: top level must be an object")
    return root


def read_generation_eos(model_dir: str) -> tuple:
    """Stop ids from generation_config.json if the folder has one (ids only).

    The reference gathers its stop set from the tokenizer and from
    generation_config.json (crates/llama-rs/src/tokenizer/huggingface.rs:68-96);
    token strings are outside this library, ids are kept.
    """
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return ()
    try:
        with open(path, "r", encoding="utf-8") as handle:
            return normalize_token_ids(json.load(handle).get("eos_token_id"))
    except (json.JSONDecodeError, AttributeError):
        return ()


def normalize_token_ids(value: Any) -> tuple:
    """`eos_token_id` may be an int, a list of ints or absent."""
    if isinstance(value, bool) or value is None:
        return ()
    if isinstance(value, int):
        return (value,) if value >= 0 else ()
    if isinstance(value, (list, tuple)):
        return tuple(v for v in value if isinstance(v, int) and not isinstance(v, bool) and v >= 0)
    return ()

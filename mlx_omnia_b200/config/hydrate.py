"""Typed configuration read from a checkpoint's config.json.

A configuration is a frozen dataclass whose field names are the checkpoint's own
keys. `hydrate` fills one from a parsed JSON object: keys the dataclass does not
name are dropped, nested dataclasses recurse, lists become tuples (so the value
stays hashable), and a key without a default that the file lacks is an error that
names it. This is the behaviour of the reference's `load_config`
(src/mlx_omnia/engine/core/config.py:12-42), with the missing-key message added.
"""

from __future__ import annotations

import dataclasses
import json
import types
import typing
from pathlib import Path
from typing import Any, TypeVar

T = TypeVar("T")


class ConfigError(ValueError):
    """A config.json that the named architecture cannot be built from."""


def read_json(source: dict[str, Any] | str | Path) -> dict[str, Any]:
    if isinstance(source, dict):
        return source
    path = Path(source)
    if path.is_dir():
        path = path / "config.json"
    parsed = json.loads(path.read_text())
    if not isinstance(parsed, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return parsed


def _dataclass_arm(annotation: Any) -> type | None:
    """The dataclass inside `X`, `X | None` or `Optional[X]`, if there is one."""
    if dataclasses.is_dataclass(annotation) and isinstance(annotation, type):
        return annotation
    if typing.get_origin(annotation) in (typing.Union, types.UnionType):
        for arm in typing.get_args(annotation):
            if dataclasses.is_dataclass(arm) and isinstance(arm, type):
                return arm
    return None


def hydrate(cls: type[T], data: dict[str, Any]) -> T:
    if not dataclasses.is_dataclass(cls):
        raise TypeError(f"{cls!r} is not a dataclass")
    hints = typing.get_type_hints(cls)
    values: dict[str, Any] = {}
    missing: list[str] = []
    for field in dataclasses.fields(cls):
        if field.name not in data:
            required = field.default is dataclasses.MISSING and field.default_factory is dataclasses.MISSING
            if required:
                missing.append(field.name)
            continue
        value = data[field.name]
        nested = _dataclass_arm(hints[field.name])
        if nested is not None and isinstance(value, dict):
            value = hydrate(nested, value)
        elif isinstance(value, list):
            value = tuple(tuple(v) if isinstance(v, list) else v for v in value)
        values[field.name] = value
    if missing:
        raise ConfigError(f"{cls.__name__}: config.json lacks the keys {missing}")
    return cls(**values)

"""One registry from an architecture's name to everything the engine needs of it.

A checkpoint names its architecture in config.json: `architectures[0]`
(e.g. "MuseGlimmerForConditionalGeneration") and `model_type` ("muse_glimmer"); both
are keys here. The reference keeps one such table keyed on `model_type`
(src/mlx_omnia/engine/task.py:174-229,415-420) and raises ValueError for a type it
does not know; so does this one.

An `Architecture` holds: the typed configuration class; `parse(config.json dict)`
returning that configuration; `model_spec(config)` returning the parts and schedule;
`tensor_name(file_name)` mapping a name in the file to the model's tensor name (None
for tensors the text engine ignores on purpose); and `random_tensors(config, seed)`
for the random-weights mode; `dropped_tensors(config)` names tensors a file may carry
that the configuration makes unused (a tied head's `lm_head.weight`, which the
reference drops too: src/mlx_omnia/engine/checkpoint.py:630-631).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from mlx_omnia_b200.parts.model import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    parse: Callable[[dict[str, Any]], Any]
    model_spec: Callable[[Any], ModelSpec]
    tensor_name: Callable[[str], str | None]
    random_tensors: Callable[[Any, int], dict[str, torch.Tensor]]
    stop_tokens: Callable[[Any], tuple[int, ...]] = lambda config: ()
    # Model tensor names a file may hold that this configuration does not use (dropped).
    dropped_tensors: Callable[[Any], tuple[str, ...]] = lambda config: ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(architecture: Architecture, *keys: str) -> None:
    for key in keys:
        if key in _ARCHITECTURES and _ARCHITECTURES[key] is not architecture:
            raise ValueError(f"architecture key {key!r} is already registered")
        _ARCHITECTURES[key] = architecture


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(config: dict[str, Any]) -> Architecture:
    """The architecture a config.json names; `architectures[0]` first, then `model_type`."""
    import mlx_omnia_b200.architectures  # noqa: F401  (registers the built-in family)

    names = list(config.get("architectures") or [])
    for key in [*names[:1], config.get("model_type")]:
        if key in _ARCHITECTURES:
            return _ARCHITECTURES[key]
    raise ValueError(f"unsupported architecture: architectures={names!r}, model_type={config.get('model_type')!r}; "
                     f"known: {known_architectures()}")

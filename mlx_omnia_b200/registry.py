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
reference drops too: src/mlx_omnia/engine/checkpoint.py:630-631); `tokenizer(folder)`
returns the folder's tokenizer (anything with `encode` and `decode`) or None;
`generation_defaults(folder, config)` returns the ids that end a generation and the
sampling the checkpoint asks for (`text.GenerationDefaults`). The last two default to a
byte-level BPE read from tokenizer.json and to generation_config.json, which is where the
reference finds them for every family.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from pathlib import Path

import torch

from mlx_omnia_b200.parts.model import ModelSpec
from mlx_omnia_b200.text.defaults import GenerationDefaults, generation_defaults, read_tokenizer


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
    tokenizer: Callable[[Path], Any] = read_tokenizer
    # The longest context the checkpoint declares (None: it declares none).
    max_context: Callable[[Any], int | None] = lambda config: None
    generation_defaults: Callable[[Path, Any], GenerationDefaults] | None = None

    def defaults(self, folder: Path, config: Any) -> GenerationDefaults:
        """What the checkpoint in `folder` says about stopping and sampling."""
        if self.generation_defaults is not None:
            return self.generation_defaults(folder, config)
        return generation_defaults(folder, self.stop_tokens(config))


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

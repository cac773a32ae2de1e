"""What a checkpoint's side files say about generation: which ids end it, and how the model
wants to be sampled when the caller does not say.

* stop ids: config.json's `eos_token_id`, plus `generation_config.json`'s, plus the id of the
  token that `tokenizer_config.json` names as `eos_token`; in that order, without repeats. The
  set is only ever widened (src/mlx_omnia/engine/checkpoint.py:214-247).
* sampling defaults: `generation_config.json`'s temperature, top_p, top_k, min_p and
  repetition_penalty where they are positive numbers; `do_sample: false` means greedy
  whatever else the file holds (src/mlx_omnia/engine/checkpoint.py:131-152).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path


@dataclass(frozen=True)
class SamplingDefaults:
    """Each knob is None where the checkpoint does not declare it (which is not the same as
    declaring it neutral); temperature 0 means greedy."""

    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None
    repetition_penalty: float | None = None


@dataclass(frozen=True)
class GenerationDefaults:
    stop: tuple[int, ...] = ()
    sampling: SamplingDefaults = field(default_factory=SamplingDefaults)


def _json(path: Path) -> dict:
    try:
        loaded = json.loads(path.read_text(encoding="utf-8"))
    except (OSError, ValueError):
        return {}
    return loaded if isinstance(loaded, dict) else {}


def _meaningful(value) -> float | None:
    """A knob counts only as a positive number: 0 is how such files spell "off"."""
    if isinstance(value, bool) or not isinstance(value, (int, float)) or value <= 0:
        return None
    return float(value)


def _named_eos(folder: Path) -> int | None:
    name = _json(folder / "tokenizer_config.json").get("eos_token")
    if isinstance(name, dict):  # written either as the string or as the whole added-token object
        name = name.get("content")
    if not isinstance(name, str):
        return None
    for entry in _json(folder / "tokenizer.json").get("added_tokens", []):
        if isinstance(entry, dict) and entry.get("content") == name and isinstance(entry.get("id"), int):
            return entry["id"]
    return None


def generation_defaults(folder: str | Path, declared_stop=()) -> GenerationDefaults:
    folder = Path(folder)
    declared = _json(folder / "generation_config.json")
    stop = [int(t) for t in declared_stop]
    more = declared.get("eos_token_id")
    stop += [t for t in (more if isinstance(more, list) else [more]) if isinstance(t, int) and not isinstance(t, bool)]
    named = _named_eos(folder)
    if named is not None:
        stop.append(named)
    if declared.get("do_sample") is False:
        sampling = SamplingDefaults(temperature=0.0)
    else:
        top_k = _meaningful(declared.get("top_k"))
        sampling = SamplingDefaults(_meaningful(declared.get("temperature")), _meaningful(declared.get("top_p")),
                                    None if top_k is None else int(top_k), _meaningful(declared.get("min_p")),
                                    _meaningful(declared.get("repetition_penalty")))
    return GenerationDefaults(tuple(dict.fromkeys(stop)), sampling)


def read_tokenizer(folder: str | Path):
    """The folder's tokenizer (tokenizer.json, a byte-level BPE), or None when it has none."""
    from mlx_omnia_b200.text.bpe import ByteLevelBPE

    path = Path(folder) / "tokenizer.json"
    return ByteLevelBPE.from_file(path) if path.is_file() else None

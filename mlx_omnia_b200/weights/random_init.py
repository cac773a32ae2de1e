"""The random-weights mode: write a model folder from a configuration and a seed.

The folder holds `config.json` (the configuration as given, with the architecture's
name) and `model.safetensors` with the architecture's own tensor names, so it loads
like any checkpoint. The reference has no such mode; its tests randomise a built tree
(tests/test_batching_families.py:1132-1155 of the reference).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import torch
from safetensors.torch import save_file

from mlx_omnia_b200.registry import resolve_architecture


def write_random_model(folder: str | Path, config: dict[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> Path:
    """Create `folder` with config.json and model.safetensors; tensors are drawn in
    float32 from `seed` and stored as `dtype` (norm vectors always as float32)."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    architecture = resolve_architecture(config)
    parsed = architecture.parse(config)
    tensors = architecture.random_tensors(parsed, seed)
    stored = {name: (t if t.dim() < 2 else t.to(dtype)).contiguous() for name, t in tensors.items()}
    save_file(stored, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder

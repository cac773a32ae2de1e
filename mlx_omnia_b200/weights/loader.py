"""Strict loading of safetensors by tensor name.

The files' names are mapped to the model's by the architecture; then the set of names
must equal the set the model's parts declare, with equal shapes. Everything wrong is
reported in one `WeightError`: missing tensors, unexpected tensors and wrong shapes,
each listed. The reference loads strictly too
(src/mlx_omnia/engine/checkpoint.py:570-589) and merges every `model*.safetensors` of
the folder (src/mlx_omnia/engine/checkpoint.py:429-437).

Dtypes: `matrix` tensors are kept in the engine's dtype (bfloat16 files stay bfloat16;
on the 32-bit path they are widened, which is exact); `vector` tensors (norm weights)
are always float32, so a value stored in 32-bit is never rounded; integer tables
become int32.
"""

from __future__ import annotations

from pathlib import Path

import torch
from safetensors import safe_open

from mlx_omnia_b200.parts.base import Runtime, TensorSpec
from mlx_omnia_b200.registry import Architecture


class WeightError(ValueError):
    """The checkpoint's tensors do not match what the model declares."""

    def __init__(self, missing: list[str], unexpected: list[str], wrong: list[str]) -> None:
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def checkpoint_files(folder: Path) -> list[Path]:
    files = sorted(folder.glob("model*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no model*.safetensors in {folder}")
    return files


def _target_dtype(spec: TensorSpec, runtime: Runtime) -> torch.dtype:
    if spec.kind == "vector":
        return torch.float32
    if spec.kind == "table_i32":
        return torch.int32
    return runtime.dtype


def load_tensors(folder: str | Path, architecture: Architecture, config, expected: dict[str, TensorSpec],
                 runtime: Runtime) -> dict[str, torch.Tensor]:
    """Read, check and place on the device every tensor in `expected`."""
    folder = Path(folder)
    dropped = set(architecture.dropped_tensors(config))
    found: dict[str, tuple[Path, str]] = {}
    unexpected: list[str] = []
    for path in checkpoint_files(folder):
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for file_name in handle.keys():
                name = architecture.tensor_name(file_name)
                if name is None or name in dropped:
                    continue
                if name in expected:
                    found[name] = (path, file_name)
                else:
                    unexpected.append(file_name)
    missing = sorted(set(expected) - set(found))
    wrong: list[str] = []
    tensors: dict[str, torch.Tensor] = {}
    by_file: dict[Path, list[tuple[str, str]]] = {}
    for name, (path, file_name) in found.items():
        by_file.setdefault(path, []).append((name, file_name))
    for path, names in by_file.items():
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for name, file_name in names:
                spec = expected[name]
                shape = tuple(handle.get_slice(file_name).get_shape())
                if shape != tuple(spec.shape):
                    wrong.append(f"{file_name}: file has {list(shape)}, model wants {list(spec.shape)}")
                    continue
                if missing or unexpected or wrong:
                    continue  # an error is coming; do not spend time reading
                tensor = handle.get_tensor(file_name)
                floating = tensor.dtype.is_floating_point
                if (spec.kind == "table_i32") == floating:
                    wrong.append(f"{file_name}: file has dtype {tensor.dtype}, model wants a {spec.kind}")
                    continue
                tensors[name] = tensor.to(_target_dtype(spec, runtime)).to(runtime.device)
    if missing or unexpected or wrong:
        raise WeightError(missing, sorted(unexpected), sorted(wrong))
    return tensors

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


class FolderSource:
    """The tensors of every `model*.safetensors` of a folder, read one at a time."""

    def __init__(self, folder: str | Path) -> None:
        self.where: dict[str, Path] = {}
        for path in checkpoint_files(Path(folder)):
            with safe_open(str(path), framework="pt", device="cpu") as handle:
                for name in handle.keys():
                    self.where[name] = path
        self._open: tuple[Path, object] | None = None

    def names(self) -> list[str]:
        return list(self.where)

    def _handle(self, name: str):
        path = self.where[name]
        if self._open is None or self._open[0] != path:
            self._open = (path, safe_open(str(path), framework="pt", device="cpu"))
        return self._open[1]

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self._handle(name).get_slice(name).get_shape())

    def tensor(self, name: str) -> torch.Tensor:
        return self._handle(name).get_tensor(name)


class DictSource:
    """Tensors already in memory, under the checkpoint's names."""

    def __init__(self, tensors: dict[str, torch.Tensor]) -> None:
        self.tensors = tensors

    def names(self) -> list[str]:
        return list(self.tensors)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.tensors[name].shape)

    def tensor(self, name: str) -> torch.Tensor:
        return self.tensors[name]


def load_tensors(source, architecture: Architecture, config, expected: dict[str, TensorSpec],
                 runtime: Runtime) -> dict[str, torch.Tensor]:
    """Check and place on the device every tensor in `expected`. `source` is a model folder
    (a path), a dict of tensors under the checkpoint's names, or anything with `names()`,
    `shape(name)` and `tensor(name)`; whichever it is, the same check runs."""
    if isinstance(source, (str, Path)):
        source = FolderSource(source)
    elif isinstance(source, dict):
        source = DictSource(source)
    dropped = set(architecture.dropped_tensors(config))
    found: dict[str, str] = {}
    unexpected: list[str] = []
    for file_name in source.names():
        name = architecture.tensor_name(file_name)
        if name is None or name in dropped:
            continue
        if name in expected:
            found[name] = file_name
        else:
            unexpected.append(file_name)
    missing = sorted(set(expected) - set(found))
    wrong: list[str] = []
    for name, file_name in found.items():
        shape = source.shape(file_name)
        if shape != tuple(expected[name].shape):
            wrong.append(f"{file_name}: file has {list(shape)}, model wants {list(expected[name].shape)}")
    tensors: dict[str, torch.Tensor] = {}
    if not (missing or unexpected or wrong):  # with an error coming, no time is spent reading
        for name, file_name in sorted(found.items(), key=lambda item: item[1]):
            spec, tensor = expected[name], source.tensor(file_name)
            if (spec.kind == "table_i32") == tensor.dtype.is_floating_point:
                wrong.append(f"{file_name}: file has dtype {tensor.dtype}, model wants a {spec.kind}")
                continue
            tensors[name] = tensor.to(_target_dtype(spec, runtime)).to(runtime.device)
    if missing or unexpected or wrong:
        raise WeightError(missing, sorted(unexpected), sorted(wrong))
    return tensors

"""Putting an engine together: configuration -> model -> weights -> cache -> step runner."""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from mlx_omnia_b200.cache.manager import CacheManager
from mlx_omnia_b200.config.hydrate import read_json
from mlx_omnia_b200.engine.step import StepRunner
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import Runtime, TensorSpec
from mlx_omnia_b200.parts.model import DecoderModel
from mlx_omnia_b200.registry import Architecture, resolve_architecture
from mlx_omnia_b200.weights.loader import WeightError, load_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


@dataclass
class EngineArgs:
    """Sizes of the engine that are not the model's.

    dtype:          "bfloat16" (what serving uses) or "float32" (everything in true 32-bit)
    page_size:      tokens per cache page
    cache_tokens:   how many tokens the page pool of each group can hold
    max_requests:   live requests (state slots) at most
    device:         the CUDA device
    cuda_graphs:    replay single-token steps from captured CUDA graphs
    """

    dtype: str = "bfloat16"
    page_size: int = 16
    cache_tokens: int = 8192
    max_requests: int = 64
    device: str = "cuda:0"
    cuda_graphs: bool = True


def _runtime(args: EngineArgs) -> Runtime:
    if args.dtype not in DTYPES:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {args.dtype!r}")
    device = torch.device(args.device)
    if device.type == "cuda":
        ops.require_cuda()
        # The 32-bit path must not fall into a reduced-precision matrix mode.
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.set_float32_matmul_precision("highest")
    return Runtime(DTYPES[args.dtype], device)


def place_tensors(tensors: dict[str, torch.Tensor], expected: dict[str, TensorSpec], runtime: Runtime,
                  architecture: Architecture, config) -> dict[str, torch.Tensor]:
    """In-memory counterpart of `load_tensors`: same strictness, no files."""
    dropped = set(architecture.dropped_tensors(config))
    named = {}
    unexpected = []
    for file_name, tensor in tensors.items():
        name = architecture.tensor_name(file_name)
        if name is None or name in dropped:
            continue
        if name in expected:
            named[name] = tensor
        else:
            unexpected.append(file_name)
    missing = sorted(set(expected) - set(named))
    wrong = [f"{n}: given {list(t.shape)}, model wants {list(expected[n].shape)}"
             for n, t in named.items() if tuple(t.shape) != tuple(expected[n].shape)]
    if missing or unexpected or wrong:
        raise WeightError(missing, sorted(unexpected), sorted(wrong))
    out = {}
    for name, tensor in named.items():
        kind = expected[name].kind
        dtype = torch.float32 if kind == "vector" else torch.int32 if kind == "table_i32" else runtime.dtype
        out[name] = tensor.to(dtype).to(runtime.device)
    return out


class Engine:
    """A loaded model with its cache and step function."""

    def __init__(self, architecture: Architecture, config: Any, model: DecoderModel, runtime: Runtime,
                 args: EngineArgs) -> None:
        self.architecture, self.config, self.model, self.runtime, self.args = architecture, config, model, runtime, args
        pages = -(-args.cache_tokens // args.page_size)
        self.cache = CacheManager(model.cache_needs(), page_size=args.page_size, pages_per_group=pages,
                                  max_requests=args.max_requests, dtype=runtime.dtype, device=runtime.device)
        self.runner = StepRunner(model, self.cache, runtime, cuda_graphs=args.cuda_graphs)

    @property
    def vocab_size(self) -> int:
        return self.model.head.vocab

    @classmethod
    def from_folder(cls, folder: str | Path, args: EngineArgs | None = None) -> "Engine":
        """Load `folder` (config.json + model*.safetensors); the model class is the one
        config.json names."""
        args = args or EngineArgs()
        raw = read_json(Path(folder))
        architecture = resolve_architecture(raw)
        config = architecture.parse(raw)
        runtime = _runtime(args)
        model = DecoderModel(architecture.model_spec(config))
        model.load(load_tensors(folder, architecture, config, model.tensors(), runtime), runtime)
        return cls(architecture, config, model, runtime, args)

    @classmethod
    def from_tensors(cls, raw_config: dict[str, Any], tensors: dict[str, torch.Tensor],
                     args: EngineArgs | None = None) -> "Engine":
        """Build from a config.json object and tensors under the checkpoint's names."""
        args = args or EngineArgs()
        architecture = resolve_architecture(raw_config)
        config = architecture.parse(raw_config)
        runtime = _runtime(args)
        model = DecoderModel(architecture.model_spec(config))
        model.load(place_tensors(tensors, model.tensors(), runtime, architecture, config), runtime)
        return cls(architecture, config, model, runtime, args)

    @classmethod
    def from_random(cls, raw_config: dict[str, Any], seed: int, args: EngineArgs | None = None,
                    stored: torch.dtype = torch.bfloat16) -> "Engine":
        """Random weights as the random-weights mode would write them (matrices rounded to
        `stored`, vectors float32), without going through a folder."""
        architecture = resolve_architecture(raw_config)
        tensors = architecture.random_tensors(architecture.parse(raw_config), seed)
        tensors = {k: (t if t.dim() < 2 else t.to(stored)) for k, t in tensors.items()}
        return cls.from_tensors(raw_config, tensors, args)

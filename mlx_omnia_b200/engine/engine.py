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
from mlx_omnia_b200.parts.base import Runtime
from mlx_omnia_b200.parts.model import DecoderModel, ModelSpec
from mlx_omnia_b200.registry import Architecture, resolve_architecture
from mlx_omnia_b200.weights.loader import load_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


@dataclass
class EngineArgs:
    """Sizes of the engine that are not the model's.

    dtype:          "bfloat16" (what serving uses) or "float32" (everything in true 32-bit)
    page_size:      tokens per cache page
    cache_tokens:   how many tokens the page pool of each group can hold; None sizes the pool
                    from the device memory that is free once the weights are placed
                    (`memory_fraction` of it, divided by the cache bytes a token costs)
    max_requests:   live requests (state slots) at most
    device:         the CUDA device
    cuda_graphs:    replay single-token steps from captured CUDA graphs
    memory_fraction: the share of free device memory that a pool sized by the engine takes
    """

    dtype: str = "bfloat16"
    page_size: int = 16
    cache_tokens: int | None = 8192
    max_requests: int = 64
    device: str = "cuda:0"
    cuda_graphs: bool = True
    memory_fraction: float = 0.8


def pool_tokens(free_bytes: int, bytes_per_token: int, page_size: int, fraction: float) -> int:
    """Tokens a pool may hold when it is given `fraction` of `free_bytes`: whole pages, at
    least one. The reference counts its cache's bytes per layer for admission
    (src/mlx_omnia/engine/core/cache/layer.py:123-127); a paged pool is sized once instead."""
    if bytes_per_token <= 0:
        return page_size
    pages = int(free_bytes * fraction) // (bytes_per_token * page_size)
    return max(pages, 1) * page_size


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


class Engine:
    """A loaded model with its cache and step function."""

    def __init__(self, architecture: Architecture, config: Any, model: DecoderModel, runtime: Runtime,
                 args: EngineArgs) -> None:
        self.architecture, self.config, self.model, self.runtime, self.args = architecture, config, model, runtime, args
        needs = model.cache_needs()
        tokens = args.cache_tokens
        if tokens is None:
            if runtime.device.type != "cuda":
                raise ValueError("cache_tokens must be given when the engine does not run on a CUDA device")
            element = torch.empty(0, dtype=runtime.dtype).element_size()
            free, _ = torch.cuda.mem_get_info(runtime.device)
            tokens = pool_tokens(free, CacheManager.bytes_per_token(needs, element), args.page_size,
                                 args.memory_fraction)
            longest = architecture.max_context(config)
            if longest:  # no more than every request at the longest context the checkpoint declares
                tokens = min(tokens, -(-longest // args.page_size) * args.page_size * args.max_requests)
        self.cache_tokens = tokens
        pages = -(-tokens // args.page_size)
        self.cache = CacheManager(needs, page_size=args.page_size, pages_per_group=pages,
                                  max_requests=args.max_requests, dtype=runtime.dtype, device=runtime.device)
        self.runner = StepRunner(model, self.cache, runtime, cuda_graphs=args.cuda_graphs)

    @property
    def vocab_size(self) -> int:
        return self.model.head.vocab

    @classmethod
    def build(cls, raw_config: dict[str, Any], source, args: EngineArgs | None = None,
              spec: ModelSpec | None = None) -> "Engine":
        """The one way an engine is put together. `source` is whatever `load_tensors` reads
        (a model folder, or a dict of tensors under the checkpoint's names); the model class
        is the one `raw_config` names. `spec` replaces the architecture's own list of parts
        (for a model put together by hand from registered parts)."""
        args = args or EngineArgs()
        architecture = resolve_architecture(raw_config)
        config = architecture.parse(raw_config)
        runtime = _runtime(args)
        model = DecoderModel(spec if spec is not None else architecture.model_spec(config))
        model.load(load_tensors(source, architecture, config, model.tensors(), runtime), runtime)
        return cls(architecture, config, model, runtime, args)

    @classmethod
    def from_folder(cls, folder: str | Path, args: EngineArgs | None = None) -> "Engine":
        """Load `folder` (config.json + model*.safetensors)."""
        return cls.build(read_json(Path(folder)), Path(folder), args)

    @classmethod
    def from_tensors(cls, raw_config: dict[str, Any], tensors: dict[str, torch.Tensor],
                     args: EngineArgs | None = None, spec: ModelSpec | None = None) -> "Engine":
        """Build from a config.json object and tensors under the checkpoint's names."""
        return cls.build(raw_config, tensors, args, spec)

    @classmethod
    def from_random(cls, raw_config: dict[str, Any], seed: int, args: EngineArgs | None = None,
                    stored: torch.dtype = torch.bfloat16) -> "Engine":
        """Random weights as the random-weights mode would write them (matrices rounded to
        `stored`, vectors float32), without going through a folder."""
        architecture = resolve_architecture(raw_config)
        tensors = architecture.random_tensors(architecture.parse(raw_config), seed)
        tensors = {k: (t if t.dim() < 2 else t.to(stored)) for k, t in tensors.items()}
        return cls.from_tensors(raw_config, tensors, args)

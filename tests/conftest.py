"""Shared fixtures. Tests marked `gpu` need a CUDA device; everything else runs on the CPU."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for path in (ROOT, ROOT / "tests"):
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a) and the compiled kernels")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def cpu_ops(monkeypatch):
    """Swap the CUDA kernels for their plain PyTorch references, so the engine's glue
    (cache manager, step function, scheduler) can be exercised without a GPU."""
    import kernel_refs
    from mlx_omnia_b200.kernels import ops

    for name in ("embed_rmsnorm", "rmsnorm", "add_rmsnorm", "qk_norm_rope_store", "paged_attention", "swiglu",
                 "softcap", "gather_rows", "linear", "linear_swiglu", "linear_softcap", "sample",
                 "argmax"):
        monkeypatch.setattr(ops, name, getattr(kernel_refs, name))
    monkeypatch.setattr(ops, "raise_on_error", lambda device: None)
    return ops

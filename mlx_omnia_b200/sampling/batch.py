"""One call of the sampling kernel for the rows of a step."""

from __future__ import annotations

import numpy as np
import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.sampling.options import SamplingParams


def sample_rows(logits: torch.Tensor, params: list[SamplingParams], seeds: list[int], draws: list[int],
                histories: list[list[int]]) -> torch.Tensor:
    """Choose one token per row of float32 `logits` [rows, vocab]. `seeds[i]` and
    `draws[i]` (how many tokens row i's request has drawn so far) fix the random stream;
    `histories[i]` are the request's latest tokens for the repetition penalty.
    -> int32 [rows] on the device."""
    device = logits.device

    def dev(values, dtype):
        return torch.from_numpy(np.asarray(values, dtype=dtype)).to(device, non_blocking=True)

    if all(p.greedy and p.repetition_penalty == 1.0 for p in params):
        return ops.argmax(logits)
    penalty = history = None
    if any(p.repetition_penalty != 1.0 for p in params):
        width = max(p.penalty_context for p in params)
        table = np.full((len(params), width), -1, dtype=np.int32)
        for i, (p, h) in enumerate(zip(params, histories)):
            recent = h[-p.penalty_context:] if p.repetition_penalty != 1.0 else []
            table[i, : len(recent)] = recent
        history = dev(table, np.int32)
        penalty = dev([p.repetition_penalty for p in params], np.float32)
    return ops.sample(logits, dev([p.temperature for p in params], np.float32), dev([p.top_k for p in params], np.int32),
                      dev([p.top_p for p in params], np.float32), dev([p.min_p for p in params], np.float32),
                      dev([s & 0x7FFFFFFFFFFFFFFF for s in seeds], np.int64), dev(draws, np.int64), penalty, history)

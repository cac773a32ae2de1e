"""Requests in one batch do not see one another: with the cache pages of one live request
overwritten, that request's logits move and every other request's stay bit for bit, in a
mixed step (a portion of one prompt beside decoded tokens of others) and in captured decode
steps. The reference checks the same of its batched rows
(tests/test_batching_families.py:1532-1555 of the reference)."""

from __future__ import annotations

import pytest
import torch

import tiny_configs
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry
from mlx_omnia_b200.engine.trace import poison_free_pages
from mlx_omnia_b200.kernels import ops

pytestmark = pytest.mark.gpu


def prepared(name, dtype, page, prompts):
    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
    engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=page, cache_tokens=1024, max_requests=4))
    requests = [engine.cache.open(f"r{i}") for i in range(len(prompts))]
    # r0 and r1 have read their prompts but for the last token; r2 has read half of its own.
    engine.runner.run([StepEntry(requests[0], prompts[0][:-3], []), StepEntry(requests[1], prompts[1][:-3], []),
                       StepEntry(requests[2], prompts[2][:40], [])])
    return engine, requests


def corrupt(engine, request, value):
    """Overwrite every page that `request` holds, in every group and layer."""
    for g, group in enumerate(engine.cache.groups):
        held = [p for p in request.tables[g] if p >= 0]
        group.pages[:, held] = value


@pytest.mark.parametrize("name,dtype,page", [("B", "float32", 8), ("B", "bfloat16", 8), ("C", "bfloat16", 16),
                                             ("C", "float32", 16)])
def test_a_corrupted_request_moves_alone(name, dtype, page):
    vocab = tiny_configs.config(name)["text_config"]["vocab_size"]
    prompts = [tiny_configs.prompt(n, vocab, 500 + n) for n in (90, 57, 101)]
    results = []
    for dirty in (False, True):
        engine, requests = prepared(name, dtype, page, prompts)
        if dirty:
            corrupt(engine, requests[0], 3.0)
        poison_free_pages(engine)
        rows = []
        # a mixed step: one decoded token each of r0 and r1 beside a portion of r2 ...
        rows.append(engine.runner.run([StepEntry(requests[0], prompts[0][-3:-2], [0]),
                                       StepEntry(requests[1], prompts[1][-3:-2], [0]),
                                       StepEntry(requests[2], prompts[2][40:], [0, 30, 60])]))
        # ... and two decode-only steps (captured graphs), the requests in another order
        for k in (-2, -1):
            poison_free_pages(engine)
            rows.append(engine.runner.run([StepEntry(requests[1], prompts[1][k:][:1], [0]),
                                           StepEntry(requests[2], prompts[2][k:][:1], [0]),
                                           StepEntry(requests[0], prompts[0][k:][:1], [0])]))
        assert engine.runner.graphs is not None and engine.runner.graphs.replays == 2
        ops.raise_on_error(engine.runtime.device)
        results.append(rows)
    clean, dirty = results
    assert not torch.isnan(torch.cat(clean)).any() and not torch.isnan(torch.cat(dirty)).any()
    # mixed step: row 0 is r0, row 1 is r1, rows 2-4 are r2
    assert not torch.equal(clean[0][0], dirty[0][0])
    assert torch.equal(clean[0][1:], dirty[0][1:])
    # decode steps: rows are r1, r2, r0
    for step in (1, 2):
        assert torch.equal(clean[step][:2], dirty[step][:2])
        assert not torch.equal(clean[step][2], dirty[step][2])

"""The replay driver and the page pool's tightness, on the CPU: the same trace the GPU
test sends through bin/trace_run is replayed in-process with the reference kernels."""

from __future__ import annotations

import io
import json

import numpy as np
import pytest
import torch

import plain_impl
import tiny_configs
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.trace import replay
from test_replay_gpu import LENGTHS, build_trace


@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_in_process(cpu_ops, tmp_path, name):
    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
    vocab = raw["text_config"]["vocab_size"]
    prompts = {rid: tiny_configs.prompt(n, vocab, i) for i, (rid, n) in enumerate(LENGTHS.items())}
    trace = build_trace(prompts)
    engine = Engine.from_tensors(raw, weights, EngineArgs(dtype="float32", page_size=16, cache_tokens=trace.peak,
                                                          max_requests=4, device="cpu"))
    done = io.StringIO()
    lines = io.StringIO("".join(json.dumps(s) + "\n" for s in trace.steps))
    assert replay(engine, lines, tmp_path, done, npy=True) == len(trace.steps)
    assert done.getvalue().split()[-1] == str(len(trace.steps) - 1)
    expect = {rid: plain_impl.forward(raw, weights, ids) for rid, ids in prompts.items()}
    for index, rows in enumerate(trace.where):
        data = torch.from_numpy(np.fromfile(tmp_path / f"{index}.f32", dtype="<f4").reshape(len(rows), vocab))
        want = torch.stack([expect[rid.split("-")[1]][position] for rid, position in rows])
        assert plain_impl.relative_diff(data, want) < 2e-5, index
    # The same logits once more, gathered per request: every position of every replayed request.
    for request in {rid for rows in trace.where for rid, _ in rows}:
        whole = torch.from_numpy(np.load(tmp_path / f"logits_{request}.npy"))
        assert whole.shape == expect[request.split("-")[1]].shape
        assert plain_impl.relative_diff(whole, expect[request.split("-")[1]]) < 2e-5, request
    assert not engine.cache.requests
    engine.cache.check()

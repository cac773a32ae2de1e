"""The engine's glue on the CPU: with the kernels swapped for their plain references,
the step function and the cache manager must reproduce the plain implementation in
every way of cutting the work. (The kernels themselves are tested on the GPU.)"""

from __future__ import annotations

import pytest
import torch

import plain_impl
import tiny_configs
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry


def build(name: str, cache_tokens: int, page_size: int = 4) -> tuple[Engine, dict, dict]:
    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
    args = EngineArgs(dtype="float32", page_size=page_size, cache_tokens=cache_tokens, max_requests=4, device="cpu")
    return Engine.from_tensors(raw, weights, args), raw, weights


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt(cpu_ops, name):
    engine, raw, weights = build(name, 64)
    ids = tiny_configs.prompt(37, engine.vocab_size, 0)
    request = engine.cache.open("r")
    logits = engine.runner.run([StepEntry(request, ids, list(range(len(ids))))])
    expect = plain_impl.forward(raw, weights, ids)
    assert plain_impl.relative_diff(logits, expect) < 2e-5
    engine.cache.close("r")
    engine.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_and_decode(cpu_ops, name):
    engine, raw, weights = build(name, 64)
    ids = tiny_configs.prompt(45, engine.vocab_size, 1)
    expect = plain_impl.forward(raw, weights, ids)
    request = engine.cache.open("r")
    got, at = [], 0
    for size in (7, 2, 11, 3, 2, 5):
        got.append(engine.runner.run([StepEntry(request, ids[at: at + size], list(range(size)))]))
        at += size
    while at < len(ids):
        got.append(engine.runner.run([StepEntry(request, ids[at: at + 1], [0])]))
        at += 1
    assert plain_impl.relative_diff(torch.cat(got), expect) < 2e-5
    engine.cache.close("r")
    engine.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_with_page_reuse(cpu_ops, name):
    """Four requests, portions beside decoded tokens, in a pool so small that pages of
    finished requests (and, in B, of passed windows) are handed out again."""
    engine, raw, weights = build(name, 112, page_size=4)
    vocab = engine.vocab_size
    prompts = {k: tiny_configs.prompt(n, vocab, 10 + i) for i, (k, n) in enumerate(
        [("a", 40), ("b", 23), ("c", 31), ("d", 18), ("e", 36)])}
    expect = {k: plain_impl.forward(raw, weights, v) for k, v in prompts.items()}
    got = {k: [] for k in prompts}
    at = {k: 0 for k in prompts}
    plan = [
        {"a": 16, "b": 5},
        {"a": 9, "b": 2, "c": 13},
        {"a": 1, "b": 7, "c": 1, "d": 6},
        {"a": 1, "b": 9, "c": 17, "d": 12},     # b and d end here
        {"a": 13, "e": 20},                      # e takes pages that b and d gave back
        {"e": 16},
    ]
    for portion in plan:
        entries = []
        for k, n in portion.items():
            request = engine.cache.requests.get(k) or engine.cache.open(k)
            entries.append(StepEntry(request, prompts[k][at[k]: at[k] + n], list(range(n))))
            at[k] += n
        logits = engine.runner.run(entries)
        offset = 0
        for k, n in portion.items():
            got[k].append(logits[offset: offset + n])
            offset += n
        for k in portion:
            if at[k] == len(prompts[k]):
                engine.cache.close(k)
        engine.cache.check()
    for k in prompts:
        assert at[k] == len(prompts[k]) or k == "c"
        assert plain_impl.relative_diff(torch.cat(got[k]), expect[k][: at[k]]) < 2e-5, k


def test_window_pages_are_given_back(cpu_ops):
    engine, raw, _ = build("B", 256, page_size=4)
    request = engine.cache.open("r")
    ids = tiny_configs.prompt(64, engine.vocab_size, 3)
    engine.runner.run([StepEntry(request, ids, [63])])
    windowed = [g for g, group in enumerate(engine.cache.groups) if group.spec.window is not None]
    full = [g for g, group in enumerate(engine.cache.groups) if group.spec.window is None]
    assert windowed and full
    # 64 tokens, window 16: positions below 49 are dead, so pages 0..11 are free again.
    assert request.tables[windowed[0]][:12] == [-1] * 12 and min(request.tables[windowed[0]][12:]) >= 0
    assert min(request.tables[full[0]]) >= 0
    engine.cache.check()

"""Generation end to end on the CPU (kernels swapped for their references): greedy ids
equal the plain implementation's, batching does not change them, and a preempted
request comes back with the same tokens."""

from __future__ import annotations

import pytest

import plain_impl
import tiny_configs
from mlx_omnia_b200 import GenerationOptions, repetition_penalty, sampler, temperature, top_k
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.generate import Generator, LanguageModel


def engine_for(name, cache_tokens=256, page_size=4, max_requests=4):
    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
    args = EngineArgs(dtype="float32", page_size=page_size, cache_tokens=cache_tokens, max_requests=max_requests,
                      device="cpu")
    return Engine.from_tensors(raw, weights, args), raw, weights


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_batch_equals_plain(cpu_ops, name):
    engine, raw, weights = engine_for(name)
    prompts = [tiny_configs.prompt(n, engine.vocab_size, 30 + n) for n in (5, 9, 13)]
    got = Generator(engine, max_tokens_per_step=8).generate(prompts, GenerationOptions(max_tokens=8, stop=()))
    assert got == [plain_impl.greedy_generate(raw, weights, p, 8) for p in prompts]
    assert not engine.cache.requests
    engine.cache.check()


def test_stream_yields_segments_and_honours_stop(cpu_ops):
    engine, raw, weights = engine_for("B")
    model = LanguageModel(engine)
    prompt = tiny_configs.prompt(11, engine.vocab_size, 2)
    expect = plain_impl.greedy_generate(raw, weights, prompt, 6)
    segments = list(model.stream(" ".join(map(str, prompt)), GenerationOptions(max_tokens=6, stop=())))
    assert [s.token_id for s in segments] == expect and segments[0].text == f"{expect[0]} "
    cut = list(model.stream(prompt, GenerationOptions(max_tokens=6, stop=(expect[3],))))
    assert [s.token_id for s in cut] == expect[: expect.index(expect[3])]
    with pytest.raises(ValueError, match="token ids"):
        list(model.stream("hello there", GenerationOptions(max_tokens=2)))


def test_preemption_does_not_change_the_tokens(cpu_ops):
    options = GenerationOptions(max_tokens=14, sampler=sampler(temperature(0.9), top_k(20), seed=11), stop=(),
                                penalty=repetition_penalty(1.3))
    engine, _, _ = engine_for("A", cache_tokens=512)
    prompts = [tiny_configs.prompt(n, engine.vocab_size, 60 + n) for n in (17, 9, 12)]
    roomy = Generator(engine).generate(prompts, options)
    tight_engine, _, _ = engine_for("A", cache_tokens=56)
    generator = Generator(tight_engine)
    requests = [generator.add(p, options) for p in prompts]
    generator.run()
    assert sum(r.preemptions for r in requests) > 0
    assert [r.generated for r in requests] == roomy
    assert all(g.pool.free == g.pool.count for g in tight_engine.cache.groups)


def test_a_step_that_raises_fails_its_requests_and_frees_what_they_hold(cpu_ops, monkeypatch):
    """The step function fails in the middle of a generation: the requests of that step end as
    aborted, every page and slot is back in the pool, and the engine goes on with new requests
    (the reference aborts the round's members and carries on: src/mlx_omnia/server/runtime/rounds.py:88-93)."""
    engine, raw, weights = engine_for("A")
    generator = Generator(engine, max_tokens_per_step=8)
    prompts = [tiny_configs.prompt(n, engine.vocab_size, 80 + n) for n in (6, 11)]
    requests = [generator.add(p, GenerationOptions(max_tokens=6, stop=())) for p in prompts]
    for _ in range(3):
        generator.step()
    assert engine.cache.requests and all(r.status == "running" for r in requests)
    real = engine.model.forward

    def broken(*args, **kwargs):
        raise RuntimeError("the device fell over")

    monkeypatch.setattr(engine.model, "forward", broken)
    with pytest.raises(RuntimeError, match="fell over"):
        generator.run()
    assert all(r.status == "finished" and r.finish_reason == "abort" for r in requests)
    assert not engine.cache.requests and engine.cache.slots.free == engine.cache.slots.count
    assert all(g.pool.free == g.pool.count for g in engine.cache.groups)
    engine.cache.check()
    monkeypatch.setattr(engine.model, "forward", real)
    again = generator.generate([prompts[0]], GenerationOptions(max_tokens=4, stop=()))
    assert again == [plain_impl.greedy_generate(raw, weights, prompts[0], 4)]
    assert requests[0].meter.prompt_tokens == 6 and requests[0].meter.completion_tokens == len(requests[0].generated)

"""The parity tests can fail: each formula of the architecture is broken on purpose, one at a
time, in an engine that is otherwise the tested one, and the logits must then leave the
tolerance that the intact engine stays within. On the CPU with the kernels swapped for their
references (32-bit), and on the GPU through the replay suite in 32-bit and in bfloat16."""

from __future__ import annotations

import pytest
import torch

import mutations
import tiny_configs
from floors import Oracle
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry
from mlx_omnia_b200.registry import resolve_architecture


def mutated_engine(name: str, mutation, args: EngineArgs):
    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name)
    architecture = resolve_architecture(raw)
    spec = architecture.model_spec(architecture.parse(raw))
    tensors = weights
    if mutation is not None:
        spec, tensors = mutation(spec, weights)
        assert spec != architecture.model_spec(architecture.parse(raw)), "the mutation changed nothing"
    return Engine.from_tensors(raw, tensors, args, spec=spec), raw, weights


def applies(name: str, mutation) -> bool:
    layers = tiny_configs.config(name)["text_config"]
    if mutation is mutations.nope_rotated:
        return 0.0 in layers["layer_rope_theta"]
    if mutation in (mutations.window_plus_one, mutations.window_minus_one):
        return "sliding_attention" in layers["layer_types"]
    return True


@pytest.mark.parametrize("mutation", [None] + mutations.ALL, ids=lambda m: m.__name__ if m else "intact")
def test_each_fault_leaves_the_tolerance_on_the_cpu(cpu_ops, mutation):
    engine, raw, weights = mutated_engine("B", mutation, EngineArgs(dtype="float32", page_size=4, cache_tokens=128,
                                                                    max_requests=2, device="cpu"))
    ids = tiny_configs.prompt(70, engine.vocab_size, 0)
    oracle = Oracle(raw, weights, {"r": ids})
    request = engine.cache.open("r")
    logits = torch.cat([engine.runner.run([StepEntry(request, ids[:41], list(range(41)))]),
                        engine.runner.run([StepEntry(request, ids[41:63], list(range(22)))])] +
                       [engine.runner.run([StepEntry(request, ids[i: i + 1], [0])]) for i in range(63, 70)])
    diff = oracle.diff("r", logits)
    if mutation is None:
        assert diff < oracle.tolerance["float32"]
    else:
        assert diff > 10 * oracle.tolerance["float32"], f"{mutation.__name__} moved the logits by {diff:.3g} only"


GPU_CASES = [(name, dtype, m) for name, dtype in (("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16"))
             for m in mutations.ALL if applies(name, m)]


@pytest.mark.gpu
@pytest.mark.parametrize("name,dtype,mutation", GPU_CASES, ids=lambda v: getattr(v, "__name__", v))
def test_each_fault_fails_the_replay_suite(tmp_path, name, dtype, mutation):
    from test_replay_gpu import LENGTHS, build_trace
    from trace_tools import stacked

    raw = tiny_configs.config(name)
    vocab = raw["text_config"]["vocab_size"]
    prompts = {rid: tiny_configs.prompt(n, vocab, i) for i, (rid, n) in enumerate(LENGTHS.items())}
    trace = build_trace(prompts)
    engine, raw, weights = mutated_engine(name, mutation, EngineArgs(dtype=dtype, page_size=16, max_requests=4,
                                                                     cache_tokens=max(trace.peak, 64)))
    oracle = Oracle(raw, weights, prompts)
    got = trace.run_engine(engine, tmp_path / "out")
    worst = max(oracle.diff(request.split("-")[1], stacked(rows)[1]) for request, rows in got.items())
    assert worst > 2 * oracle.tolerance[dtype], f"{mutation.__name__} moved the logits by {worst:.3g} only"

"""Long prompts read in portions of random sizes, up to three requests live at a time, on the
configuration whose heads the tcgen05 prefill kernel takes: once a request holds more than
some 800 tokens the kernel's blocks are listed in parts that are merged (the test checks that the
list says so), portions mix with single decoded tokens, and one layer has a window. Free pages
hold NaN before every step. The logits are held against the plain implementation in float64
with the measured bfloat16 tolerance."""

from __future__ import annotations

import random

import pytest
import torch

import tiny_configs
from floors import Oracle
from trace_tools import Trace, stacked

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [0, 1])
def test_long_prompts_in_random_portions(tmp_path, seed):
    from mlx_omnia_b200.engine.engine import Engine, EngineArgs
    from mlx_omnia_b200.engine.trace import poison_free_pages
    from mlx_omnia_b200.kernels import ops

    raw, weights = tiny_configs.config("C"), tiny_configs.tensors("C")
    text = raw["text_config"]
    vocab = text["vocab_size"]
    lengths = {"a": 1400, "b": 950, "c": 330}
    prompts = {rid: tiny_configs.prompt(n, vocab, 900 + 7 * i + seed) for i, (rid, n) in enumerate(lengths.items())}
    rng = random.Random(seed)
    trace, at = Trace(), {rid: 0 for rid in prompts}
    live = ["a"]
    while live:
        portions = {}
        for rid in live:
            left = lengths[rid] - at[rid]
            n = min(left, rng.choice([1, 1, 2, 3, 17, 40, 64, 100, 129, 300]))
            portions[rid] = prompts[rid][at[rid]: at[rid] + n]
            at[rid] += n
        done = [rid for rid in live if at[rid] == lengths[rid]]
        trace.step(portions, end=done, want="last")
        live = [rid for rid in live if rid not in done]
        for rid in ("b", "c"):  # the others join when the first is well under way
            if rid not in live and at[rid] == 0 and at["a"] > (300 if rid == "b" else 700):
                live.append(rid)
    group = text["num_attention_heads"] // text["num_key_value_heads"]
    table = ops.prefill_work_table([100], [1300], 128 // group, 64, text["num_key_value_heads"], 0,
                                   ops.prefill_places(ops.sm_count()))
    assert ((table[:, 5] & 255) > 1).any()  # such a step's blocks are cut into parts
    engine = Engine.from_tensors(raw, weights, EngineArgs(dtype="bfloat16", page_size=16, cache_tokens=trace.peak + 64,
                                                          max_requests=4, cuda_graphs=True))
    got = trace.run_engine(engine, tmp_path / "out", before_step=lambda eng, record: poison_free_pages(eng))
    oracle = Oracle(raw, weights, prompts)
    for rid in prompts:
        positions, logits = stacked(got[rid])
        assert len(positions) >= 2 and not torch.isnan(logits).any()
        assert oracle.diff(rid, logits, positions) < oracle.tolerance["bfloat16"], rid
    ops.raise_on_error(engine.runtime.device)
    engine.cache.check()

"""Trace replay through `bin/trace_run` against the plain implementation: each request
whole; most of it in one step and the last 32 tokens one by one; in portions of
changing size, down to two tokens; and mixed, up to four live requests with portions
of some beside decoded tokens of others, in a pool so small that pages are used
again. In 32-bit and in bfloat16, for two tiny configurations that differ in
everything (and a third with 64-wide heads), at pages of 4, 8 and 16 tokens. Before every
step the pages that no request holds are filled with NaN, so a step that reads a page it
was not given shows it. Tolerances are measured floors (see floors.py)."""

from __future__ import annotations

import pytest
import torch

import tiny_configs
from floors import Oracle
from trace_tools import Trace, stacked, write_folder

pytestmark = pytest.mark.gpu

LENGTHS = {"a": 70, "b": 45, "c": 90, "d": 57, "e": 130, "f": 38}
PORTIONS = [13, 2, 7, 3, 2, 29, 5, 2, 17, 4]


def build_trace(prompts: dict[str, list[int]]) -> Trace:
    trace = Trace()
    # 1. whole
    for rid in "abcd":
        trace.step({f"whole-{rid}": prompts[rid]}, end=[f"whole-{rid}"])
    # 2. most in one step, the last 32 one by one
    for rid in "ae":
        ids = prompts[rid]
        trace.step({f"tail-{rid}": ids[:-32]})
        for i in range(len(ids) - 32, len(ids)):
            trace.step({f"tail-{rid}": ids[i: i + 1]}, end=[f"tail-{rid}"] if i == len(ids) - 1 else [])
    # 3. portions of changing size
    for rid in "ce":
        ids, at, k = prompts[rid], 0, 0
        while at < len(ids):
            n = min(PORTIONS[k % len(PORTIONS)], len(ids) - at)
            trace.step({f"cut-{rid}": ids[at: at + n]}, end=[f"cut-{rid}"] if at + n == len(ids) else [])
            at, k = at + n, k + 1
    # 4. mixed: four live, portions beside decoded tokens, finished requests' pages reused
    at = {rid: 0 for rid in prompts}

    def take(rid: str, n: int) -> list[int]:
        piece = prompts[rid][at[rid]: at[rid] + n]
        at[rid] += len(piece)
        return piece

    def ended(*rids: str) -> list[str]:
        return [f"mix-{r}" for r in rids if at[r] == len(prompts[r])]

    trace.step({"mix-a": take("a", 40), "mix-b": take("b", 20)})
    trace.step({"mix-a": take("a", 1), "mix-b": take("b", 23), "mix-c": take("c", 50)})
    trace.step({"mix-a": take("a", 1), "mix-b": take("b", 2), "mix-c": take("c", 1), "mix-d": take("d", 31)},
               end=ended("b"))
    trace.step({"mix-a": take("a", 28), "mix-c": take("c", 1), "mix-d": take("d", 26), "mix-f": take("f", 2)},
               end=ended("a", "d"))
    trace.step({"mix-c": take("c", 1), "mix-f": take("f", 30), "mix-e": take("e", 64)})
    trace.step({"mix-c": take("c", 37), "mix-f": take("f", 1), "mix-e": take("e", 3)}, end=ended("c"))
    for _ in range(5):
        trace.step({"mix-f": take("f", 1), "mix-e": take("e", 1)}, end=ended("f"))
    trace.step({"mix-e": take("e", 58)}, end=ended("e"))
    assert all(at[r] == len(prompts[r]) for r in prompts)
    return trace


# Tiny A and B at the page sizes their workloads name (4 and 8) and at 16; C, whose 64-wide
# heads take the tcgen05 prefill kernel at pages of 16 and the mma.sync kernel below that.
CASES = [("A", "float32", 4), ("B", "float32", 8), ("A", "bfloat16", 4), ("B", "bfloat16", 8),
         ("A", "float32", 16), ("B", "bfloat16", 16), ("C", "bfloat16", 16), ("C", "float32", 16), ("C", "bfloat16", 8)]


@pytest.mark.parametrize("name,dtype,page", CASES)
def test_replay_matches_plain(tmp_path, name, dtype, page):
    raw, weights = write_folder(tmp_path / "model", name)
    vocab = raw["text_config"]["vocab_size"]
    prompts = {rid: tiny_configs.prompt(n, vocab, i) for i, (rid, n) in enumerate(LENGTHS.items())}
    oracle = Oracle(raw, weights, prompts)
    trace = build_trace(prompts)
    got = trace.run(tmp_path / "model", dtype, tmp_path / "out",
                    extra=["--page-size", str(page), "--poison-free-pages"])
    worst = {}
    for request, per_position in got.items():
        mode, rid = request.split("-")
        positions, logits = stacked(per_position)
        assert positions == list(range(len(prompts[rid]))), request
        worst[request] = oracle.diff(rid, logits)
    assert len(worst) == 4 + 2 + 2 + 6
    bad = {k: v for k, v in worst.items() if not v < oracle.tolerance[dtype]}
    assert not bad, f"{bad} (tolerance {oracle.tolerance[dtype]:.3g}; all: {worst})"

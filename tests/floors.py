"""Tolerances that are measured, not guessed.

The plain implementation is run three ways on the very prompts a test uses: in float64 (the
exact result, for this purpose), in float32, and in float32 with every activation rounded to
bfloat16 the way a run of the reference in that precision rounds (`plain_impl.Rounding`). The
distance of the second from the first is the float32 noise floor of this model and these
prompts, the distance of the third the bfloat16 one.

* 32-bit tests allow three floors, as the reference's own parity tests do
  (tests/conftest.py:70-77 of the reference), and never less than two units in the last place.
  The engine's 32-bit path was measured at 1.0 to 1.2 floors on the tiny configurations.
* bfloat16 tests allow one floor of the faithful bfloat16 run. The engine keeps the residual
  stream in float32 and was measured at 0.5 to 0.65 of that floor, so a formula that is wrong
  by more than rounding does not hide under it (the mutation tests show that for each one).

Everything is compared with the float64 result, so a tolerance never absorbs the plain
float32 run's own error.
"""

from __future__ import annotations

import torch

import plain_impl

FP32_EPS = 2.0 ** -23
FLOAT32_FLOORS = 3.0
BFLOAT16_FLOORS = 1.0


class Oracle:
    """The exact logits of some prompts and the two tolerances that go with them."""

    def __init__(self, raw: dict, weights: dict, prompts: dict[str, list[int]], schedule=None, rows=None) -> None:
        """`rows(ids)`, when given, names the positions of a prompt whose logits are computed
        (all of them otherwise)."""
        run = lambda ids, **how: plain_impl.forward(raw, weights, ids, schedule=schedule,
                                                    rows=None if rows is None else rows(ids), **how)
        self.exact = {rid: run(ids, dtype=torch.float64) for rid, ids in prompts.items()}
        floor32 = max(plain_impl.relative_diff(run(ids), self.exact[rid]) for rid, ids in prompts.items())
        floor16 = max(plain_impl.relative_diff(run(ids, activations=torch.bfloat16), self.exact[rid])
                      for rid, ids in prompts.items())
        self.floors = {"float32": floor32, "bfloat16": floor16}
        self.tolerance = {"float32": max(FLOAT32_FLOORS * floor32, 2 * FP32_EPS),
                          "bfloat16": BFLOAT16_FLOORS * floor16}

    def diff(self, rid: str, logits: torch.Tensor, rows=slice(None)) -> float:
        return plain_impl.relative_diff(logits, self.exact[rid][rows])

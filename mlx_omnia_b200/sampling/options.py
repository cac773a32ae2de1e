"""Sampling options in the reference's vocabulary.

The reference composes a sampler from filters, `sampler(temperature(0.8), top_k(40),
top_p(0.9), seed=1)`, and passes it in `GenerationOptions`
(src/mlx_omnia/engine/generate.py:162-252, src/mlx_omnia/engine/language.py:91-140).
The same names exist here with the same meanings and the same argument checks; they
build a plain record of numbers, because the choice itself runs in one CUDA kernel in
the order the reference's server uses: temperature -> top_k -> top_p -> min_p
(src/mlx_omnia/server/api/responses/sampling.py:92-99). Filters given in another order
are refused rather than silently reordered.
"""

from __future__ import annotations

from collections.abc import Collection
from dataclasses import dataclass, replace


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 means greedy; top_k 0, top_p 1, min_p 0 and repetition_penalty 1
    switch the respective stage off. `seed` None draws a fresh seed per request."""

    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    penalty_context: int = 20
    seed: int | None = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


@dataclass(frozen=True)
class Filter:
    stage: str
    value: float


def temperature(value: float) -> Filter:
    """Divides the logits; must be positive (src/mlx_omnia/engine/generate.py:166-170)."""
    if value <= 0:
        raise ValueError(f"temperature must be positive: {value}")
    return Filter("temperature", float(value))


def top_k(k: int) -> Filter:
    """Keeps the k largest logits, a tie at the k-th value included whole
    (src/mlx_omnia/engine/generate.py:173-183)."""
    if k < 1:
        raise ValueError(f"top_k must be at least 1: {k}")
    return Filter("top_k", int(k))


def top_p(p: float) -> Filter:
    """Keeps the smallest set of tokens whose probabilities reach p
    (src/mlx_omnia/engine/generate.py:186-201)."""
    if not 0 < p <= 1:
        raise ValueError(f"top_p must be in (0, 1]: {p}")
    return Filter("top_p", float(p))


def min_p(p: float) -> Filter:
    """Keeps tokens at least p times as probable as the most probable one
    (src/mlx_omnia/engine/generate.py:204-214)."""
    if not 0 <= p < 1:
        raise ValueError(f"min_p must be in [0, 1): {p}")
    return Filter("min_p", float(p))


@dataclass(frozen=True)
class Penalty:
    value: float
    context: int = 20


def repetition_penalty(value: float, *, context: int = 20) -> Penalty:
    """Pushes down the ids seen in the last `context` positions, prompt included
    (src/mlx_omnia/engine/generate.py:217-233)."""
    if value <= 0:
        raise ValueError(f"repetition_penalty must be positive: {value}")
    if not 1 <= context <= 1024:
        raise ValueError(f"repetition_penalty context must be in [1, 1024]: {context}")
    return Penalty(float(value), int(context))


_ORDER = ("temperature", "top_k", "top_p", "min_p")


def sampler(*filters: Filter, seed: int | None = None) -> SamplingParams:
    """Draws from the distribution the filters shape (src/mlx_omnia/engine/generate.py:236-252).
    Without a temperature filter the logits are drawn from as they are (temperature 1)."""
    stages = [f.stage for f in filters]
    if len(set(stages)) != len(stages):
        raise ValueError(f"a filter is given twice: {stages}")
    if stages != [s for s in _ORDER if s in stages]:
        raise ValueError(f"filters run in the order {_ORDER}; got {stages}")
    values = {f.stage: f.value for f in filters}
    return SamplingParams(temperature=values.get("temperature", 1.0), top_k=int(values.get("top_k", 0)),
                          top_p=values.get("top_p", 1.0), min_p=values.get("min_p", 0.0), seed=seed)


greedy = SamplingParams()
"""The default sampler: the first largest logit (src/mlx_omnia/engine/generate.py:162-163)."""


@dataclass(frozen=True)
class GenerationOptions:
    """What one generation asks for (src/mlx_omnia/engine/language.py:91-140).

    max_tokens:     tokens to generate at most
    sampler:        `greedy` or what `sampler(...)` returns
    stop:           token ids that end the generation without being emitted; None means
                    the model's own (config.json's eos_token_id)
    penalty:        what `repetition_penalty(...)` returns, or None
    context_limit:  ceiling on prompt and generation together, or None
    meter:          an `engine.meter.Meter` that the generation fills (token counts, time to the
                    first token, decode rate), or None
    The reference's remaining fields (constraint, prefix, reasoning_budget, speculate) belong
    to its server, grammar and drafter, which this engine leaves out.
    """

    max_tokens: int
    sampler: SamplingParams = greedy
    stop: Collection[int] | None = None
    penalty: Penalty | None = None
    context_limit: int | None = None
    meter: object | None = None

    def params(self) -> SamplingParams:
        if self.penalty is None:
            return self.sampler
        return replace(self.sampler, repetition_penalty=self.penalty.value, penalty_context=self.penalty.context)

"""The scheduler: which requests run in the next step, and with how many tokens.

Every step is one flattened batch under a token budget. The plan is made in this
order: (1) every running request whose prompt is in the cache decodes one token;
(2) running requests still reading their prompt take the next portion of it, oldest
first; (3) waiting requests are admitted, oldest first, while there is a free slot,
budget and pages. A portion is cut to the budget and to the pages that are free, down
to one token; a request that cannot get even that waits for the next step.

When pages run out for a decoding request, the most recently admitted running request
is preempted: everything it holds is given back and it returns to the head of the
waiting queue; when it is admitted again its prompt and the tokens it has generated
are recomputed as one prompt (its sampling continues with the same draw indices, so
the tokens that follow are the same). The oldest request is never preempted in favour
of a newer one, so some request always makes progress. A request whose prompt alone
exceeds the pool is refused when it is added; `max_tokens` is cut to what the pool
can hold, as the reference cuts it to the context limit
(src/mlx_omnia/engine/language.py:407-409).

A request ends when it samples a stop token (which is not emitted, as in
src/mlx_omnia/engine/batching.py:653-655), when it has generated `max_tokens`
(src/mlx_omnia/engine/batching.py:667), or when it is aborted; its pages and slot go
back to the cache manager at once.

The reference's scheduling lives in its server: first come first served, one prompt
block of 2048 tokens per request per tick in a forward of its own, then one shared
decode forward (src/mlx_omnia/server/runtime/rounds.py:143-252,
src/mlx_omnia/engine/core/prefill.py:23). The token budget, mixed batches and
preemption are this engine's own design. The scheduler is host code only and is
tested without a GPU.
"""

from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field

from mlx_omnia_b200.cache.manager import CacheManager, RequestCache
from mlx_omnia_b200.sampling.options import SamplingParams


@dataclass(eq=False)
class Request:
    request_id: str
    prompt: list[int]
    max_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop: frozenset[int] = frozenset()
    generated: list[int] = field(default_factory=list)
    computed: int = 0  # tokens of prompt + generated that are in the cache
    cache: RequestCache | None = None
    status: str = "waiting"  # waiting | running | finished
    finish_reason: str | None = None  # stop | length | abort
    preemptions: int = 0
    order: int = 0
    meter: object | None = None  # an engine.meter.Meter, filled by the generation loop

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.generated

    def token_slice(self, start: int, count: int) -> list[int]:
        """tokens[start: start + count] without building the whole list."""
        split = len(self.prompt)
        if start >= split:
            return self.generated[start - split: start - split + count]
        if start + count <= split:
            return self.prompt[start: start + count]
        return self.prompt[start:] + self.generated[: start + count - split]

    @property
    def pending(self) -> int:
        """Tokens known but not yet in the cache."""
        return len(self.prompt) + len(self.generated) - self.computed


@dataclass
class PlannedEntry:
    request: Request
    start: int  # index into request.tokens of the first token this step runs
    count: int
    samples: bool  # the portion reaches the last known token: its logits choose the next one


@dataclass
class StepPlan:
    entries: list[PlannedEntry]
    preempted: list[Request]

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


@dataclass
class StepOutput:
    request: Request
    token: int | None  # None when the sampled token was a stop token
    finished: bool


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_tokens_per_step: int = 2048, max_running: int | None = None) -> None:
        if max_tokens_per_step < 1:
            raise ValueError("max_tokens_per_step must be at least 1")
        self.cache = cache
        self.max_tokens_per_step = max_tokens_per_step
        self.max_running = min(max_running or cache.slots.count, cache.slots.count)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._order = itertools.count()
        self.capacity = cache.capacity_tokens()

    # -- requests ------------------------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if request.max_tokens < 0:
            raise ValueError("max_tokens must not be negative")
        if len(request.prompt) >= self.capacity:
            raise ValueError(f"a prompt of {len(request.prompt)} tokens does not fit the cache pool of "
                             f"{self.capacity} tokens")
        request.max_tokens = min(request.max_tokens, self.capacity - len(request.prompt))
        request.order = next(self._order)
        request.status = "waiting"
        self.waiting.append(request)

    def abort(self, request_id: str) -> Request | None:
        for request in list(self.running):
            if request.request_id == request_id:
                self._finish(request, "abort")
                return request
        for request in list(self.waiting):
            if request.request_id == request_id:
                self.waiting.remove(request)
                request.status, request.finish_reason = "finished", "abort"
                return request
        return None

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # -- planning ------------------------------------------------------------------------
    def _preempt(self, request: Request) -> None:
        self.cache.close(request.request_id)
        request.cache, request.computed, request.status = None, 0, "waiting"
        request.preemptions += 1
        if request.meter is not None:
            request.meter.preemptions += 1
        self.running.remove(request)
        self.waiting.appendleft(request)

    def _finish(self, request: Request, reason: str) -> None:
        if request.cache is not None:
            self.cache.close(request.request_id)
            request.cache = None
        if request in self.running:
            self.running.remove(request)
        request.status, request.finish_reason = "finished", reason

    def _affordable(self, request: Request, wanted: int, reserved: list[int]) -> int:
        """The largest portion <= wanted whose pages are free in every group, `reserved`
        pages per group being already promised to earlier entries of this plan."""
        cache = self.cache
        held = request.cache.tokens if request.cache is not None else 0
        for g, group in enumerate(cache.groups):
            pages = cache.pages_for(g, held) + max(group.pool.free - reserved[g], 0)
            wanted = min(wanted, pages * cache.page_size * group.spec.stride - held)
        return max(0, wanted)

    def _reserve(self, request: Request, count: int, reserved: list[int]) -> None:
        held = request.cache.tokens if request.cache is not None else 0
        for g in range(len(reserved)):
            reserved[g] += self.cache.pages_for(g, held + count) - self.cache.pages_for(g, held)

    def plan(self) -> StepPlan:
        reserved = [0] * len(self.cache.groups)
        entries: list[PlannedEntry] = []
        preempted: list[Request] = []
        budget = self.max_tokens_per_step

        # (1) decoding requests, oldest first; preempt the newest while pages are short.
        decoding = sorted((r for r in self.running if r.pending == 1 and r.generated), key=lambda r: r.order)
        planned: set[int] = set()  # ids of requests that have an entry in this plan
        for request in decoding:
            if request.status != "running" or budget < 1:
                continue
            while self._affordable(request, 1, reserved) < 1:
                victim = max(self.running, key=lambda r: r.order)
                if id(victim) in planned:  # give back what the plan promised it
                    planned.discard(id(victim))
                    entries[:] = [e for e in entries if e.request is not victim]
                    reserved = [0] * len(self.cache.groups)
                    for e in entries:
                        self._reserve(e.request, e.count, reserved)
                    budget += 1
                self._preempt(victim)
                preempted.append(victim)
                if victim is request:
                    break
            if request.status != "running":
                continue
            entries.append(PlannedEntry(request, request.computed, 1, True))
            self._reserve(request, 1, reserved)
            planned.add(id(request))
            budget -= 1

        # (2) running requests that still have a prompt (or a recomputation) to read.
        for request in sorted((r for r in self.running if id(r) not in planned and r.pending > 0),
                              key=lambda r: r.order):
            if budget < 1:
                break
            count = self._affordable(request, min(request.pending, budget), reserved)
            if count < 1:
                continue
            entries.append(PlannedEntry(request, request.computed, count, count == request.pending))
            self._reserve(request, count, reserved)
            budget -= count

        # (3) admissions, strictly first come first served.
        while self.waiting and budget >= 1 and len(self.running) < self.max_running and self.cache.slots.free > 0:
            request = self.waiting[0]
            if any(request is p for p in preempted):
                break  # it lost its pages in this very plan
            count = self._affordable(request, min(request.pending, budget), reserved)
            if count < 1:
                break
            self.waiting.popleft()
            request.cache = self.cache.open(request.request_id)
            request.status = "running"
            self.running.append(request)
            entries.append(PlannedEntry(request, 0, count, count == request.pending))
            self._reserve(request, count, reserved)
            budget -= count
        return StepPlan(entries, preempted)

    # -- after the step --------------------------------------------------------------------
    def commit(self, plan: StepPlan, sampled: dict[str, int]) -> list[StepOutput]:
        """Record that the plan ran; `sampled` maps the ids of entries with `samples`
        to the token their logits chose."""
        outputs: list[StepOutput] = []
        for entry in plan.entries:
            request = entry.request
            request.computed += entry.count
            if not entry.samples:
                continue
            if len(request.generated) >= request.max_tokens:
                self._finish(request, "length")  # max_tokens == 0: the prompt was only read
                outputs.append(StepOutput(request, None, True))
                continue
            token = sampled[request.request_id]
            if token in request.stop:
                self._finish(request, "stop")
                outputs.append(StepOutput(request, None, True))
                continue
            request.generated.append(token)
            done = len(request.generated) >= request.max_tokens
            if done:
                self._finish(request, "length")
            outputs.append(StepOutput(request, token, done))
        return outputs

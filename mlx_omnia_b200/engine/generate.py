"""Generation: the loop that plans a step, runs it, samples and commits; and the
`load(path)` -> `model.stream(prompt, GenerationOptions(...))` entry point.

The reference's entry point is `load` (src/mlx_omnia/engine/task.py:486-547) returning a
facade whose `stream(input, options)` yields segments with `.text`
(src/mlx_omnia/engine/model.py:201-202, src/mlx_omnia/engine/language.py:483-552), over a
continuous-batching loop of `begin_batch`/`step_batch`
(src/mlx_omnia/engine/batching.py:223-341,408-437). Here the loop is the scheduler's
plan -> the step function -> the sampling kernel -> commit, with one device-to-host
read of the chosen tokens per step.
"""

from __future__ import annotations

import itertools
import secrets
from collections.abc import Iterator, Sequence
from dataclasses import dataclass
from pathlib import Path

import torch

from mlx_omnia_b200.engine.engine import DTYPES, Engine, EngineArgs
from mlx_omnia_b200.engine.meter import Meter
from mlx_omnia_b200.engine.scheduler import PlannedEntry, Request, Scheduler, StepOutput, StepPlan
from mlx_omnia_b200.engine.step import StepEntry
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.sampling.batch import sample_rows
from mlx_omnia_b200.sampling.options import GenerationOptions
from mlx_omnia_b200.text.bpe import Detokenizer
from mlx_omnia_b200.text.defaults import GenerationDefaults


@dataclass(frozen=True)
class Segment:
    """One piece of a streamed answer."""

    text: str
    token_id: int


@dataclass(frozen=True)
class Text:
    """A text prompt, as the reference's `Text` input (src/mlx_omnia/engine/language.py:60-79)."""

    prompt: str | Sequence[int]


class TokenIdTokenizer:
    """Stands in when a model folder has no tokenizer: text is token ids in decimal,
    separated by spaces, both ways."""

    def encode(self, text: str) -> list[int]:
        try:
            return [int(piece) for piece in text.replace(",", " ").split()]
        except ValueError:
            raise ValueError("this model folder has no tokenizer.json; give the prompt as token ids "
                             "(integers separated by spaces) or as a list of ints") from None

    def decode(self, ids: Sequence[int]) -> str:
        return "".join(f"{i} " for i in ids)


@dataclass
class _Launched:
    """A step that is running on the GPU: its plan, the requests it samples for and their
    chosen tokens (still on the device)."""

    plan: StepPlan
    sampling: list[Request]
    chosen: torch.Tensor | None
    host_tokens: torch.Tensor | None = None  # pinned copy of `chosen`, on its way since the launch
    copied: "torch.cuda.Event | None" = None  # recorded behind that copy


class Generator:
    """Continuous batching over one `Engine`."""

    def __init__(self, engine: Engine, *, max_tokens_per_step: int = 2048, max_running: int | None = None,
                 stop: Sequence[int] | None = None) -> None:
        """`stop`: the ids that end a generation whose options name none (None: config.json's own)."""
        self.engine = engine
        self.default_stop = tuple(stop) if stop is not None else \
            tuple(engine.architecture.stop_tokens(engine.config))
        self.scheduler = Scheduler(engine.cache, max_tokens_per_step=max_tokens_per_step, max_running=max_running)
        self._ids = itertools.count()
        self._seeds: dict[str, int] = {}
        self._in_flight: _Launched | None = None
        self._token_slots: list[torch.Tensor] = []  # pinned buffers the chosen tokens come back in, used in turn
        self._token_slot = 0
        self.pipelined = True  # launch the next decode step before reading this one's tokens

    def add(self, prompt: Sequence[int], options: GenerationOptions, request_id: str | None = None) -> Request:
        prompt = [int(t) for t in prompt]
        vocab = self.engine.vocab_size
        if any(not 0 <= t < vocab for t in prompt):
            raise ValueError(f"a prompt token lies outside the vocabulary of {vocab}")
        budget = options.max_tokens
        if options.context_limit is not None:
            budget = min(budget, options.context_limit - len(prompt))
        stop = options.stop if options.stop is not None else self.default_stop
        params = options.params()
        request = Request(request_id or f"req-{next(self._ids)}", prompt, max(budget, 0), params, frozenset(stop))
        request.meter = options.meter if options.meter is not None else Meter()
        request.meter.begin(len(prompt))
        self.scheduler.add(request)
        self._seeds[request.request_id] = params.seed if params.seed is not None else secrets.randbits(63)
        return request

    def abort(self, request_id: str) -> None:
        self.scheduler.abort(request_id)
        self._seeds.pop(request_id, None)

    def drain(self) -> list[StepOutput]:
        """Commit the step that is still in flight, if any."""
        launched, self._in_flight = self._in_flight, None
        return self._finalize(launched) if launched is not None else []

    # -- one step -----------------------------------------------------------------------------
    # A decode step's tokens are chosen on the GPU and can feed the next step from there, so the
    # host need not wait for them before it launches that step: while the GPU runs step n + 1 the
    # host reads step n's tokens (one step late, as the reference does: src/mlx_omnia/engine/
    # batching.py:598-604), commits them and prepares step n + 2. A request that turns out to
    # have ended on a stop token has then computed one token too many, which is dropped.

    def _launch(self, plan: StepPlan, device_tokens: torch.Tensor | None = None) -> "_Launched":
        entries = []
        for planned in plan.entries:
            tokens = [0] * planned.count if device_tokens is not None else \
                planned.request.token_slice(planned.start, planned.count)
            entries.append(StepEntry(planned.request.cache, tokens, [planned.count - 1] if planned.samples else []))
        try:
            logits = self.engine.runner.run(entries, copy=False, device_tokens=device_tokens)
        except Exception:
            for planned in plan.entries:  # a failed step fails its requests and frees what they hold
                self.scheduler._finish(planned.request, "abort")
            raise
        sampling = [p.request for p in plan.entries if p.samples]
        chosen = None
        if sampling:
            ahead = 1 if device_tokens is not None else 0  # draws already spent by the step not yet committed
            histories = [r.token_slice(max(0, len(r.prompt) + len(r.generated) - r.sampling.penalty_context),
                                       r.sampling.penalty_context) if r.sampling.repetition_penalty != 1.0 else []
                         for r in sampling]
            chosen = sample_rows(logits, [r.sampling for r in sampling], [self._seeds[r.request_id] for r in sampling],
                                 [len(r.generated) + ahead for r in sampling], histories)
        launched = _Launched(plan, sampling, chosen)
        if chosen is not None and chosen.is_cuda:
            # The tokens start for the host at once, behind this step only. Read with a blocking copy
            # when the host wants them, they would come behind everything launched since, the
            # next step included, and the host would prepare the step after that with the GPU idle.
            if not self._token_slots or self._token_slots[0].numel() < chosen.numel():
                self._token_slots = [torch.empty(max(64, chosen.numel()), dtype=torch.int32).pin_memory()
                                     for _ in range(4)]
            self._token_slot = (self._token_slot + 1) % len(self._token_slots)
            launched.host_tokens = self._token_slots[self._token_slot][: chosen.numel()]
            launched.host_tokens.copy_(chosen, non_blocking=True)
            launched.copied = torch.cuda.Event()
            launched.copied.record()
        return launched

    def _finalize(self, launched: "_Launched") -> list[StepOutput]:
        """Read the launched step's tokens (this waits for it) and commit them."""
        plan = launched.plan
        if launched.copied is not None:
            launched.copied.synchronize()
            tokens = launched.host_tokens.tolist()
        else:
            tokens = launched.chosen.tolist() if launched.chosen is not None else []
        sampled = dict(zip((r.request_id for r in launched.sampling), tokens))
        # A request that ended (a stop token, an abort) after this step was launched is left out.
        live = [e for e in plan.entries if e.request.status == "running"]
        outputs = self.scheduler.commit(StepPlan(live, plan.preempted), sampled)
        for output in outputs:
            if output.token is not None:
                output.request.meter.token()
            if output.finished:
                self._seeds.pop(output.request.request_id, None)
        return outputs

    def _next_decode_plan(self, launched: "_Launched") -> StepPlan | None:
        """The plan of the step after `launched`, if it can be made before `launched`'s tokens
        are known: every entry decodes, nobody waits for admission, no request needs its own
        last token on the host (repetition penalty), and the pages are there."""
        if self.engine.runner.graphs is None or self.scheduler.waiting or not self.pipelined:
            return None
        entries = launched.plan.entries
        if len(entries) != len(self.scheduler.running) or not all(e.count == 1 and e.samples for e in entries):
            return None
        following = []
        reserved = [0] * len(self.engine.cache.groups)
        for e in entries:
            r = e.request
            if r.status != "running" or r.sampling.repetition_penalty != 1.0:
                return None
            if len(r.generated) + 2 > r.max_tokens:  # it ends with the launched step's token: plan normally
                return None
            if self.scheduler._affordable(r, 1, reserved) < 1:  # (the launched step's page is already taken)
                return None
            self.scheduler._reserve(r, 1, reserved)
            following.append(PlannedEntry(r, e.start + 1, 1, True))
        return StepPlan(following, [])

    def step(self) -> list[StepOutput]:
        """Run one step (or, in steady decoding, launch the next one and) return what the oldest
        step in flight produced for each sampling request."""
        if self._in_flight is None:
            plan = self.scheduler.plan()
            if not plan.entries:
                return []
            self._in_flight = self._launch(plan)
        launched = self._in_flight
        following = self._next_decode_plan(launched)
        if following is not None:
            self._in_flight = self._launch(following, device_tokens=launched.chosen)
        else:
            self._in_flight = None
        return self._finalize(launched)

    def run(self) -> None:
        """Step until every request has finished."""
        while not self.scheduler.idle or self._in_flight is not None:
            if not self.step() and self._in_flight is None and not self.scheduler.running and self.scheduler.waiting:
                raise RuntimeError("the scheduler can admit nothing: the cache pool is too small")

    def generate(self, prompts: Sequence[Sequence[int]], options: GenerationOptions) -> list[list[int]]:
        """Generate for all prompts together; returns the generated ids per prompt."""
        requests = [self.add(p, options) for p in prompts]
        self.run()
        ops.raise_on_error(self.engine.runtime.device)
        return [r.generated for r in requests]


class LanguageModel:
    """What `load` returns: a model that streams text (or token ids)."""

    def __init__(self, engine: Engine, tokenizer=None, defaults: GenerationDefaults | None = None,
                 **generator_args) -> None:
        self.engine = engine
        self.tokenizer = tokenizer or TokenIdTokenizer()
        self.defaults = defaults or GenerationDefaults(tuple(engine.architecture.stop_tokens(engine.config)))
        self.generator = Generator(engine, stop=self.defaults.stop, **generator_args)

    def _ids(self, prompt) -> list[int]:
        if isinstance(prompt, Text):
            prompt = prompt.prompt
        return list(self.tokenizer.encode(prompt)) if isinstance(prompt, str) else [int(t) for t in prompt]

    def stream(self, input, options: GenerationOptions) -> Iterator[Segment]:
        """Generate for one prompt, yielding each token as it is chosen. A segment's text is
        whole characters: bytes that do not yet end one wait for the token that completes them."""
        request = self.generator.add(self._ids(input), options)
        pieces = Detokenizer(self.tokenizer)
        try:
            while request.status != "finished":
                for output in self.generator.step():
                    if output.request is request and output.token is not None:
                        yield Segment(pieces.feed(output.token), output.token)
            rest = pieces.flush()
            if rest:
                yield Segment(rest, -1)
        finally:
            if request.status != "finished":
                self.generator.abort(request.request_id)

    def generate(self, inputs: Sequence, options: GenerationOptions) -> list[list[int]]:
        """Generate for several prompts in one continuous batch; ids per prompt."""
        return self.generator.generate([self._ids(p) for p in inputs], options)


def load(model: str | Path, *, dtype=None, quantize=None, page_size: int = 16, cache_tokens: int | None = None,
         max_requests: int = 64, max_tokens_per_step: int = 2048, device: str = "cuda:0") -> LanguageModel:
    """Load a model folder (config.json + safetensors, and tokenizer.json / generation_config.json
    where it has them).

    dtype: None or "bfloat16" keeps the checkpoint's bfloat16; "float32" runs everything
    in true 32-bit. `quantize` exists in the reference's signature; this engine has no
    quantised path and refuses it. The remaining arguments size the engine: tokens per
    cache page, tokens the page pool holds (None: sized from the device memory that is free
    once the weights are placed), live requests, tokens per step."""
    if quantize is not None:
        raise ValueError("quantised weights are not part of this engine")
    if isinstance(dtype, torch.dtype):
        dtype = {v: k for k, v in DTYPES.items()}[dtype]
    folder = Path(model)
    if not (folder / "config.json").exists():
        raise ValueError(f"{folder} is not a model folder (no config.json); hub downloads are not part of this engine")
    engine = Engine.from_folder(folder, EngineArgs(dtype=dtype or "bfloat16", page_size=page_size,
                                                   cache_tokens=cache_tokens, max_requests=max_requests, device=device))
    architecture = engine.architecture
    return LanguageModel(engine, tokenizer=architecture.tokenizer(folder),
                         defaults=architecture.defaults(folder, engine.config), max_tokens_per_step=max_tokens_per_step)

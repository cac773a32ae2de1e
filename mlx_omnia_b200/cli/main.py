"""`omnia run`: one prompt, one answer, on stdout.

The reference's `omnia` is an HTTP client of its daemon
(src/mlx_omnia/cli/main.py:179-207): `omnia run -m MODEL [prompt...] [--max-tokens 512]
[--temperature 1.0]`, the prompt read from stdin when absent (:133-149), stdout carrying
the model's text only (:6-8). This one keeps those names, defaults and meanings but runs
the engine in-process: there is no server here, so `--url`, `chat`, `models` and `status`
have nothing to talk to and are not offered. Added options size or seed the local run.
Sampling options that are not given take the checkpoint's own (generation_config.json), as
the reference's server does (src/mlx_omnia/engine/checkpoint.py:131-152); where the
checkpoint says nothing, the reference's defaults stand (temperature 1.0). `--verbose`
prints the request's numbers (token counts, time to first token, decode rate) on stderr.
"""

from __future__ import annotations

import argparse
import sys
from collections.abc import Sequence


def note(message: str) -> None:
    print(message, file=sys.stderr, flush=True)


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="omnia", description="run a model folder on one B200")
    commands = parser.add_subparsers(dest="command", required=True)
    run = commands.add_parser("run", help="one prompt, one answer, on stdout")
    run.add_argument("-m", "--model", required=True, help="folder with config.json and model.safetensors")
    run.add_argument("prompt", nargs="*", help="the prompt; read from stdin when absent")
    run.add_argument("--max-tokens", type=int, default=512)
    run.add_argument("--temperature", type=float, default=None,
                     help="0 selects greedy decoding (default: the checkpoint's own, else 1.0)")
    run.add_argument("--top-k", type=int, default=None)
    run.add_argument("--top-p", type=float, default=None)
    run.add_argument("--min-p", type=float, default=None)
    run.add_argument("--repetition-penalty", type=float, default=None)
    run.add_argument("--seed", type=int, default=None)
    run.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    run.add_argument("--verbose", action="store_true", help="print the request's numbers on stderr")
    return parser


def _options(args, defaults, meter=None):
    """The generation's options: what the command line says, else what the checkpoint says
    (`defaults`, a text.SamplingDefaults), else temperature 1.0 and every filter off."""
    from mlx_omnia_b200 import sampling

    def pick(given, declared, neutral):
        return given if given is not None else declared if declared is not None else neutral

    temperature = pick(args.temperature, defaults.temperature, 1.0)
    top_k, top_p = pick(args.top_k, defaults.top_k, 0), pick(args.top_p, defaults.top_p, 1.0)
    min_p = pick(args.min_p, defaults.min_p, 0.0)
    repetition = pick(args.repetition_penalty, defaults.repetition_penalty, 1.0)
    if temperature <= 0:
        chosen = sampling.greedy
    else:
        filters = [sampling.temperature(temperature)]
        if top_k:
            filters.append(sampling.top_k(top_k))
        if top_p < 1:
            filters.append(sampling.top_p(top_p))
        if min_p > 0:
            filters.append(sampling.min_p(min_p))
        chosen = sampling.sampler(*filters, seed=args.seed)
    penalty = sampling.repetition_penalty(repetition) if repetition != 1.0 else None
    return sampling.GenerationOptions(max_tokens=args.max_tokens, sampler=chosen, penalty=penalty, meter=meter)


def main(argv: Sequence[str] | None = None) -> int:
    args = _parser().parse_args(argv)
    prompt = " ".join(args.prompt).strip()
    if not prompt and not sys.stdin.isatty():
        prompt = sys.stdin.read().strip()
    if not prompt:
        note("nothing to say: pass a prompt or pipe one in")
        return 2
    try:
        from mlx_omnia_b200 import load
        from mlx_omnia_b200.engine.meter import Meter

        # The pool is sized from the memory that is free once the weights are placed; a prompt
        # that still does not fit beside its answer has the answer cut, and is told so.
        model = load(args.model, dtype=args.dtype, max_requests=1)
        meter = Meter()
        options = _options(args, model.defaults.sampling, meter)
        ids = model._ids(prompt)
        room = model.generator.scheduler.capacity - len(ids)
        if 0 < room < args.max_tokens:
            note(f"omnia: the cache holds {model.generator.scheduler.capacity} tokens; the answer is cut to {room}")
        wrote = ""
        for segment in model.stream(ids, options):
            wrote = segment.text or wrote
            sys.stdout.write(segment.text)
            sys.stdout.flush()
        if args.verbose:
            note(meter.line())
    except KeyboardInterrupt:
        note("^C")
        return 130
    except (ValueError, FileNotFoundError, RuntimeError) as error:
        note(f"omnia: {error}")
        return 1
    if wrote and not wrote.endswith("\n"):
        sys.stdout.write("\n")
    return 0


def run() -> None:
    sys.exit(main())

"""`omnia run`: one prompt, one answer, on stdout.

The reference's `omnia` is an HTTP client of its daemon
(src/mlx_omnia/cli/main.py:179-207): `omnia run -m MODEL [prompt...] [--max-tokens 512]
[--temperature 1.0]`, the prompt read from stdin when absent (:133-149), stdout carrying
the model's text only (:6-8). This one keeps those names, defaults and meanings but runs
the engine in-process: there is no server here, so `--url`, `chat`, `models` and `status`
have nothing to talk to and are not offered. Added options size or seed the local run.
"""

from __future__ import annotations

import argparse
import sys
from collections.abc import Sequence


def note(message: str) -> None:
    print(message, file=sys.stderr, flush=True)


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="omnia", description="run a Muse-Glimmer model folder on one B200")
    commands = parser.add_subparsers(dest="command", required=True)
    run = commands.add_parser("run", help="one prompt, one answer, on stdout")
    run.add_argument("-m", "--model", required=True, help="folder with config.json and model.safetensors")
    run.add_argument("prompt", nargs="*", help="the prompt; read from stdin when absent")
    run.add_argument("--max-tokens", type=int, default=512)
    run.add_argument("--temperature", type=float, default=1.0, help="0 selects greedy decoding")
    run.add_argument("--top-k", type=int, default=0)
    run.add_argument("--top-p", type=float, default=1.0)
    run.add_argument("--min-p", type=float, default=0.0)
    run.add_argument("--repetition-penalty", type=float, default=1.0)
    run.add_argument("--seed", type=int, default=None)
    run.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    return parser


def _options(args):
    from mlx_omnia_b200 import sampling

    if args.temperature <= 0:
        chosen = sampling.greedy
    else:
        filters = [sampling.temperature(args.temperature)]
        if args.top_k:
            filters.append(sampling.top_k(args.top_k))
        if args.top_p < 1:
            filters.append(sampling.top_p(args.top_p))
        if args.min_p > 0:
            filters.append(sampling.min_p(args.min_p))
        chosen = sampling.sampler(*filters, seed=args.seed)
    penalty = sampling.repetition_penalty(args.repetition_penalty) if args.repetition_penalty != 1.0 else None
    return sampling.GenerationOptions(max_tokens=args.max_tokens, sampler=chosen, penalty=penalty)


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

        options = _options(args)
        model = load(args.model, dtype=args.dtype, cache_tokens=max(4096, 2 * args.max_tokens))
        wrote = ""
        for segment in model.stream(prompt, options):
            wrote = segment.text
            sys.stdout.write(segment.text)
            sys.stdout.flush()
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

"""Trace replay: feed given token ids through the model step by step, write logits.

It samples nothing and owns no forward pass, cache or loader: it drives the same
`Engine` (model, step function, cache manager, kernels) that generation uses.

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` are one batch; `want` are the places among an entry's tokens whose logits
are written; `end` lists requests that finish after the step. For a step that wants
something, `<out>/<step>.f32` holds the logits as little-endian float32
[wanted, vocab] in the order of the entries and of `want`. After each step the line
`done <step>` is printed and flushed. With `--npy`, a request's wanted logits are also
gathered in the order they were produced and written as `<out>/logits_<id>.npy`
[wanted positions, vocab] float32 when the request ends (or the input does).
"""

from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import IO


from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry
from mlx_omnia_b200.kernels import ops

TOKEN_ROUNDING = 64


def poison_free_pages(engine: Engine, value: float = float("nan")) -> None:
    """Fill every cache page that no request holds with `value`: a step that reads a page it
    was not given then shows it in its logits. (A debugging aid of the replay program.)"""
    for group in engine.cache.groups:
        free = [page for page in range(group.pool.count) if page not in set(group.pool.held())]
        if free and group.pages is not None:
            group.pages[:, free] = value


def replay(engine: Engine, lines: IO[str], out_dir: Path, done: IO[str] = sys.stdout, before_step=None,
           npy: bool = False) -> int:
    """Run every step read from `lines`; returns how many steps ran. `before_step(engine,
    record)`, when given, runs ahead of each step; `npy` also writes one .npy per request."""
    import numpy as np

    out_dir.mkdir(parents=True, exist_ok=True)
    count = 0
    gathered: dict[str, list] = {}

    def write_request(request_id: str) -> None:
        rows = gathered.pop(request_id, None)
        if rows:
            np.save(out_dir / f"logits_{request_id}.npy", np.concatenate(rows).astype("<f4", copy=False))

    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        if before_step is not None:
            before_step(engine, record)
        entries = []
        for item in record.get("entries", []):
            request_id = str(item["id"])
            request = engine.cache.requests.get(request_id) or engine.cache.open(request_id)
            entries.append(StepEntry(request, [int(t) for t in item["tokens"]], [int(w) for w in item.get("want", [])]))
        if entries:
            logits = engine.runner.run(entries)
            if logits.shape[0]:
                host = logits.to("cpu").numpy().astype("<f4", copy=False)
                host.tofile(out_dir / f"{record['step']}.f32")
                if npy:
                    at = 0
                    for item in record["entries"]:
                        wanted = len(item.get("want", []))
                        if wanted:
                            gathered.setdefault(str(item["id"]), []).append(host[at: at + wanted].copy())
                        at += wanted
            ops.raise_on_error(engine.runtime.device)
        for request_id in record.get("end", []):
            engine.cache.close(str(request_id))
            write_request(str(request_id))
        print(f"done {record['step']}", file=done, flush=True)
        count += 1
    for request_id in list(gathered):
        write_request(request_id)
    return count


def main(argv: list[str] | None = None) -> int:
    import argparse

    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--out", required=True, help="folder the logits are written to")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time, each request rounded up to 64")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    parser.add_argument("--max-requests", type=int, default=4, help="requests that may be live at a time")
    parser.add_argument("--npy", action="store_true",
                        help="also write each request's wanted logits as logits_<id>.npy when it ends")
    parser.add_argument("--poison-free-pages", action="store_true",
                        help="before every step fill the cache pages that no request holds with NaN")
    args = parser.parse_args(argv)
    if TOKEN_ROUNDING % args.page_size:
        parser.error("--page-size must divide 64")
    print(f"[trace_run] loading {args.model} in {args.dtype}", file=sys.stderr, flush=True)
    engine = Engine.from_folder(args.model, EngineArgs(dtype=args.dtype, page_size=args.page_size,
                                                       cache_tokens=max(args.max_tokens, TOKEN_ROUNDING),
                                                       max_requests=args.max_requests))
    replay(engine, sys.stdin, Path(args.out), npy=args.npy,
           before_step=(lambda e, record: poison_free_pages(e)) if args.poison_free_pages else None)
    return 0

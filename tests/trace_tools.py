"""Helpers for the replay tests: write a tiny model folder, build traces, run
`bin/trace_run` as a user would, and gather the logits it wrote per request."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch
from safetensors.torch import save_file

import tiny_configs

ROOT = Path(__file__).resolve().parent.parent


def write_folder(folder: Path, name: str, **kwargs) -> tuple[dict, dict]:
    """A model folder for tiny configuration `name`; matrices stored as bfloat16."""
    raw, weights = tiny_configs.config(name), tiny_configs.tensors(name, **kwargs)
    folder.mkdir(parents=True, exist_ok=True)
    save_file({k: (t if t.dim() < 2 else t.to(torch.bfloat16)).contiguous() for k, t in weights.items()},
              str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(raw))
    return raw, weights


class Trace:
    """Steps of a replay, with the bookkeeping to find each request's logits again."""

    def __init__(self) -> None:
        self.steps: list[dict] = []
        self.where: list[list[tuple[str, int]]] = []  # per step: (request, position) of each wanted row
        self.held: dict[str, int] = {}
        self.peak = 0

    def step(self, portions: dict[str, list[int]], end: list[str] = (), want: str = "all") -> None:
        entries, rows = [], []
        for rid, tokens in portions.items():
            start = self.held.get(rid, 0)
            wanted = list(range(len(tokens))) if want == "all" else [len(tokens) - 1] if want == "last" else []
            entries.append({"id": rid, "tokens": tokens, "want": wanted})
            rows += [(rid, start + w) for w in wanted]
            self.held[rid] = start + len(tokens)
        self.peak = max(self.peak, sum(-(-n // 64) * 64 for n in self.held.values()))
        self.steps.append({"step": len(self.steps), "entries": entries, "end": list(end)})
        self.where.append(rows)
        for rid in end:
            del self.held[rid]

    def text(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)

    def run(self, model: Path, dtype: str, out: Path, max_tokens: int | None = None, extra: list[str] = ()) -> dict:
        """Replay through bin/trace_run; returns {request: {position: logits}}."""
        command = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype,
                   "--out", str(out), "--max-tokens", str(max_tokens or self.peak), *extra]
        done = subprocess.run(command, input=self.text(), capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-4000:]
        assert done.stdout.split() == [w for s in self.steps for w in ("done", str(s["step"]))], done.stdout[-2000:]
        vocab = json.loads((model / "config.json").read_text())["text_config"]["vocab_size"]
        return self.gather(out, vocab)

    def run_engine(self, engine, out: Path, before_step=None) -> dict:
        """Replay in this process through the package's own replay loop over `engine` (what
        bin/trace_run does after loading); `before_step(engine, record)` runs ahead of every step."""
        import io

        from mlx_omnia_b200.engine.trace import replay

        replay(engine, io.StringIO(self.text()), out, done=io.StringIO(), before_step=before_step)
        return self.gather(out, engine.vocab_size)

    def gather(self, out: Path, vocab: int) -> dict:
        got: dict[str, dict[int, torch.Tensor]] = {}
        for index, rows in enumerate(self.where):
            if not rows:
                assert not (out / f"{index}.f32").exists()
                continue
            data = np.fromfile(out / f"{index}.f32", dtype="<f4").reshape(len(rows), vocab)
            for row, (rid, position) in enumerate(rows):
                got.setdefault(rid, {})[position] = torch.from_numpy(data[row].copy())
        return got


def stacked(per_position: dict[int, torch.Tensor]) -> tuple[list[int], torch.Tensor]:
    positions = sorted(per_position)
    return positions, torch.stack([per_position[p] for p in positions])

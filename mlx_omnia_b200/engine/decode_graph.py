"""Decode steps as replayed CUDA graphs.

A step in which every request brings one token launches some three hundred small
kernels; issued one by one from Python they cost more host time than the GPU needs to
run them. Such steps are therefore captured once per *bucket* (requests rounded up to
a power of two, block-table width rounded up to three significant bits) and replayed: the
host writes the step's metadata into one pinned buffer, one copy brings it to the
device buffer the captured kernels read, and the graph runs. Rows beyond the live
requests are padding: sequence length 0, slot -1, position -1, which every kernel
treats as "nothing to do".

The kernels and the model code are the same as in an uncaptured step; only the way
they are launched differs, so logits agree bit for bit with an eager step of the same
bucket. Capture is used only when every mixer of the model declares `graph_safe`
(no host-side loops over requests).

The reference compiles its one-token forward per (mode, batch, capacity) with
mx.compile and pads decode rows to buckets 1/2/4/8
(src/mlx_omnia/engine/core/decode.py:202-317, src/mlx_omnia/engine/batching.py:54,158-220);
CUDA graphs are this engine's counterpart.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import StepContext


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


@dataclass
class _Captured:
    graph: torch.cuda.CUDAGraph
    step: StepContext
    host: np.ndarray  # pinned int32 mirror of `device`
    host_tensor: torch.Tensor
    device: torch.Tensor
    fields: dict[str, tuple[int, int]]  # name -> (offset, length) in int32 units
    logits: torch.Tensor
    batch: int
    width: int
    launches: int = 0  # this package's kernels inside the graph (counted at capture)
    copied: torch.cuda.Event | None = None  # the last host-to-device copy of the metadata


class DecodeGraphs:
    def __init__(self, runner) -> None:
        self.runner = runner
        self.captured: dict[tuple[int, int], _Captured] = {}
        self.replays = 0

    @staticmethod
    def supported(model) -> bool:
        return all(getattr(block.mixer, "graph_safe", False) for block in model.blocks)

    # -- layout of the metadata buffer -------------------------------------------------
    def _layout(self, batch: int, width: int) -> tuple[dict[str, tuple[int, int]], int]:
        fields, at = {}, 0
        for name, length in [("token_ids", batch), ("positions", batch), ("cu_seqlens", batch + 1),
                             ("seq_lens", batch), ("state_slots", batch), ("fresh", batch), ("logit_rows", batch)]:
            fields[name] = (at, length)
            at += length
        for g in range(len(self.runner.cache.groups)):
            fields[f"table{g}"] = (at, batch * width)
            at += batch * width
        at += at % 2  # int64 fields start on 8 bytes
        for g in range(len(self.runner.cache.groups)):
            fields[f"slots{g}"] = (at, 2 * batch)
            at += 2 * batch
        return fields, at

    def _capture(self, batch: int, width: int) -> _Captured:
        runner = self.runner
        device = runner.runtime.device
        fields, total = self._layout(batch, width)
        host_tensor = torch.zeros(total, dtype=torch.int32).pin_memory()
        host = host_tensor.numpy()
        dev = torch.zeros(total, dtype=torch.int32, device=device)

        def view(name: str) -> torch.Tensor:
            offset, length = fields[name]
            return dev[offset: offset + length]

        groups = {}
        for g in range(len(runner.cache.groups)):
            slots = view(f"slots{g}").view(torch.int64)
            groups[g] = (view(f"table{g}").view(batch, width), slots)
        context_bound = width * runner.cache.page_size
        # Kernels that need scratch memory keep it here, for as long as the graph lives.
        workspace = {"private": True}
        step = StepContext(
            num_tokens=batch, num_seqs=batch, token_ids=view("token_ids"), positions=view("positions"),
            cu_seqlens=view("cu_seqlens"), seq_lens=view("seq_lens"), state_slots=view("state_slots"),
            fresh=view("fresh"), logit_rows=view("logit_rows"), q_lens=[1] * batch, seq_lens_host=[], max_q_len=1,
            max_seq_len=context_bound, decode_only=True, groups=groups, workspace=workspace)
        # Padding everywhere, so the warm-up and the capture touch no page.
        self._fill(host, fields, batch, width, [], [])
        dev.copy_(host_tensor)
        layers = runner.layer_contexts(step)
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            runner.model.forward(step, layers)  # warm-up: loads kernels, sizes library workspaces
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        with torch.cuda.graph(graph):
            logits = runner.model.forward(step, layers)
        return _Captured(graph, step, host, host_tensor, dev, fields, logits, batch, width, ops.launches - before)

    def _fill(self, host: np.ndarray, fields, batch: int, width: int, entries, starts) -> None:
        cache = self.runner.cache
        n = len(entries)

        def put(name: str, values, pad: int) -> None:
            offset, length = fields[name]
            host[offset: offset + length] = pad
            if len(values):
                host[offset: offset + len(values)] = values

        put("token_ids", [e.tokens[0] for e in entries], 0)
        put("positions", starts, -1)
        offset, length = fields["cu_seqlens"]
        host[offset: offset + length] = np.arange(length, dtype=np.int32)
        put("seq_lens", [s + 1 for s in starts], 0)
        put("state_slots", [e.request.slot for e in entries], 0)
        put("fresh", [int(e.request.fresh) for e in entries], 0)
        offset, length = fields["logit_rows"]
        host[offset: offset + length] = np.arange(length, dtype=np.int32)
        page = cache.page_size
        for g in range(len(cache.groups)):
            offset, length = fields[f"table{g}"]
            table = host[offset: offset + length].reshape(batch, width)
            table[:] = -1
            slots = np.full(batch, -1, dtype=np.int64)
            for i, (e, start) in enumerate(zip(entries, starts)):
                pages = e.request.table_array(g)
                table[i, : len(pages)] = pages
                slots[i] = int(pages[start // page]) * page + start % page
            offset, length = fields[f"slots{g}"]
            host[offset: offset + length].view(np.int64)[:] = slots

    # -- one step ----------------------------------------------------------------------
    def run(self, entries, copy: bool = True, device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Run a step whose entries all bring one token. -> logits [wanted, vocab].
        With `copy` False the result is the graph's own buffer, valid until the next step.
        `device_tokens` (int32 [entries], on the device) replace the entries' token ids."""
        runner, cache = self.runner, self.runner.cache
        starts = [e.request.tokens for e in entries]
        grown = []
        try:
            for e in entries:
                cache.grow(e.request, 1)
                grown.append(e.request)
        except Exception:
            for request in grown:
                runner._shrink(request, 1)
            raise
        batch = _bucket(len(entries))
        width = ops.width_bucket(max(max(len(t) for t in e.request.tables) for e in entries))
        key = (batch, width)
        captured = self.captured.get(key)
        if captured is None:
            captured = self.captured[key] = self._capture(batch, width)
        if captured.copied is not None:
            captured.copied.synchronize()  # the pinned buffer is free to be written again
        self._fill(captured.host, captured.fields, batch, width, entries, starts)
        captured.device.copy_(captured.host_tensor, non_blocking=True)
        if device_tokens is not None:
            captured.step.token_ids[: len(entries)].copy_(device_tokens[: len(entries)])
        if captured.copied is None:
            captured.copied = torch.cuda.Event()
        captured.copied.record()
        captured.graph.replay()
        self.replays += 1
        ops.launches += captured.launches  # the replay launches what the capture recorded
        wanted = [i for i, e in enumerate(entries) if e.want]
        if len(wanted) == len(entries):
            logits = captured.logits[: len(entries)]
        elif wanted:
            return captured.logits[torch.as_tensor(wanted, device=captured.logits.device)]
        else:
            return captured.logits[:0]
        # The graph owns its output buffer; the next replay overwrites it.
        return logits.clone() if copy else logits

"""Decode steps as replayed CUDA graphs.

A step in which every request brings one token launches some three hundred small
kernels; issued one by one from Python they cost more host time than the GPU needs to
run them. Such steps are therefore captured once per *bucket* (requests rounded up to
a power of two, block-table width rounded up to three significant bits) and replayed: the
host writes the step's metadata into one pinned buffer, one copy brings it to the
device buffer the captured kernels read, and the graph runs. Rows beyond the live
requests are padding: sequence length 0, cache slot -1, position -1, which every kernel
treats as "nothing to do", and the scratch state slot, which belongs to no request (so
a mixer with state of its own may read and write it freely). The metadata is laid out
and filled by the same `StepLayout` as an uncaptured step's.

At most `MAX_GRAPHS` captured graphs are kept; the one replayed longest ago is dropped
for a new bucket (each holds its own logits, activations and scratch buffers).

Mixed steps (`MixedGraphs`). A step of a few hundred tokens, portions of prompts beside
decoded tokens, launches some 230 kernels one by one from Python and is bound by the host
(16 us a launch) long before the GPU. In continuous batching such steps repeat in shape:
the same requests decode while a long prompt is read in portions of the token budget. So
a step whose shape (tokens per request, wanted rows per request, the bucket of the
longest decoding request, the width of the block tables: the next power of two above the
longest request's pages, so a prompt doubles before it leaves its graph; whether its
prompts all start at their first token, which kernels are chosen by) comes for the
third time is captured with exactly that shape, and replayed whenever it comes again. The
small lists that the attention kernels read (which block of query tokens runs where) are
given a place on the device before the capture and filled by the host before every replay
(`ops.fill_step_lists`). The capturing step runs uncaptured on the buffers the graph will
use (so every scratch buffer and list exists before the capture), and the capture that
follows runs nothing, so a mixer's state is never stepped twice; from its fourth coming on
the shape is replayed. (A capture costs about three steps' time. In a stream of 64 requests
of many lengths most shapes come once or twice: capturing at the second coming, with tables
as wide as the pool, made such a stream twice as slow as launching every step kernel by
kernel.)

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

import contextlib
import gc
from dataclasses import dataclass

import numpy as np
import torch

from mlx_omnia_b200.engine.step import StepLayout
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import StepContext

MAX_GRAPHS = 24


@contextlib.contextmanager
def capturing(graph: torch.cuda.CUDAGraph, **options):
    """`torch.cuda.graph` with the garbage collector out of the way. An object that owns a captured
    graph or CUDA memory and is kept alive by reference cycles only (an engine dropped a while ago)
    is freed whenever the collector next runs; if that is in the middle of a capture, freeing it is
    an operation the capturing stream does not permit, and the capture is lost. So what is dead is
    collected before the capture and nothing is collected during it."""
    gc.collect()
    enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, **options):
            yield
    finally:
        if enabled:
            gc.enable()


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


@dataclass
class _Captured:
    graph: torch.cuda.CUDAGraph
    step: StepContext
    layout: StepLayout
    host_tensor: torch.Tensor  # pinned int32 mirror of `device`
    device: torch.Tensor
    logits: torch.Tensor
    launches: int = 0  # this package's kernels inside the graph (counted at capture)
    copied: torch.cuda.Event | None = None  # the last host-to-device copy of the metadata


class DecodeGraphs:
    def __init__(self, runner) -> None:
        self.runner = runner
        self.captured: dict[tuple[int, int], _Captured] = {}  # in order of last use, oldest first
        self.replays = 0

    @staticmethod
    def supported(model) -> bool:
        return all(getattr(block.mixer, "graph_safe", False) for block in model.blocks)

    def _capture(self, batch: int, width: int) -> _Captured:
        runner = self.runner
        device = runner.runtime.device
        layout = StepLayout(batch, batch, batch, [width] * len(runner.cache.groups))
        host_tensor = torch.zeros(layout.words, dtype=torch.int32).pin_memory()
        dev = torch.zeros(layout.words, dtype=torch.int32, device=device)
        # Kernels that need scratch memory keep it in the workspace, for as long as the graph lives.
        step = layout.context(dev, q_lens=[1] * batch, seq_lens_host=[], max_q_len=1,
                              max_seq_len=width * runner.cache.page_size, decode_only=True,
                              workspace={"private": True})
        # Padding everywhere, so the warm-up and the capture touch no page.
        layout.fill(host_tensor.numpy(), runner.cache, [], [], np.arange(batch, dtype=np.int32))
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
        with capturing(graph):
            logits = runner.model.forward(step, layers)
        return _Captured(graph, step, layout, host_tensor, dev, logits, ops.launches - before)

    def _graph_for(self, batch: int, width: int) -> _Captured:
        key = (batch, width)
        captured = self.captured.pop(key, None)
        if captured is None:
            while len(self.captured) >= MAX_GRAPHS:
                oldest = next(iter(self.captured))
                torch.cuda.synchronize(self.runner.runtime.device)  # nothing of it is still running
                del self.captured[oldest]
            captured = self._capture(batch, width)
        self.captured[key] = captured  # most recently used last
        return captured

    # -- one step ----------------------------------------------------------------------
    def run(self, entries, copy: bool = True, device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Run a step whose entries all bring one token. -> logits [wanted, vocab].
        With `copy` False the result is the graph's own buffer, valid until the next step.
        `device_tokens` (int32 [entries], on the device) replace the entries' token ids."""
        runner = self.runner
        starts = runner.take_pages(entries)
        batch = _bucket(len(entries))
        width = ops.width_bucket(max(max(len(t) for t in e.request.tables) for e in entries))
        captured = self._graph_for(batch, width)
        if captured.copied is not None:
            captured.copied.synchronize()  # the pinned buffer is free to be written again
        captured.layout.fill(captured.host_tensor.numpy(), runner.cache, entries, starts,
                             np.arange(batch, dtype=np.int32))
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


MIXED_MAX_TOKENS = 4096
"""Steps of more tokens stay uncaptured (a captured step keeps buffers of its own for as long as its
graph lives). Steps of thousands of tokens are bound by the GPU, not by launching them, yet a replayed
graph still runs them faster: a kernel that follows a library product cannot start its preamble early,
and in a graph the gap between the two is shorter (a 2,048-token step: 7.71 -> 7.37 ms)."""
MIXED_MAX_REQUESTS = 16
"""Steps of more requests stay uncaptured: they are bound by the GPU (the decoding requests' attention
alone outlasts the launching of the step), and in a stream of many requests their shapes change
with every request that joins or leaves."""
MIXED_MAX_GRAPHS = 8
MIXED_CAPTURE_AT = 3
"""A shape is captured at this coming: a capture costs about three steps' time, and in a stream of
requests of many lengths most shapes come once or twice."""


class MixedGraphs:
    """Captured steps of mixed shape, keyed by that shape (see the head of the file)."""

    def __init__(self, runner) -> None:
        self.runner = runner
        self.seen: dict[tuple, int] = {}
        self.captured: dict[tuple, _Captured] = {}  # in order of last use, oldest first
        self.replays = 0
        cache = runner.cache
        # No block table is wider than the longest request the pools can hold.
        self.widest = [cache.pages_for(g, cache.capacity_tokens()) for g in range(len(cache.groups))]

    @staticmethod
    def supported(model) -> bool:
        return all(getattr(block.mixer, "graph_safe_mixed", False) for block in model.blocks)

    def key(self, entries) -> tuple | None:
        q_lens = tuple(len(e.tokens) for e in entries)
        if sum(q_lens) > MIXED_MAX_TOKENS or len(q_lens) > MIXED_MAX_REQUESTS or all(q == 1 for q in q_lens):
            return None
        page = self.runner.cache.page_size
        longest = max((e.request.tokens + 1 for e, q in zip(entries, q_lens) if q == 1), default=0)
        # Block tables are as wide as the next power of two above the longest request of the step: a
        # prompt that is read in portions doubles before it leaves its graph, and a step's tables
        # are at most twice what its requests need (tables as wide as the pool cost a step of 64
        # requests 2.4 MB of metadata to fill and to copy).
        pages = max(-(-(e.request.tokens + q) // page) for e, q in zip(entries, q_lens))
        # Whether every prompt of the step starts at its first token: kernels are chosen by it (a step's
        # launches are the captured ones for as long as its key is the same).
        fresh = all(e.request.tokens == 0 for e, q in zip(entries, q_lens) if q > 1)
        return (q_lens, tuple(len(e.want) for e in entries), ops.width_bucket(-(-longest // page)) if longest else 0,
                max(64, 1 << (pages - 1).bit_length()), fresh)

    def wants(self, entries) -> tuple | None:
        """The shape's key if this step should run from a graph: the shape has come before."""
        key = self.key(entries)
        if key is None:
            return None
        if key in self.captured:
            return key
        self.seen[key] = self.seen.get(key, 0) + 1
        if len(self.seen) > 4096:
            self.seen.clear()
        return key if self.seen[key] >= MIXED_CAPTURE_AT else None

    def run(self, key: tuple, entries, copy: bool = True) -> torch.Tensor:
        runner = self.runner
        for entry in entries:
            if any(not 0 <= w < len(entry.tokens) for w in entry.want):
                raise ValueError(f"request {entry.request.request_id!r}: a wanted place lies outside its tokens")
        starts = runner.take_pages(entries)
        at, rows = 0, []
        for e in entries:
            rows += [at + w for w in e.want]
            at += len(e.tokens)
        captured = self.captured.pop(key, None)
        fresh = captured is None
        if fresh:
            while len(self.captured) >= MIXED_MAX_GRAPHS:
                torch.cuda.synchronize(runner.runtime.device)
                del self.captured[next(iter(self.captured))]
            layout = StepLayout(at, len(entries), len(rows), [min(key[3], widest) for widest in self.widest])
            host_tensor = torch.zeros(layout.words, dtype=torch.int32).pin_memory()
            dev = torch.zeros(layout.words, dtype=torch.int32, device=runner.runtime.device)
        else:
            layout, host_tensor, dev = captured.layout, captured.host_tensor, captured.device
            if captured.copied is not None:
                captured.copied.synchronize()  # the pinned buffers are free to be written again
        q_lens, held = layout.fill(host_tensor.numpy(), runner.cache, entries, starts, rows)
        dev.copy_(host_tensor, non_blocking=True)
        if fresh:
            # This step runs kernel by kernel on the graph's buffers; then the same launches are captured.
            step = layout.context(dev, q_lens=q_lens, seq_lens_host=held, max_q_len=max(q_lens), max_seq_len=max(held),
                                  decode_only=False, workspace={"private": True})
            layers = runner.layer_contexts(step)
            result = runner.model.forward(step, layers)
            torch.cuda.synchronize(runner.runtime.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launches
            with capturing(graph):
                logits = runner.model.forward(step, layers)
            launches = ops.launches - before
            ops.launches = before  # the capture launched nothing
            self.captured[key] = _Captured(graph, step, layout, host_tensor, dev, logits, launches)
            return result
        captured.step.seq_lens_host, captured.step.max_seq_len = held, max(held)
        self.captured[key] = captured  # most recently used last
        ops.fill_step_lists(captured.step)
        if captured.copied is None:
            captured.copied = torch.cuda.Event()
        captured.copied.record()
        captured.graph.replay()
        self.replays += 1
        ops.launches += captured.launches
        return captured.logits.clone() if copy else captured.logits

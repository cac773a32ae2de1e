"""The step function: one batch of (request, its next tokens) through the model.

A step takes entries `(request, tokens, want)`: the request's next tokens, any number
from one (a decoded token) to a whole prompt, cut anywhere, and the places among them
whose logits are wanted. All entries run as one flattened batch; only these tokens
are computed, everything earlier is read from the cache. It returns float32 logits
`[wanted, vocab]` in the order of the entries and of `want`.

The reference runs either one request's prompt block or a batch of single decode
tokens per forward, never both (src/mlx_omnia/server/runtime/rounds.py:159-202,
src/mlx_omnia/engine/batching.py:283-301,541-576); the mixed flattened batch is this
engine's own design.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from mlx_omnia_b200.cache.manager import CacheManager, RequestCache
from mlx_omnia_b200.parts.base import KVView, LayerContext, Runtime, StepContext
from mlx_omnia_b200.parts.model import DecoderModel


@dataclass
class StepEntry:
    request: RequestCache
    tokens: list[int]
    want: list[int] = field(default_factory=list)  # indices into `tokens`


class StepLayout:
    """Where each field of a step's metadata sits in one buffer of int32 words, so that one
    copy brings all of it to the device. A layout is made for `tokens` rows of the batch,
    `seqs` requests, `wanted` logit rows and a block-table width per group; a step with fewer
    requests than `seqs` pads the rest (each padding request brings one padding token). Both
    the eager step and the captured decode graphs lay their metadata out through this class
    and fill it with `fill`, so they cannot drift apart."""

    def __init__(self, tokens: int, seqs: int, wanted: int, widths: list[int]) -> None:
        self.tokens, self.seqs, self.wanted, self.widths = tokens, seqs, wanted, list(widths)
        self.fields: dict[str, tuple[int, int]] = {}
        at = 0
        # The int64 slot mappings come first, so they start on 8 bytes.
        for name, length in ([(f"slots{g}", 2 * tokens) for g in range(len(widths))] +
                             [("token_ids", tokens), ("positions", tokens), ("cu_seqlens", seqs + 1),
                              ("seq_lens", seqs), ("state_slots", seqs), ("fresh", seqs), ("logit_rows", wanted)] +
                             [(f"table{g}", seqs * w) for g, w in enumerate(widths)]):
            self.fields[name] = (at, length)
            at += length
        self.words = max(at, 1)

    def view(self, buffer, name: str):
        """The field `name` of `buffer` (a numpy array or a tensor of int32 words)."""
        at, length = self.fields[name]
        return buffer[at: at + length]

    def fill(self, host: np.ndarray, cache: CacheManager, entries: list[StepEntry], starts: list[int],
             wanted_rows) -> tuple[list[int], list[int]]:
        """Write the metadata of `entries` (whose requests held `starts[i]` positions before
        this step and have been grown since) into `host`; rows and requests beyond them become
        padding: position -1, sequence length 0, cache slot -1, the scratch state slot, block
        tables of -1. -> (tokens per entry, positions held after the step per entry)"""
        n, page = len(entries), cache.page_size
        q_lens = [len(e.tokens) for e in entries]
        total = sum(q_lens)
        if self.tokens - total != self.seqs - n or n > self.seqs:
            raise ValueError("a padded step brings one padding token per padding request")
        cu = np.arange(self.seqs + 1, dtype=np.int32) + (total - n)
        cu[0] = 0
        cu[1: n + 1] = np.cumsum(q_lens)
        self.view(host, "cu_seqlens")[:] = cu
        ids, positions = self.view(host, "token_ids"), self.view(host, "positions")
        ids[total:], positions[total:] = 0, -1
        for i, (e, s) in enumerate(zip(entries, starts)):
            ids[cu[i]: cu[i + 1]] = e.tokens
            positions[cu[i]: cu[i + 1]] = np.arange(s, s + q_lens[i], dtype=np.int32)
        held = [s + q for s, q in zip(starts, q_lens)]
        for name, values, pad in (("seq_lens", held, 0), ("state_slots", [e.request.slot for e in entries],
                                                           cache.scratch_slot),
                                  ("fresh", [int(e.request.fresh) for e in entries], 0)):
            field_ = self.view(host, name)
            field_[:n], field_[n:] = values, pad
        self.view(host, "logit_rows")[:] = wanted_rows
        for g, group in enumerate(cache.groups):
            table = self.view(host, f"table{g}").reshape(self.seqs, self.widths[g])
            table.fill(-1)
            slots = self.view(host, f"slots{g}").view(np.int64)
            slots[total:] = -1
            stride = group.spec.stride
            for i, e in enumerate(entries):
                t = e.request.table_array(g)
                table[i, : len(t)] = t
                row = positions[cu[i]: cu[i + 1]].astype(np.int64) // stride
                slots[cu[i]: cu[i + 1]] = t[row // page].astype(np.int64) * page + row % page
        return q_lens, held

    def context(self, device: torch.Tensor, **host_side) -> StepContext:
        """The step as the parts see it, its tensors being views of the `device` buffer."""
        groups = {g: (self.view(device, f"table{g}").view(self.seqs, w), self.view(device, f"slots{g}").view(torch.int64))
                  for g, w in enumerate(self.widths)}
        return StepContext(
            num_tokens=self.tokens, num_seqs=self.seqs, token_ids=self.view(device, "token_ids"),
            positions=self.view(device, "positions"), cu_seqlens=self.view(device, "cu_seqlens"),
            seq_lens=self.view(device, "seq_lens"), state_slots=self.view(device, "state_slots"),
            fresh=self.view(device, "fresh"), logit_rows=self.view(device, "logit_rows"), groups=groups, **host_side)


class StepRunner:
    """Owns nothing but the glue: the model, the cache manager and the runtime."""

    def __init__(self, model: DecoderModel, cache: CacheManager, runtime: Runtime, cuda_graphs: bool = False) -> None:
        self.model, self.cache, self.runtime = model, cache, runtime
        self.steps_run = 0
        self.graphs = self.mixed_graphs = None
        if cuda_graphs and runtime.device.type == "cuda":
            from mlx_omnia_b200.engine.decode_graph import DecodeGraphs, MixedGraphs

            if DecodeGraphs.supported(model):
                self.graphs = DecodeGraphs(self)
                if MixedGraphs.supported(model):
                    self.mixed_graphs = MixedGraphs(self)

    # -- metadata ----------------------------------------------------------------------
    def take_pages(self, entries: list[StepEntry]) -> list[int]:
        """Grow every entry's request by its tokens, or none of them (the error is raised
        after what this step took has been given back). -> positions held before the step"""
        starts = [entry.request.tokens for entry in entries]
        grown: list[tuple[RequestCache, int]] = []
        try:
            for entry in entries:
                self.cache.grow(entry.request, len(entry.tokens))
                grown.append((entry.request, len(entry.tokens)))
        except Exception:
            for request, count in grown:
                self._shrink(request, count)
            raise
        return starts

    def build_context(self, entries: list[StepEntry]) -> StepContext:
        """Take the pages the entries' tokens need and lay the batch out."""
        cache = self.cache
        if not entries:
            raise ValueError("a step needs at least one entry")
        for entry in entries:
            if not entry.tokens:
                raise ValueError(f"request {entry.request.request_id!r} brings no tokens to this step")
            if any(not 0 <= w < len(entry.tokens) for w in entry.want):
                raise ValueError(f"request {entry.request.request_id!r}: a wanted place lies outside its tokens")
        starts = self.take_pages(entries)
        at, rows = 0, []
        for e in entries:
            rows += [at + w for w in e.want]
            at += len(e.tokens)
        widths = [max(max(len(e.request.tables[g]) for e in entries), 1) for g in range(len(cache.groups))]
        layout = StepLayout(at, len(entries), len(rows), widths)
        pinned = self.runtime.device.type == "cuda"
        host_tensor = torch.empty(layout.words, dtype=torch.int32, pin_memory=pinned)
        q_lens, held = layout.fill(host_tensor.numpy(), cache, entries, starts, rows)
        device = host_tensor.to(self.runtime.device, non_blocking=True) if pinned else host_tensor
        return layout.context(device, q_lens=q_lens, seq_lens_host=held, max_q_len=max(q_lens),
                              max_seq_len=max(held), decode_only=all(q == 1 for q in q_lens))

    def _shrink(self, request: RequestCache, count: int) -> None:
        """Undo a `grow` of `count` tokens that no kernel has used."""
        request.tokens -= count
        for g, (group, table) in enumerate(zip(self.cache.groups, request.tables)):
            keep = self.cache.pages_for(g, request.tokens)
            while len(table) > keep:
                group.pool.give(table.pop())
                request.arrays[g][len(table)] = -1

    def layer_contexts(self, step: StepContext) -> list[LayerContext]:
        cache = self.cache
        contexts = []
        for entry, need in enumerate(cache.needs):
            kv = None
            if entry in cache.group_of_entry:
                g, _ = cache.group_of_entry[entry]
                table, slots = step.groups[g]
                kv = KVView(cache.entry_pages(entry), table, slots, cache.page_size, cache.groups[g].spec.window,
                            writes=need.reads is None, spec=cache.groups[g].spec)
            contexts.append(LayerContext(step, kv, cache.state.get(entry), entry))
        return contexts

    # -- the step ----------------------------------------------------------------------
    def run(self, entries: list[StepEntry], copy: bool = True, device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """One step. Steps in which every request brings a single token are replayed
        from a captured CUDA graph when graphs are on; `copy=False` then returns the
        graph's own logits buffer, which the next step overwrites. `device_tokens`
        (int32 on the device, one per entry; graph steps only) are the step's tokens when
        the host does not know them yet."""
        fresh_slots = [e.request.slot for e in entries if e.request.fresh]
        if fresh_slots and self.cache.state:
            index = torch.as_tensor(fresh_slots, device=self.runtime.device)
            for entry, state in self.cache.state.items():
                initial = self.cache.initial_state.get(entry)
                if initial is None:
                    state.index_fill_(0, index, 0)
                else:
                    state[index] = initial
        if self.graphs is not None and entries and all(len(e.tokens) == 1 and e.want in ([], [0]) for e in entries):
            logits = self.graphs.run(entries, copy, device_tokens)
        else:
            if device_tokens is not None:
                raise ValueError("tokens that live on the device can only feed a captured single-token step")
            shape = self.mixed_graphs.wants(entries) if self.mixed_graphs is not None and entries else None
            if shape is not None:
                logits = self.mixed_graphs.run(shape, entries, copy)
            else:
                step = self.build_context(entries)
                logits = self.model.forward(step, self.layer_contexts(step))
        for entry in entries:
            entry.request.fresh = False
            self.cache.release_behind_window(entry.request)
        self.steps_run += 1
        return logits

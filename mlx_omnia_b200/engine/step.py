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


class StepRunner:
    """Owns nothing but the glue: the model, the cache manager and the runtime."""

    def __init__(self, model: DecoderModel, cache: CacheManager, runtime: Runtime, cuda_graphs: bool = False) -> None:
        self.model, self.cache, self.runtime = model, cache, runtime
        self.steps_run = 0
        self.graphs = None
        if cuda_graphs and runtime.device.type == "cuda":
            from mlx_omnia_b200.engine.decode_graph import DecodeGraphs

            if DecodeGraphs.supported(model):
                self.graphs = DecodeGraphs(self)

    # -- metadata ----------------------------------------------------------------------
    def build_context(self, entries: list[StepEntry]) -> StepContext:
        """Take the pages the entries' tokens need and lay the batch out."""
        cache, page = self.cache, self.cache.page_size
        if not entries:
            raise ValueError("a step needs at least one entry")
        for entry in entries:
            if not entry.tokens:
                raise ValueError(f"request {entry.request.request_id!r} brings no tokens to this step")
            if any(not 0 <= w < len(entry.tokens) for w in entry.want):
                raise ValueError(f"request {entry.request.request_id!r}: a wanted place lies outside its tokens")
        starts = [entry.request.tokens for entry in entries]
        grown: list[tuple[RequestCache, int]] = []
        try:
            for entry in entries:
                cache.grow(entry.request, len(entry.tokens))
                grown.append((entry.request, len(entry.tokens)))
        except Exception:
            for request, count in grown:  # give back what this step took
                self._shrink(request, count)
            raise
        q_lens = [len(e.tokens) for e in entries]
        total = sum(q_lens)
        n = len(entries)
        cu = np.zeros(n + 1, dtype=np.int32)
        cu[1:] = np.cumsum(q_lens)
        rows = [int(cu[i]) + w for i, e in enumerate(entries) for w in e.want]
        widths = [max(max(len(e.request.tables[g]) for e in entries), 1) for g in range(len(cache.groups))]
        # Everything goes to the device in one copy: the fields are laid out in one pinned buffer of
        # int32 words (the int64 slot mappings first, so they start on 8 bytes).
        fields: dict[str, tuple[int, int]] = {}
        offset = 0
        for name, length in ([(f"slots{g}", 2 * total) for g in range(len(cache.groups))] +
                             [("token_ids", total), ("positions", total), ("cu_seqlens", n + 1), ("seq_lens", n),
                              ("state_slots", n), ("fresh", n), ("logit_rows", len(rows))] +
                             [(f"table{g}", n * widths[g]) for g in range(len(cache.groups))]):
            fields[name] = (offset, length)
            offset += length
        pinned = self.runtime.device.type == "cuda"
        host_tensor = torch.empty(max(offset, 1), dtype=torch.int32, pin_memory=pinned)
        host = host_tensor.numpy()

        def field_of(name: str) -> np.ndarray:
            at, length = fields[name]
            return host[at: at + length]

        positions = field_of("positions")
        for i, (e, s) in enumerate(zip(entries, starts)):
            field_of("token_ids")[cu[i]: cu[i + 1]] = e.tokens
            positions[cu[i]: cu[i + 1]] = np.arange(s, s + q_lens[i], dtype=np.int32)
        field_of("cu_seqlens")[:] = cu
        seq_lens = field_of("seq_lens")
        seq_lens[:] = [e.request.tokens for e in entries]
        field_of("state_slots")[:] = [e.request.slot for e in entries]
        field_of("fresh")[:] = [int(e.request.fresh) for e in entries]
        field_of("logit_rows")[:] = rows
        for g in range(len(cache.groups)):
            table = field_of(f"table{g}").reshape(n, widths[g])
            table.fill(-1)
            slots = field_of(f"slots{g}").view(np.int64)
            for i, e in enumerate(entries):
                t = e.request.table_array(g)
                table[i, : len(t)] = t
                pos = positions[cu[i]: cu[i + 1]].astype(np.int64)
                slots[cu[i]: cu[i + 1]] = t[pos // page].astype(np.int64) * page + pos % page
        device = host_tensor.to(self.runtime.device, non_blocking=True) if pinned else host_tensor

        def on_device(name: str) -> torch.Tensor:
            at, length = fields[name]
            return device[at: at + length]

        groups = {g: (on_device(f"table{g}").view(n, widths[g]), on_device(f"slots{g}").view(torch.int64))
                  for g in range(len(cache.groups))}
        return StepContext(
            num_tokens=total, num_seqs=n,
            token_ids=on_device("token_ids"), positions=on_device("positions"), cu_seqlens=on_device("cu_seqlens"),
            seq_lens=on_device("seq_lens"), state_slots=on_device("state_slots"), fresh=on_device("fresh"),
            logit_rows=on_device("logit_rows"),
            q_lens=q_lens, seq_lens_host=[int(s) for s in seq_lens], max_q_len=max(q_lens),
            max_seq_len=int(seq_lens.max()), decode_only=all(q == 1 for q in q_lens), groups=groups)

    def _shrink(self, request: RequestCache, count: int) -> None:
        """Undo a `grow` of `count` tokens that no kernel has used."""
        page = self.cache.page_size
        request.tokens -= count
        keep = -(-request.tokens // page)
        for g, (group, table) in enumerate(zip(self.cache.groups, request.tables)):
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
                            writes=need.reads is None)
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
            for state in self.cache.state.values():
                state.index_fill_(0, index, 0)
        if self.graphs is not None and entries and all(len(e.tokens) == 1 and e.want in ([], [0]) for e in entries):
            logits = self.graphs.run(entries, copy, device_tokens)
        else:
            if device_tokens is not None:
                raise ValueError("tokens that live on the device can only feed a captured single-token step")
            step = self.build_context(entries)
            logits = self.model.forward(step, self.layer_contexts(step))
        for entry in entries:
            entry.request.fresh = False
            self.cache.release_behind_window(entry.request)
        self.steps_run += 1
        return logits

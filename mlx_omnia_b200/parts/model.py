"""A decoder as data, and the object that runs it.

`ModelSpec` lists the parts (each a `PartSpec`) and the *schedule*: the order in which
layers run. The schedule is a list of entries; an entry names a layer (so a layer may
run twice, each run with a cache of its own) and may name an earlier entry whose cache
it reads instead of owning one. Cache pages and per-request state belong to schedule
entries, not to layers.

`DecoderModel` builds the parts through the registries, knows every tensor it wants by
full name, and runs one step over a flattened batch. It holds no sizes of its own.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import (BLOCKS, EMBEDDINGS, HEADS, NORMS, KVSpec, LayerContext, PartSpec, Runtime,
                                       StateSpec, StepContext, TensorSpec)


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec  # a registered block; its params name the mixer, feed-forward and norms
    prefix: str  # tensor-name prefix of the layer, e.g. "model.layers.3"


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int  # index into ModelSpec.layers
    reads: int | None = None  # index of an earlier schedule entry whose cache this one reads


@dataclass(frozen=True)
class ModelSpec:
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    embedding_prefix: str = "model.embed_tokens"
    final_norm_prefix: str = "model.norm"
    head_prefix: str = "lm_head"

    def __post_init__(self) -> None:
        for e, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {e} names layer {entry.layer} of {len(self.layers)}")
            if entry.reads is not None:
                if not 0 <= entry.reads < e:
                    raise ValueError(f"schedule entry {e} reads entry {entry.reads}, which does not run before it")
                if self.schedule[entry.reads].reads is not None:
                    raise ValueError(f"schedule entry {e} reads entry {entry.reads}, which owns no cache")


@dataclass(frozen=True)
class CacheNeed:
    """What one schedule entry asks of the cache manager."""

    kv: KVSpec | None  # pages it owns (None: none, or it reads another entry's)
    state: StateSpec | None
    reads: int | None
    initial_state: torch.Tensor | None = None  # what a request's state starts as (None: zeros)


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.embedding = EMBEDDINGS.build(spec.embedding)
        self.blocks = [BLOCKS.build(layer.block) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.head = HEADS.build(spec.head)
        self.runtime: Runtime | None = None

    # -- tensors ---------------------------------------------------------------------
    def _named_parts(self):
        yield self.spec.embedding_prefix, self.embedding
        for layer, block in zip(self.spec.layers, self.blocks):
            yield layer.prefix, block
        yield self.spec.final_norm_prefix, self.final_norm
        yield self.spec.head_prefix, self.head

    def tensors(self) -> dict[str, TensorSpec]:
        """Every tensor the model loads, by full name."""
        return {f"{prefix}.{local}": spec for prefix, part in self._named_parts()
                for local, spec in part.tensors().items()}

    def load(self, tensors: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        for prefix, part in self._named_parts():
            dot = prefix + "."
            part.load({k[len(dot):]: v for k, v in tensors.items() if k.startswith(dot)}, runtime)
        if hasattr(self.head, "bind"):
            self.head.bind(self.embedding.weight)

    # -- cache -----------------------------------------------------------------------
    def cache_needs(self) -> list[CacheNeed]:
        needs = []
        for entry in self.spec.schedule:
            mixer = self.blocks[entry.layer].mixer
            kv, state = mixer.kv_spec(), mixer.state_spec()
            if entry.reads is not None:
                owner = self.blocks[self.spec.schedule[entry.reads].layer].mixer.kv_spec()
                if kv != owner:
                    raise ValueError(f"a schedule entry reads a cache of {owner} but its mixer keeps {kv}")
                kv = None
            needs.append(CacheNeed(kv, state, entry.reads, mixer.initial_state() if state is not None else None))
        return needs

    # -- the step --------------------------------------------------------------------
    def forward(self, step: StepContext, layers: list[LayerContext]) -> torch.Tensor:
        """Run this step's tokens through the schedule. -> float32 logits [wanted, vocab]"""
        schedule = self.spec.schedule
        ops.begin_pass(step)
        x = self.embedding.forward(step.token_ids, step.positions)
        h = self.blocks[schedule[0].layer].entry_norm.forward(x)
        for e, entry in enumerate(schedule):
            after = self.blocks[schedule[e + 1].layer] if e + 1 < len(schedule) else None
            following = after.entry_norm if after is not None else self.final_norm
            layers[e].exit_may_pend = after is not None and getattr(after.mixer, "takes_pending", False)
            x, h = self.blocks[entry.layer].forward(x, h, layers[e], following)
        if step.logit_rows.shape[0] == 0:
            return torch.empty(0, self.head.vocab, dtype=torch.float32, device=x.device)
        return self.head.forward(ops.gather_rows(h, step.logit_rows))

"""Decode-only steps of many requests: 17, 32, 64 and 100 requests of unequal lengths, each
bringing one token, replayed from captured graphs and launched kernel by kernel, against the
plain implementation in 32-bit and in bfloat16; on a tiny configuration and at the benchmark's
layer widths (two layers, a short vocabulary). These are the shapes whose products run on the
17-to-128-row kernels and whose block tables are the widest a graph bucket sees."""

from __future__ import annotations

import copy

import pytest
import torch

import tiny_configs
from floors import Oracle
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.registry import resolve_architecture

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["MuseGlimmerForConditionalGeneration"], "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 2048, "intermediate_size": 6144, "num_hidden_layers": 2, "num_attention_heads": 16,
        "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 8192, "rms_norm_eps": 1e-6, "post_norm_eps": 1e-6,
        "sliding_window": 48, "qk_scale_factor": 1.0, "output_multiplier": 1.0, "final_logit_softcapping": 30.0,
        "layer_types": ["full_attention", "sliding_attention"], "layer_rope_theta": [1000000.0, 1000000.0],
        "eos_token_id": [], "tie_word_embeddings": True,
    },
}
DECODED = 3


def wide_tensors():
    architecture = resolve_architecture(WIDE)
    tensors = architecture.random_tensors(architecture.parse(WIDE), 2)
    # Larger than N(0, 0.02), so that the branches weigh as much as the residual stream and the
    # logits reach the bend of the soft cap.
    tensors = {k: (t * (2.0 if "proj" in k else 1.0) if t.dim() == 2 else t) for k, t in tensors.items()}
    tensors["model.language_model.embed_tokens.weight"] *= 20.0
    return {k: (t if t.dim() < 2 else t.bfloat16().float()) for k, t in tensors.items()}


def lengths(count: int, longest: int) -> list[int]:
    g = torch.Generator().manual_seed(count)
    drawn = torch.randint(DECODED + 1, longest, (count,), generator=g).tolist()
    drawn[0], drawn[-1] = longest, DECODED + 1  # the extremes are always there
    return drawn


def decode_logits(raw, weights, prompts, dtype, graphs):
    """Every prompt but its last DECODED tokens in mixed steps of up to 2,048 tokens, then
    DECODED decode-only steps of all requests. -> [DECODED, requests, vocab]"""
    engine = Engine.from_tensors(copy.deepcopy(raw), weights, EngineArgs(
        dtype=dtype, page_size=16, cache_tokens=16 * sum(-(-len(p) // 16) for p in prompts), max_requests=len(prompts),
        cuda_graphs=graphs))
    requests = [engine.cache.open(f"r{i}") for i in range(len(prompts))]
    batch, held = [], 0
    for request, prompt in zip(requests, prompts):
        if held + len(prompt) > 2048 and batch:
            engine.runner.run(batch)
            batch, held = [], 0
        batch.append(StepEntry(request, prompt[:-DECODED], []))
        held += len(prompt)
    engine.runner.run(batch)
    rows = []
    for k in range(DECODED):
        entries = [StepEntry(r, [p[len(p) - DECODED + k]], [0]) for r, p in zip(requests, prompts)]
        rows.append(engine.runner.run(entries))
    assert (engine.runner.graphs is not None and engine.runner.graphs.replays == DECODED) == graphs
    ops.raise_on_error(engine.runtime.device)
    out = torch.stack(rows).cpu()
    del engine
    torch.cuda.empty_cache()
    return out


def check(raw, weights, count, longest, dtype):
    vocab = raw["text_config"]["vocab_size"]
    prompts = [tiny_configs.prompt(n, vocab, 700 + i) for i, n in enumerate(lengths(count, longest))]
    oracle = Oracle(raw, weights, {str(i): p for i, p in enumerate(prompts)},
                    rows=lambda ids: list(range(len(ids) - DECODED, len(ids))))
    eager = decode_logits(raw, weights, prompts, dtype, graphs=False)
    replayed = decode_logits(raw, weights, prompts, dtype, graphs=True)
    # A graph runs the bucket's batch (a power of two), an eager step the real one. Where the two
    # are equal the kernels get the same shapes and the logits agree bit for bit; otherwise a
    # product of 17 rows and one of 32 may add in another order, and both must match the plain
    # implementation.
    if count & (count - 1) == 0:
        assert torch.equal(eager, replayed)
    for name, got in (("eager", eager), ("replayed", replayed)):
        worst = max(oracle.diff(str(i), got[:, i]) for i in range(count))
        assert worst < oracle.tolerance[dtype], (name, worst, oracle.tolerance[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("count", [17, 32, 64, 100])
def test_tiny_decode_batches(count, dtype):
    raw, weights = tiny_configs.config("C"), tiny_configs.tensors("C")
    check(raw, weights, count, 150, dtype)


@pytest.mark.parametrize("count,dtype", [(17, "bfloat16"), (64, "bfloat16"), (100, "bfloat16"), (33, "float32")])
def test_decode_batches_at_the_benchmark_widths(count, dtype):
    check(WIDE, wide_tensors(), count, 120, dtype)

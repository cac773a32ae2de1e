"""The benchmark's layer sizes (hidden 2048, 16/8 heads of 128, intermediate 6144, vocabulary
151936, tied head; two layers only, to keep the test short) through every way of cutting: the
bfloat16 engine, whose steps run on the tcgen05, skinny and decode kernels at their real shapes,
against the engine's own true 32-bit path, and the 32-bit path against the plain implementation.
One query is made to match a key hundreds of positions back, so a fault in a far page shows."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_impl
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.registry import resolve_architecture

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["MuseGlimmerForConditionalGeneration"], "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 2048, "intermediate_size": 6144, "num_hidden_layers": 2, "num_attention_heads": 16,
        "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936, "rms_norm_eps": 1e-6, "post_norm_eps": 1e-6,
        "sliding_window": 600, "qk_scale_factor": 1.0, "output_multiplier": 1.0, "final_logit_softcapping": 30.0,
        "layer_types": ["full_attention", "sliding_attention"], "layer_rope_theta": [1000000.0, 1000000.0],
        "eos_token_id": [], "tie_word_embeddings": True,
    },
}
LENGTH = 1500


@pytest.fixture(scope="module")
def model():
    architecture = resolve_architecture(CONFIG)
    tensors = architecture.random_tensors(architecture.parse(CONFIG), 2)
    # Larger weights than N(0, 0.02), so that the branches weigh as much as the residual stream and
    # the logits reach the bend of the soft cap.
    tensors = {k: (t * (2.0 if "proj" in k else 1.0) if t.dim() == 2 else t) for k, t in tensors.items()}
    tensors["model.language_model.embed_tokens.weight"] *= 20.0
    tensors = {k: (t if t.dim() < 2 else t.bfloat16().float()) for k, t in tensors.items()}
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, 151936, (LENGTH,), generator=g).tolist()
    ids[LENGTH - 40] = ids[700]  # a repeated token: its query finds its own earlier key far back
    return tensors, ids


def run(tensors, ids, dtype, cuts, wanted_from):
    engine = Engine.from_tensors(copy.deepcopy(CONFIG), tensors, EngineArgs(dtype=dtype, page_size=16, cache_tokens=4096,
                                                                             max_requests=4))
    request = engine.cache.open("r")
    rows, at = [], 0
    for n in cuts:
        want = [i for i in range(n) if at + i >= wanted_from]
        logits = engine.runner.run([StepEntry(request, ids[at: at + n], want)])
        rows.append(logits.clone())
        at += n
    assert at == len(ids)
    ops.raise_on_error(engine.runtime.device)
    engine.cache.close("r")
    out = torch.cat(rows).cpu()
    del engine
    torch.cuda.empty_cache()
    return out


def test_every_cut_at_the_benchmark_sizes(model):
    tensors, ids = model
    tail = LENGTH - 64  # compare the logits of the last 64 positions
    whole = [LENGTH]
    chunks = [512, 2, 301, 128, 7, LENGTH - 950 - 32] + [1] * 32
    assert sum(chunks) == LENGTH
    reference = run(tensors, ids, "float32", whole, tail)
    cut32 = run(tensors, ids, "float32", chunks, tail)
    assert plain_impl.relative_diff(cut32, reference) < 1e-4
    worst = {}
    for name, cuts in (("whole", whole), ("chunks", chunks), ("tail", [1000, 500 - 32] + [1] * 32)):
        got = run(tensors, ids, "bfloat16", cuts, tail)
        worst[name] = plain_impl.relative_diff(got, reference)
        assert (got.argmax(-1) == reference.argmax(-1)).float().mean() > 0.9, name
    assert max(worst.values()) < 3e-2, worst


def test_32_bit_path_matches_plain_at_the_benchmark_widths(model):
    tensors, ids = model
    short = ids[:200]
    expect = plain_impl.forward(CONFIG, tensors, short)[-16:]
    got = run(tensors, short, "float32", [150, 34] + [1] * 16, 200 - 16)
    assert plain_impl.relative_diff(got, expect) < 1e-4

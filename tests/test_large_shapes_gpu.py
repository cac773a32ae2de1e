"""The benchmark's layer sizes (hidden 2048, 16/8 heads of 128, intermediate 6144, vocabulary
151936, tied head; two layers only, to keep the test short) through every way of cutting: the
bfloat16 engine, whose steps run on the tcgen05, skinny and decode kernels at their real shapes,
and its true 32-bit path, both against the plain implementation itself (run whole in float64 on
the CPU, the head on the compared rows only). One query is made to match a key hundreds of
positions back, so a fault in a far page shows. Then the head counts and widths of the two
larger benchmark configurations (groups of 4 and 5 query heads, hidden 4096 and 5120; two layers,
a short vocabulary), so that those groupings and the wide residual stream pass every cut too."""

from __future__ import annotations

import copy

import pytest
import torch

from floors import Oracle
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
LENGTH = 1600  # whole, its attention input projection has the norms, the rotation and the cache write in its epilogue


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


def run(config, tensors, ids, dtype, cuts, wanted_from):
    engine = Engine.from_tensors(copy.deepcopy(config), tensors, EngineArgs(dtype=dtype, page_size=16, cache_tokens=4096,
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


TAIL = 64  # the logits of the last 64 positions are compared


def exact_and_tolerances(config, tensors, ids):
    oracle = Oracle(config, tensors, {"r": ids}, rows=lambda all_ids: list(range(len(all_ids) - TAIL, len(all_ids))))
    return oracle


CUTS = {"whole": [LENGTH], "chunks": [512, 2, 301, 128, 7, LENGTH - 950 - 32] + [1] * 32,
        "tail": [1000, LENGTH - 1000 - 32] + [1] * 32}


def test_every_cut_at_the_benchmark_sizes(model):
    tensors, ids = model
    oracle = exact_and_tolerances(CONFIG, tensors, ids)
    worst = {}
    for dtype, names in (("float32", ("whole", "chunks")), ("bfloat16", ("whole", "chunks", "tail"))):
        for name in names:
            assert sum(CUTS[name]) == LENGTH
            got = run(CONFIG, tensors, ids, dtype, CUTS[name], LENGTH - TAIL)
            worst[dtype, name] = oracle.diff("r", got) / oracle.tolerance[dtype]
    assert max(worst.values()) < 1.0, f"in units of the tolerance: {worst}"


def larger(hidden, heads, inner):
    raw = copy.deepcopy(CONFIG)
    raw["text_config"].update(hidden_size=hidden, num_attention_heads=heads, intermediate_size=inner, vocab_size=8192,
                              tie_word_embeddings=False, sliding_window=300)
    return raw


@pytest.mark.parametrize("hidden,heads,inner", [(4096, 32, 12288), (5120, 40, 17408)])
def test_the_larger_configurations_head_counts_and_widths(hidden, heads, inner):
    """Groups of 4 and 5 query heads per key/value head at head size 128, residual streams of
    4,096 and 5,120: whole, in portions, and decoded one by one (the decode path of streams wider
    than 2,048), in bfloat16 against the plain implementation."""
    raw = larger(hidden, heads, inner)
    architecture = resolve_architecture(raw)
    tensors = architecture.random_tensors(architecture.parse(raw), 3)
    tensors = {k: (t * (2.0 if "proj" in k else 1.0) if t.dim() == 2 else t) for k, t in tensors.items()}
    tensors["lm_head.weight"] *= 20.0
    tensors = {k: (t if t.dim() < 2 else t.bfloat16().float()) for k, t in tensors.items()}
    g = torch.Generator().manual_seed(hidden)
    length = 700
    ids = torch.randint(0, 8192, (length,), generator=g).tolist()
    ids[length - 20] = ids[333]
    oracle = exact_and_tolerances(raw, tensors, ids)
    worst = {}
    for name, cuts in (("whole", [length]), ("chunks", [300, 2, 129, 7, length - 438 - 32] + [1] * 32)):
        assert sum(cuts) == length
        got = run(raw, tensors, ids, "bfloat16", cuts, length - TAIL)
        worst[name] = oracle.diff("r", got) / oracle.tolerance["bfloat16"]
    assert max(worst.values()) < 1.0, f"in units of the tolerance: {worst}"

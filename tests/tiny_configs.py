"""Two tiny Muse-Glimmer configurations that differ in every size and option, and the
helpers that draw weights for them. Tests use these, never a real checkpoint."""

from __future__ import annotations

import copy

import torch

TINY_A = {
    "architectures": ["MuseGlimmerForConditionalGeneration"],
    "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 64, "intermediate_size": 192, "num_hidden_layers": 2, "num_attention_heads": 4,
        "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 512, "rms_norm_eps": 1e-6, "post_norm_eps": 1e-6,
        "sliding_window": 8, "qk_scale_factor": 1.0, "output_multiplier": 1.0, "final_logit_softcapping": 30.0,
        "layer_types": ["full_attention", "full_attention"], "layer_rope_theta": [10000.0, 10000.0],
        "rope_parameters": {"rope_theta": 10000.0, "rope_type": "default"}, "eos_token_id": 0,
        "tie_word_embeddings": True,
    },
}

TINY_B = {
    "architectures": ["MuseGlimmerForConditionalGeneration"],
    "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 96, "intermediate_size": 320, "num_hidden_layers": 3, "num_attention_heads": 8,
        "num_key_value_heads": 1, "head_dim": 24, "vocab_size": 1000, "rms_norm_eps": 1e-5, "post_norm_eps": 1e-6,
        "sliding_window": 16, "qk_scale_factor": 1.25, "output_multiplier": 0.5, "final_logit_softcapping": 20.0,
        "layer_types": ["sliding_attention", "full_attention", "sliding_attention"],
        "layer_rope_theta": [1000000.0, 0.0, 1000000.0],
        "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"}, "eos_token_id": [1, 2],
        "tie_word_embeddings": False,
    },
}

# A third shape with 64-wide heads, for the tiled bfloat16 kernels that tiny A and B are too small for.
TINY_C = {
    "architectures": ["MuseGlimmerForConditionalGeneration"],
    "model_type": "muse_glimmer",
    "text_config": {
        "hidden_size": 160, "intermediate_size": 224, "num_hidden_layers": 2, "num_attention_heads": 6,
        "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 777, "rms_norm_eps": 1e-6, "post_norm_eps": 1e-5,
        "sliding_window": 40, "qk_scale_factor": 0.8, "output_multiplier": 2.0, "final_logit_softcapping": 25.0,
        "layer_types": ["full_attention", "sliding_attention"], "layer_rope_theta": [50000.0, 10000.0],
        "eos_token_id": 3, "tie_word_embeddings": False,
    },
}

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 5)}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name][0])


def tensors(name: str, *, head_gain: float = 40.0, stored: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    """Random tensors for a tiny configuration, under the checkpoint's names, as float32
    values that are exactly representable in `stored` (so the 32-bit and the bfloat16
    engine and the plain implementation all see the same numbers). The table that feeds
    the head is scaled by `head_gain` so that logits reach the soft cap's bend."""
    from mlx_omnia_b200.registry import resolve_architecture

    raw, seed = CONFIGS[name]
    architecture = resolve_architecture(raw)
    drawn = architecture.random_tensors(architecture.parse(raw), seed)
    head = "lm_head.weight" if "lm_head.weight" in drawn else "model.language_model.embed_tokens.weight"
    drawn[head] = drawn[head] * head_gain
    return {k: (t if t.dim() < 2 else t.to(stored).float()) for k, t in drawn.items()}


def prompt(length: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()

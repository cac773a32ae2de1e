"""mlx_omnia_b200: a single-GPU (sm_100a) inference engine for the Muse-Glimmer decoder.

    from mlx_omnia_b200 import load, GenerationOptions
    model = load("path/to/folder")
    for segment in model.stream("1 2 3", GenerationOptions(max_tokens=16)):
        print(segment.text, end="")
"""

from mlx_omnia_b200.engine.generate import LanguageModel, Segment, Text, load
from mlx_omnia_b200.parts import (register_block, register_feed_forward, register_mixer, register_norm,
                                  register_position)
from mlx_omnia_b200.registry import register_architecture
from mlx_omnia_b200.sampling import (GenerationOptions, greedy, min_p, repetition_penalty, sampler, temperature, top_k,
                                     top_p)

__version__ = "0.1.0"

__all__ = ["GenerationOptions", "LanguageModel", "Segment", "Text", "greedy", "load", "min_p", "register_architecture",
           "register_block", "register_feed_forward", "register_mixer", "register_norm", "register_position",
           "repetition_penalty", "sampler", "temperature", "top_k", "top_p"]

"""Text in and out: the byte-level BPE a checkpoint's tokenizer.json describes, and what a
checkpoint's side files say about stopping and sampling."""

from mlx_omnia_b200.text.bpe import ByteLevelBPE, Detokenizer
from mlx_omnia_b200.text.defaults import GenerationDefaults, SamplingDefaults, generation_defaults, read_tokenizer

__all__ = ["ByteLevelBPE", "Detokenizer", "GenerationDefaults", "SamplingDefaults", "generation_defaults",
           "read_tokenizer"]

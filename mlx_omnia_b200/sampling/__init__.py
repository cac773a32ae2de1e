"""Sampling: options in the reference's names, and the per-step call of the kernel."""

from mlx_omnia_b200.sampling.options import (GenerationOptions, Penalty, SamplingParams, greedy, min_p,
                                             repetition_penalty, sampler, temperature, top_k, top_p)

__all__ = ["GenerationOptions", "Penalty", "SamplingParams", "greedy", "min_p", "repetition_penalty", "sampler",
           "temperature", "top_k", "top_p"]

"""Sampling: greedy, temperature, top-k and top-p."""

from simply_b200.sampling.params import SamplingParams

__all__ = ["SamplingParams"]

"""Greedy, temperature, race and nucleus sampling on the device."""
from .sampler import SamplingParams, pick

__all__ = ["SamplingParams", "pick"]

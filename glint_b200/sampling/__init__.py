"""Greedy and stochastic token choice."""
from .sampler import SamplingParams, Xorshift64, DeviceSampler

__all__ = ["SamplingParams", "Xorshift64", "DeviceSampler"]

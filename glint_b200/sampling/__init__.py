"""Greedy and stochastic token choice."""
from .sampler import SamplingParams, Xorshift64, DeviceSampler, TokenCounts

__all__ = ["SamplingParams", "Xorshift64", "DeviceSampler", "TokenCounts"]

"""Greedy and temperature / top-k token selection."""

from .sampler import SamplingParams, select

__all__ = ["SamplingParams", "select"]

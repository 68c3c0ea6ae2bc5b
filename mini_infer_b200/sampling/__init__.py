"""Greedy, temperature and nucleus sampling."""

from .params import SamplingParams, philox4x32, uniform

__all__ = ["SamplingParams", "philox4x32", "uniform"]

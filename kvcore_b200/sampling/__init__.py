"""Sampling parameters and the batch sampler."""
from .params import SamplingParams
from .sampler import SAMPLING_EPS, Sampler

__all__ = ["SAMPLING_EPS", "Sampler", "SamplingParams"]

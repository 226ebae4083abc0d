"""Sampling: parameters and the device sampler."""
from .sampler import Sampler, SamplingParams, uniform01

__all__ = ["Sampler", "SamplingParams", "uniform01"]

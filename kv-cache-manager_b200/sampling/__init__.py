"""Sampling: greedy and temperature, on the device."""
from .sampler import Sampler, uniform_for

__all__ = ["Sampler", "uniform_for"]

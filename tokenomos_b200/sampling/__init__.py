"""Sampling: parameters (``SamplingParams``) and the host side of the sampling kernel."""

from tokenomos_b200.sampling.params import SamplingParams

__all__ = ["SamplingParams"]

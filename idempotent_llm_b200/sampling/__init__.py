"""Greedy and temperature sampling."""

from .sampler import mix64, row_key, sample_tokens

__all__ = ["mix64", "row_key", "sample_tokens"]

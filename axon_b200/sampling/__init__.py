"""Greedy and temperature sampling with top-k, top-p, min-p and a repeat penalty."""

from .sampler import DEFAULT_TEMP, FLAGS, RowSampler, SampleArgs, SampleCfg, pick_tokens, random_seed

__all__ = ["DEFAULT_TEMP", "FLAGS", "RowSampler", "SampleArgs", "SampleCfg", "pick_tokens", "random_seed"]

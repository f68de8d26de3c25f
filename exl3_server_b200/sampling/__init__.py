"""Greedy, temperature, top-k / top-p / min-p and penalty sampling."""
from .host import apply_penalties, sample_token
from .options import DEFAULT_SEED, SampleOptions, SplitMix64
from .sampler import RowSampler, sample_rows

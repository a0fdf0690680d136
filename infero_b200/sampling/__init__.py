from .params import SamplingParams
from .sampler import RowSampler, sample_rows

__all__ = ["SamplingParams", "RowSampler", "sample_rows"]

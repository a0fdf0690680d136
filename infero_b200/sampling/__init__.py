from .params import SamplingParams
from .sampler import DeviceFault, PendingTokens, ReadyTokens, RowSampler, sample_rows, sample_rows_async

__all__ = ["SamplingParams", "RowSampler", "sample_rows", "sample_rows_async", "PendingTokens", "ReadyTokens", "DeviceFault"]

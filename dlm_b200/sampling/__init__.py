from .sampler import RequestSampler, SamplingParams, SplitMix64, sample_rows

__all__ = ["RequestSampler", "SamplingParams", "SplitMix64", "sample_rows"]

from .sampler import HISTORY_CAP, Sampler, SamplingParams

__all__ = ["HISTORY_CAP", "Sampler", "SamplingParams"]

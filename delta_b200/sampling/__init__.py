from .sampler import SamplingParams, sample, uniform_of

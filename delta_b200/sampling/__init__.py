from .sampler import SamplingParams, uniform_of

from .sampler import Sampler, SamplingParams, uniform01

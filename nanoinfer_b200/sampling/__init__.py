from .sampler import Sampler, SamplingParams, xorshift64star_state

__all__ = ["Sampler", "SamplingParams", "xorshift64star_state"]

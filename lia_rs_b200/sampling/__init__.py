from .sampler import MT19937, RequestSampler, Sampling, distribution, gumbel_noise, murmur_hash

__all__ = ["MT19937", "RequestSampler", "Sampling", "distribution", "gumbel_noise", "murmur_hash"]

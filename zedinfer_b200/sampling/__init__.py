from .sampler import Sampler, fresh_seed, uniform_for

__all__ = ["Sampler", "fresh_seed", "uniform_for"]

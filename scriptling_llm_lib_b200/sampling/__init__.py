from .sampler import STRATEGIES, Sampler, SamplingOptions, pack_params

__all__ = ["STRATEGIES", "Sampler", "SamplingOptions", "pack_params"]

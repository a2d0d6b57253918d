from .params import SamplingParams
from .sampler import Sampler, derive_seed

__all__ = ["SamplingParams", "Sampler", "derive_seed"]

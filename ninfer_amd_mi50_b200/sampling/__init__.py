from .params import SamplingParams
from .sampler import Sampler, check_params, sample_reference, uniform_draw

__all__ = ["SamplingParams", "Sampler", "check_params", "sample_reference", "uniform_draw"]

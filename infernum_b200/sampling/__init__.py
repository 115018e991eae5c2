from .params import GenerateOptions, SamplingParams
from .sampler import Sampler, recent_window, uniform_for

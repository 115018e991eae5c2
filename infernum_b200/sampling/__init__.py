from .params import GenerateOptions, SamplingParams
from .sampler import Sampler, pack_choices, recent_window, uniform_for

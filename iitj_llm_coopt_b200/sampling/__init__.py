from .params import SamplingParams
from .sampler import Sampler, mix64, row_key

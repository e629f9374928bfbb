from .params import GenParams, GenStats
from .sampler import Sampler

from .rng import uniform
from .sampler import Sampler

from .sampler import Sampler
from . import rng

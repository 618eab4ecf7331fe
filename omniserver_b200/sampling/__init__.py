from .sampler import SampleHandle, Sampler
from . import rng

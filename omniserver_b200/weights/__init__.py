from .loader import WeightsError, load_weights
from .random_init import fill_random, random_state_dict, write_random_model

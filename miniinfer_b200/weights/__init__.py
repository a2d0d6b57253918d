from .loader import WeightLoadError, load_weights
from .random_init import init_random_on_device, random_state_dict, write_random_model

__all__ = ["WeightLoadError", "load_weights", "init_random_on_device", "random_state_dict", "write_random_model"]

from .loader import WeightsError, check_against_specs, collect_tensor_specs, load_tensors, place_tensors
from .random_init import random_tensors, write_random_model

__all__ = [
    "WeightsError", "check_against_specs", "collect_tensor_specs", "load_tensors", "place_tensors",
    "random_tensors", "write_random_model",
]

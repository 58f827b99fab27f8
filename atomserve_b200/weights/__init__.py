from atomserve_b200.weights.loader import WeightsError, load_model, load_tensors_into
from atomserve_b200.weights.random_init import RandomTensors, random_model, write_model_folder

__all__ = [
    "RandomTensors",
    "WeightsError",
    "load_model",
    "load_tensors_into",
    "random_model",
    "write_model_folder",
]

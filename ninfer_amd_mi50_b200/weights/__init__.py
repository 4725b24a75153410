from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .loader import (CheckpointSource, RandomSource, WeightError, check_specs, held_dtype,
                     load_model)
from .random_init import write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "write_safetensors", "CheckpointSource",
           "RandomSource", "WeightError", "check_specs", "held_dtype", "load_model",
           "write_random_model"]

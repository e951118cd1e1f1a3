from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401
from .store import SafetensorsStore, TensorDictStore, WeightError, WeightStore  # noqa: F401
from .random_init import RandomStore, random_tensors, write_random_model  # noqa: F401

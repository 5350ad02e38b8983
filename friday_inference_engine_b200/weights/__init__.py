from .loader import WeightsError, check_names, load_weights, storage_dtype  # noqa: F401
from .random_init import RandomSource, expected_params, write_model_dir  # noqa: F401
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401

from .plan import SourceTensor, WeightBinding
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors
from .loader import WeightError, kept_dtype, load_weights, read_config_json

__all__ = ["SourceTensor", "WeightBinding", "Checkpoint", "SafetensorsError", "SafetensorsFile",
           "write_safetensors", "WeightError", "kept_dtype", "load_weights", "read_config_json"]

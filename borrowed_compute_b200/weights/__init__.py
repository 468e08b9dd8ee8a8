from .loader import check_tensors, load_tensors, read_config_json, read_generation_stop_ids
from .random_init import random_tensor, random_tensors, write_model_folder
from .safetensors_io import SafetensorsFile, TensorSource, write_safetensors

__all__ = ["check_tensors", "load_tensors", "read_config_json", "read_generation_stop_ids", "random_tensor", "random_tensors", "write_model_folder",
           "SafetensorsFile", "TensorSource", "write_safetensors"]

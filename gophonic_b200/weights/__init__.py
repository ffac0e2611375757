from .declare import declare_model
from .loader import WeightsError, load_tensors
from .random_init import InitScales, random_tensors_on_device, write_random_model
from .safetensors_io import Checkpoint, CheckpointError, write_safetensors

__all__ = ["Checkpoint", "CheckpointError", "InitScales", "WeightsError", "declare_model", "load_tensors",
           "random_tensors_on_device", "write_random_model", "write_safetensors"]

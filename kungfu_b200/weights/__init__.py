from .safetensors_io import SafetensorsFile, TensorInfo, WeightFileError, open_model_tensors, write_safetensors
from .store import TensorSpec, WeightError, WeightStore, random_tensor
from .random_init import write_random_model

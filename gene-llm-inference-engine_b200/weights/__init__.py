from .loader import WeightsError, load_model_folder, read_config, read_tensors
from .plan import TensorRule, WeightPlan, llama_weight_plan
from .random_init import write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, ShardedSafetensors, write_safetensors

__all__ = ["WeightsError", "load_model_folder", "read_config", "read_tensors", "TensorRule", "WeightPlan",
           "llama_weight_plan", "write_random_model", "SafetensorsError", "SafetensorsFile", "ShardedSafetensors", "write_safetensors"]

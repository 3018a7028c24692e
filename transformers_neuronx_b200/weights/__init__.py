from .loader import TensorSpec, WeightError, load_tensors, match_tensors
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsFile, save_safetensors
from .model_files import open_model_files, SplitTensorFolder, StateDictFile

from .loader import (DictSource, FolderSource, TensorSource, WeightError, check_against, load_into,
                     stored_precision)
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, checkpoint_files, write_safetensors

from .loader import ExpectedTensor, WeightsError, check_names_and_shapes, kept_dtype, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import CheckpointFormatError, SafetensorsFile, open_checkpoint, write_safetensors

from .loader import WeightError, checkpoint_index, expected_tensors, load_parameters
from .random_init import random_checkpoint, random_parameters, write_model_dir
